// Linear layer for very small batches (M <= 8): out[m,n] = bias[n] + sum_k term(x[m,k], w[n,k]).
//
// With so few rows every packed weight is used M times and then never again: the layer is bound by
// reading the packed weights once (HBM, or L2 when the layer was used a moment ago) and by launch
// latency.  Layout of the work (shift.cu:57-120 gives one thread per output and walks K serially):
//
//   * a warp owns CN neighbouring output columns and all M rows; its 32 lanes split K: lane l takes
//     packed words l, l+32, ... of each of its rows (one coalesced 128-byte request per row and
//     step; 16- or 8-byte requests per lane when rows are whole groups of four or two words, and
//     16- or 8-byte requests on x when a word's weights are), decodes each word's
//     fields once through a small lookup table in shared memory, and applies every weight to the M
//     activations it meets (exact integer arithmetic: shift, then multiply by +-1 / +-2^k / 0);
//   * when the columns alone do not fill the GPU, WPC warps of a CTA share a column group and split
//     K between them as well;
//   * the partial sums meet in a warp-shuffle tree (and, across the WPC warps, in shared memory);
//     one lane per output then applies the epilogue.  No atomics, no second pass: fused
//     epilogues work for every shape.
#include "ds_gemm_common.cuh"

namespace ds {
namespace {

constexpr int SM_WARPS = 8;
constexpr int SM_THREADS = SM_WARPS * 32;

template <int MR, int CN, int INK>
__global__ void __launch_bounds__(SM_THREADS) small_linear_kernel(const GemmParams p, int wpc, int vecw)
{
    __shared__ int2 lut[256];                       // (right shift, multiplier) per field value
    __shared__ int part[SM_WARPS][MR * CN];         // partial sums of the warps that share a column group
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    if (p.gate && *p.gate != p.gate_want) return;
    for (int f = t; f < (1 << p.dec.fw); f += SM_THREADS) {
        int shv, mul;
        decode_int(uint32_t(f), p.dec, true, shv, mul);
        lut[f] = make_int2(shv, mul);
    }
    __syncthreads();

    const int groups_per_cta = SM_WARPS / wpc;
    const int group = blockIdx.x * groups_per_cta + warp / wpc;  // column group of this warp
    const int ksplit = warp % wpc;                               // its share of K within the group
    const int n0 = group * CN;
    const int m0 = blockIdx.y * MR;
    const uint32_t fmask = (1u << p.dec.fw) - 1u;
    const int num = p.dec.num, fw = p.dec.fw;
    int acc[MR][CN];
#pragma unroll
    for (int m = 0; m < MR; ++m)
#pragma unroll
        for (int c = 0; c < CN; ++c) acc[m][c] = 0;

    const int32_t* xi = static_cast<const int32_t*>(p.x);
    // one packed word of every column against the activations it meets
    const bool vecx = (num == 4) && (p.K % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.x) & 15u) == 0);
    const bool pairx = !vecx && (num % 2 == 0) && (p.K % 2 == 0) && ((reinterpret_cast<uintptr_t>(p.x) & 7u) == 0);
    auto word_step = [&](int w, const uint32_t (&word)[CN]) {
        const int k0 = w * num;
        if (vecx) {
            // four weights per word and rows of whole 16-byte groups: one 16-byte load per row
            int xv[MR][4];
#pragma unroll
            for (int m = 0; m < MR; ++m) {
                int4 r = make_int4(0, 0, 0, 0);
                if (m0 + m < p.M && DS_X_OK(p, xi + (size_t)(m0 + m) * p.K + k0, 16))
                    r = __ldg(reinterpret_cast<const int4*>(xi + (size_t)(m0 + m) * p.K + k0));
                xv[m][0] = __float_as_int(operand_of<false, INK>(p, r.x));
                xv[m][1] = __float_as_int(operand_of<false, INK>(p, r.y));
                xv[m][2] = __float_as_int(operand_of<false, INK>(p, r.z));
                xv[m][3] = __float_as_int(operand_of<false, INK>(p, r.w));
                if (m0 + m >= p.M) xv[m][0] = xv[m][1] = xv[m][2] = xv[m][3] = 0;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int c = 0; c < CN; ++c) {
                    const int2 d = lut[(word[c] >> (j * fw)) & fmask];
#pragma unroll
                    for (int m = 0; m < MR; ++m) acc[m][c] += (xv[m][j] >> d.x) * d.y;
                }
            return;
        }
        if (pairx) {
            // an even number of weights per word and rows of whole 8-byte groups: x in pairs
            for (int j = 0; j < num; j += 2) {
                const int k = k0 + j;
                if (k >= p.K) break;  // K is even: k + 1 < K as well
                int xv[MR][2];
#pragma unroll
                for (int m = 0; m < MR; ++m) {
                    int2 r = make_int2(0, 0);
                    if (m0 + m < p.M && DS_X_OK(p, xi + (size_t)(m0 + m) * p.K + k, 8))
                        r = __ldg(reinterpret_cast<const int2*>(xi + (size_t)(m0 + m) * p.K + k));
                    xv[m][0] = __float_as_int(operand_of<false, INK>(p, r.x));
                    xv[m][1] = __float_as_int(operand_of<false, INK>(p, r.y));
                    if (m0 + m >= p.M) xv[m][0] = xv[m][1] = 0;
                }
#pragma unroll
                for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                    for (int c = 0; c < CN; ++c) {
                        const int2 d = lut[(word[c] >> ((j + jj) * fw)) & fmask];
#pragma unroll
                        for (int m = 0; m < MR; ++m) acc[m][c] += (xv[m][jj] >> d.x) * d.y;
                    }
            }
            return;
        }
        for (int j = 0; j < num; ++j) {
            const int k = k0 + j;
            if (k >= p.K) break;
            int xv[MR];
#pragma unroll
            for (int m = 0; m < MR; ++m) {
                xv[m] = 0;
                if (m0 + m < p.M && DS_X_OK(p, xi + (size_t)(m0 + m) * p.K + k, 4))
                    xv[m] = __float_as_int(operand_of<false, INK>(p, __ldg(xi + (size_t)(m0 + m) * p.K + k)));
            }
#pragma unroll
            for (int c = 0; c < CN; ++c) {
                const int2 d = lut[(word[c] >> (j * fw)) & fmask];
#pragma unroll
                for (int m = 0; m < MR; ++m) acc[m][c] += (xv[m] >> d.x) * d.y;
            }
        }
    };

    if (n0 < p.N) {
        const int lanes = 32 * wpc, me = ksplit * 32 + lane;
        if (vecw == 2) {
            // rows are whole 8-byte groups: two words per lane and request
            const int row2 = p.dec.row_len >> 1;
            for (int q = me; q < row2; q += lanes) {
                uint2 wq[CN];
#pragma unroll
                for (int c = 0; c < CN; ++c) {
                    wq[c] = make_uint2(0, 0);
                    if (n0 + c < p.N && DS_W_OK(p, reinterpret_cast<const uint2*>(p.packed + (size_t)(n0 + c) * p.dec.row_len) + q, 8))
                        wq[c] = __ldg(reinterpret_cast<const uint2*>(p.packed + (size_t)(n0 + c) * p.dec.row_len) + q);
                }
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    uint32_t word[CN];
#pragma unroll
                    for (int c = 0; c < CN; ++c) word[c] = e == 0 ? wq[c].x : wq[c].y;
                    word_step(2 * q + e, word);
                }
            }
        } else if (vecw == 4) {
            // rows are whole 16-byte groups: four words per lane and request
            const int row4 = p.dec.row_len >> 2;
            for (int q = me; q < row4; q += lanes) {
                uint4 wq[CN];
#pragma unroll
                for (int c = 0; c < CN; ++c) {
                    wq[c] = make_uint4(0, 0, 0, 0);
                    if (n0 + c < p.N && DS_W_OK(p, reinterpret_cast<const uint4*>(p.packed + (size_t)(n0 + c) * p.dec.row_len) + q, 16))
                        wq[c] = __ldg(reinterpret_cast<const uint4*>(p.packed + (size_t)(n0 + c) * p.dec.row_len) + q);
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    uint32_t word[CN];
#pragma unroll
                    for (int c = 0; c < CN; ++c) word[c] = e == 0 ? wq[c].x : (e == 1 ? wq[c].y : (e == 2 ? wq[c].z : wq[c].w));
                    word_step(4 * q + e, word);
                }
            }
        } else {
            for (int w = me; w < p.dec.row_len; w += lanes) {
                uint32_t word[CN];
#pragma unroll
                for (int c = 0; c < CN; ++c)
                    word[c] = (n0 + c < p.N && DS_W_OK(p, p.packed + (size_t)(n0 + c) * p.dec.row_len + w, 4))
                                  ? uint32_t(__ldg(p.packed + (size_t)(n0 + c) * p.dec.row_len + w)) : 0u;
                word_step(w, word);
            }
        }
    }
    // K-split reduction: shuffle tree inside the warp, shared memory across the warps of a group
#pragma unroll
    for (int m = 0; m < MR; ++m)
#pragma unroll
        for (int c = 0; c < CN; ++c) {
            int v = acc[m][c];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            acc[m][c] = v;
        }
    if (wpc > 1) {
        if (lane == 0) {
#pragma unroll
            for (int m = 0; m < MR; ++m)
#pragma unroll
                for (int c = 0; c < CN; ++c) part[warp][m * CN + c] = acc[m][c];
        }
        __syncthreads();
        if (ksplit != 0) return;
#pragma unroll
        for (int m = 0; m < MR; ++m)
#pragma unroll
            for (int c = 0; c < CN; ++c) {
                int v = 0;
                for (int q = 0; q < wpc; ++q) v += part[warp + q][m * CN + c];
                acc[m][c] = v;
            }
    }
    // epilogue: lane e of the warp finishes output e = (m, c) of the group
    if (n0 >= p.N) return;
#pragma unroll
    for (int m = 0; m < MR; ++m)
#pragma unroll
        for (int c = 0; c < CN; ++c) {
            if (lane != m * CN + c) continue;
            const int n = n0 + c, row = m0 + m;
            if (n >= p.N || row >= p.M) continue;
            const size_t o = (size_t)row * p.N + n;
            int v = acc[m][c];
            if (p.bias) v += __ldg(p.bias + n);
            if (p.residual && DS_O_OK(p, p.residual, p.residual + o, 4))
                v = __float2int_rn(__int2float_rn(v) + __int2float_rn(__ldg(p.residual + o)));
            if (p.relu) v = max(v, 0);
            if (p.requant) v = min(max(v, p.rq_lo), p.rq_hi) * p.rq_mul + p.rq_add;
            if (p.round_f32) v = __float2int_rn(__int2float_rn(v));
            if (!DS_O_OK(p, p.out, static_cast<int*>(p.out) + o, 4)) continue;
            if (p.out_kind == DS_OUT_I32) static_cast<int*>(p.out)[o] = v;
            else static_cast<float*>(p.out)[o] = __int2float_rn(v) * p.inv_scale;
        }
}

template <int MR, int CN>
int launch_small(const GemmParams& p, cudaStream_t st)
{
    const int groups = (p.N + CN - 1) / CN;
    // warps that share a column group: enough for two full rounds of warps on the GPU, at most 8,
    // and never more than there are 32-word slices of a row
    int wpc = 1;
    const long long row_blocks = (long long)(p.M + MR - 1) / MR;
    while (wpc < SM_WARPS && (long long)groups * wpc * row_blocks < 2LL * 148 * 16 && p.dec.row_len > 32 * wpc) wpc *= 2;
    const int groups_per_cta = SM_WARPS / wpc;
    const long long gx = ((long long)groups + groups_per_cta - 1) / groups_per_cta;
    if (gx > 2147483647LL || row_blocks > 65535) return DS_ERR_RANGE;
    // packed words per request: 4 or 2 where every row starts on such a boundary, else 1
    const uintptr_t pw = reinterpret_cast<uintptr_t>(p.packed);
    const int vecw = (p.dec.row_len % 4 == 0 && (pw & 15u) == 0) ? 4 : ((p.dec.row_len % 2 == 0 && (pw & 7u) == 0) ? 2 : 1);
    const dim3 grid((unsigned)gx, (unsigned)row_blocks);
    if (p.in_kind == DS_IN_I32)
        small_linear_kernel<MR, CN, INK_I32><<<grid, SM_THREADS, 0, st>>>(p, wpc, vecw);
    else if (p.in_kind == DS_IN_I32_CLAMP)
        small_linear_kernel<MR, CN, INK_I32_CLAMP><<<grid, SM_THREADS, 0, st>>>(p, wpc, vecw);
    else
        small_linear_kernel<MR, CN, INK_F32><<<grid, SM_THREADS, 0, st>>>(p, wpc, vecw);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
}

}  // namespace

int launch_small_linear(const GemmParams& p, cudaStream_t st)
{
    if (p.M <= 1) return launch_small<1, 4>(p, st);
    if (p.M <= 2) return launch_small<2, 4>(p, st);
    if (p.M <= 4) return launch_small<4, 4>(p, st);
    return launch_small<8, 4>(p, st);  // blocks of 8 rows
}

}  // namespace ds
