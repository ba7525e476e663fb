// Linear layer for small batches (M <= 64): out[m,n] = bias[n] + sum_k term(x[m,k], w[n,k]).
//
// With so few rows the work per weight is tiny, so the layer is bound by launch latency and by
// reading the packed weights once (1.5-4 shift-ops per byte at M = 1).  A CTA owns MT rows and
// 1024 / MT columns and walks K in chunks: the x chunk and the decoded (shift, multiplier) pairs
// of the chunk go to shared memory, each thread accumulates one row x four columns with the exact
// integer arithmetic (shift, then multiply-add).  When nothing is fused into the epilogue the K
// range is also split across gridDim.z and the partial sums are added into the zeroed output with
// integer atomics, which keeps the result bit-exact and fills the GPU.
#include "ds_gemm_common.cuh"

namespace ds {
namespace {

constexpr int SM_THREADS = 256;

// MT rows x NTILE columns per CTA, CPT columns per thread (256 threads).
template <int MT, int CPT>
struct SmallCfg {
    static constexpr int NTILE = SM_THREADS / MT * CPT;
    static constexpr int KC = (NTILE > 64) ? 16 : 32;  // k values per chunk
};

template <int MT, int CPT>
__global__ void __launch_bounds__(SM_THREADS) small_linear_kernel(const GemmParams p, int chunks_per_split)
{
    using Cfg = SmallCfg<MT, CPT>;
    constexpr int NTILE = Cfg::NTILE, KC = Cfg::KC;
    __shared__ int xs[MT][KC];
    __shared__ __align__(16) int2 wv[KC][NTILE];
    __shared__ int lut_s[256], lut_m[256];

    const int t = threadIdx.x;
    const int n0 = blockIdx.x * NTILE, m0 = blockIdx.y * MT;
    for (int f = t; f < (1 << p.dec.fw); f += SM_THREADS) {
        int shv, mul;
        decode_int(uint32_t(f), p.dec, true, shv, mul);
        lut_s[f] = shv;
        lut_m[f] = mul;
    }
    const int tm = t / (NTILE / CPT), tn = t % (NTILE / CPT);
    int acc[CPT];
#pragma unroll
    for (int j = 0; j < CPT; ++j) acc[j] = 0;
    const uint32_t fmask = (1u << p.dec.fw) - 1u;
    const int nchunks = (p.K + KC - 1) / KC;
    const int c_begin = blockIdx.z * chunks_per_split;
    const int c_end = min(nchunks, c_begin + chunks_per_split);
    __syncthreads();

    for (int c = c_begin; c < c_end; ++c) {
        const int k0 = c * KC;
        // x chunk: int32 codes (fp32 inputs are quantised here)
        for (int i = t; i < MT * KC; i += SM_THREADS) {
            const int ml = i / KC, kl = i % KC;
            const int m = m0 + ml, k = k0 + kl;
            int v = 0;
            if (m < p.M && k < p.K) {
                const int raw = __ldg(static_cast<const int*>(p.x) + ((long long)m * p.K + k));
                with_input_kind(p, [&](auto ink_tag) {
                    v = __float_as_int(operand_of<false, decltype(ink_tag)::value>(p, raw));
                });
            }
            xs[ml][kl] = v;
        }
        // decoded weights of the chunk
        for (int i = t; i < KC * NTILE; i += SM_THREADS) {
            const int n = i % NTILE, kl = i / NTILE;
            const int k = k0 + kl;
            int2 w = make_int2(0, 0);
            if (k < p.K && n0 + n < p.N) {
                const int wi = k / p.dec.num, slot = k - wi * p.dec.num;
                const uint32_t word = uint32_t(__ldg(p.packed + (long long)(n0 + n) * p.dec.row_len + wi));
                const uint32_t f = (word >> (slot * p.dec.fw)) & fmask;
                w = make_int2(lut_s[f], lut_m[f]);
            }
            wv[kl][n] = w;
        }
        __syncthreads();
#pragma unroll 4
        for (int kl = 0; kl < KC; ++kl) {
            const int xv = xs[tm][kl];
#pragma unroll
            for (int j = 0; j < CPT; ++j) {
                const int2 w = wv[kl][CPT * tn + j];
                acc[j] += (xv >> w.x) * w.y;
            }
        }
        __syncthreads();
    }

    const int m = m0 + tm;
    if (m >= p.M) return;
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
        const int n = n0 + CPT * tn + j;
        if (n >= p.N) continue;
        const long long o = (long long)m * p.N + n;
        int v = acc[j];
        if (gridDim.z > 1) {  // split along K: plain sums only, bias once
            if (blockIdx.z == 0 && p.bias) v += __ldg(p.bias + n);
            atomicAdd(static_cast<int*>(p.out) + o, v);
            continue;
        }
        if (p.bias) v += __ldg(p.bias + n);
        if (p.residual) v = __float2int_rn(__int2float_rn(v) + __int2float_rn(__ldg(p.residual + o)));
        if (p.relu) v = max(v, 0);
        if (p.requant) v = min(max(v, p.rq_lo), p.rq_hi) * p.rq_mul + p.rq_add;
        if (p.round_f32) v = __float2int_rn(__int2float_rn(v));
        if (p.out_kind == DS_OUT_I32) static_cast<int*>(p.out)[o] = v;
        else static_cast<float*>(p.out)[o] = __int2float_rn(v) * p.inv_scale;
    }
}

template <int MT, int CPT>
int launch_small(const GemmParams& p, cudaStream_t st)
{
    using Cfg = SmallCfg<MT, CPT>;
    const int gx = (p.N + Cfg::NTILE - 1) / Cfg::NTILE, gy = (p.M + MT - 1) / MT;
    const int nchunks = (p.K + Cfg::KC - 1) / Cfg::KC;
    const bool plain = p.out_kind == DS_OUT_I32 && !p.relu && !p.requant && !p.round_f32 && !p.residual;
    int splits = 1;
    if (plain) {
        while (splits < 16 && gx * gy * splits < 296 && nchunks / (splits * 2) >= 4) splits *= 2;
    }
    int per = (nchunks + splits - 1) / splits;
    splits = (nchunks + per - 1) / per;
    if (splits > 1 && cudaMemsetAsync(p.out, 0, size_t(p.M) * size_t(p.N) * 4, st) != cudaSuccess) return DS_ERR_CUDA;
    small_linear_kernel<MT, CPT><<<dim3(gx, gy, splits), SM_THREADS, 0, st>>>(p, per);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
}

}  // namespace

int launch_small_linear(const GemmParams& p, cudaStream_t st)
{
    if (p.N > 65535 * 64) return DS_ERR_RANGE;
    if (p.M <= 4) return launch_small<4, 4>(p, st);
    // few columns: one column per thread, four times as many CTAs
    const long long ctas4 = (long long)((p.N + 63) / 64) * ((p.M + 15) / 16);
    return ctas4 >= 148 ? launch_small<16, 4>(p, st) : launch_small<16, 1>(p, st);
}

}  // namespace ds
