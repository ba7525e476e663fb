// Declarations shared by the two GEMM/convolution kernels (ds_gemm.cu, ds_gemm_ws.cu).
#pragma once
#include <cstddef>
#include <type_traits>

#include "ds_common.cuh"

namespace ds {

constexpr int kTM = 8;  // rows of x per thread
constexpr int kPadMarker = 0x7FC0DEAD;  // NaN pattern standing for "integer 0, do not quantise"
constexpr int MODE_INT = 0, MODE_FP = 1;
constexpr int AM_LINEAR = -1, AM_TABLE = 0;  // AM >= 1: row mode with KW = AM
// Row mode for 3-wide windows with stride 1 and padding 1 along W, W a multiple of 4 and x 16-byte
// aligned: a producer thread fetches four neighbouring pixels of a row with one 16-byte load plus
// the two values beside them, and stores the three shifted copies as 16-byte vectors.
constexpr int AM_QUAD3 = 13;
// The same for W a multiple of 2 only and x 8-byte aligned: two pixels per 8-byte load.
constexpr int AM_PAIR3 = 23;
// Row mode for 7-wide windows with stride 2 and padding 3 along W (the stem of the ImageNet
// ResNets), W a multiple of 8 and x 16-byte aligned: a producer thread fetches the sixteen input
// values under four neighbouring output pixels with four 16-byte loads and stores the seven
// window columns as 16-byte vectors.
constexpr int AM_S2K7 = 27;

struct GemmParams {
    const void* x;        // int32 or fp32
    const int32_t* packed;
    const int32_t* bias;  // may be null
    void* out;            // int32 or fp32
    const int32_t* residual;
    int M, K, N;
    Decode dec;
    int kt_words;     // packed words per row per k-tile
    int bk;           // k values per tile = kt_words * num
    int ntiles;       // ceil(row_len / kt_words)
    int flush_tiles;  // FP path: tiles between drains of the float accumulators
    int tail_neg;     // FP path: slots k >= K inside the last tile; each decodes as a negative weight
    // convolution geometry
    int C, H, W, OC, KH, KW, sh, sw, ph, pw, OH, OW, P;  // P = OH*OW
    unsigned magic_khw, magic_kw, magic_kh;  // ceil(2^32 / d), 0 for d == 1: __umulhi(k, magic) == k / d
    int rows_per_tile;  // row mode: (ic,kh) rows per k-tile = bk / KW
    // fused prologue / epilogue
    int in_kind, out_kind, relu, requant, round_f32;
    // split-K (warp-specialised kernel): gridDim.z CTAs share one output tile
    int grid_m, grid_n;  // output tiles along M and N
    int splits;          // 1 = off
    int tiles_per_split; // k-tiles per split
    int* counters;       // one arrival counter per output tile, zero between launches
    long long counter_slots;
    // tail split (warp-specialised kernel): the output tiles that would form a last, mostly empty
    // wave are each shared by tail_splits CTAs, which exchange partial sums through `partials`
    int full_units;      // work units before the tail: grid_m * grid_n * splits, or the full waves
    int tail_first;      // first output tile of the tail
    int tail_items;      // output tiles in the tail, 0 = off
    int tail_splits;
    int tail_tps;        // k-tiles per tail split
    int* partials;       // [tail item][split][kTM * TN][consumer thread]
    long long partial_bytes;
    // weights expanded once per launch (warp-specialised kernel): +-2^-r as floats, 0 beyond K or N
    const float* wd;     // [ntiles * bk][npad], null = the producers decode the packed words
    const int* negpre;   // [ntiles + 1][npad]: negative weights of a column in the k-tiles before t
    int npad;            // grid_n * BN
    int* err_flag;       // set to 1 by a kernel whose bounded wait ran out
    // Range-gated launch (act_bits = DS_ACT_BITS_AUTO): the kernel runs only if *gate == gate_want.  A
    // one-pass kernel has written 0 there when every activation is within the FP32-pipe bound, else 1;
    // the FP32-pipe launch wants 0, the integer-path launch behind it wants 1.  Null = always run.
    const int* gate;
    int gate_want;
    // Checked build (-DDS_BOUNDS_CHECK) only: byte extents of x, of the packed weights and of the output
    // (the residual has the output's element count), and where the first violation goes.
    long long chk_x_bytes, chk_w_bytes, chk_o_bytes;
    int* chk_status;
    // weights expanded ahead of time by the caller (ds_conv2d_prepare)
    const void* prepared;
    long long prepared_bytes;
    int prepare_only;        // this call only fills `prepared` (or reports its size), no convolution
    long long* needed_out;   // host: receives the bytes `prepared` needs for this geometry
    Quant q;
    // round_to_fixed on a value that already is an int32 code (DS_IN_I32_CLAMP, `requant`):
    // code' = clamp(code, rq_lo, rq_hi) * rq_mul + rq_add.  I >= 2: the clamp alone (mul 1, add 0).
    // I == 1 (utils.py:12-13, sign(x) - 1): clamp to [-1, 1], times 2^F, minus 2^F.
    int rq_lo, rq_hi, rq_mul, rq_add;
    int pad_raw;  // what a position outside the image or matrix is read as, so that its code is 0: 0 for
                  // int32 codes, 1 under the sign rule (code' of 1 is 0), kPadMarker for fp32 inputs
    int in_mul2, in_add2;  // FP path: float bits of 1.5*2^22 + code' + 0.5 = clamp * in_mul2 + in_add2
    float inv_scale;  // 2^-F
};

// Leading int32 slots of a caller's workspace that hold arrival counters; partial sums follow.
constexpr int kWorkspaceCounters = 16384;
// The last counter word is never handed out as a counter: it holds the range flag of gated launches.
constexpr int kWorkspaceGateSlot = kWorkspaceCounters - 1;

struct alignas(16) KEntry {
    int off;  // byte offset of the tap (table mode) or of the row start (row mode)
    int kh;   // 31 marks an entry past the end of K (bit 31 of a row mask is never set)
    int kw;
    int pad;
};

// ---- checked build ------------------------------------------------------------------------------
// With -DDS_BOUNDS_CHECK every global load of x, of the packed weights and of the residual, and every
// global store, first tests its address against the extent the host derived from the call's
// arguments.  An access outside is NOT performed; the first one leaves a site code in a status word
// (ds_bounds_status).  Nothing traps.  Without the flag the tests compile to nothing.
#ifdef DS_BOUNDS_CHECK
__device__ __forceinline__ bool bounds_ok(int* status, const void* base, long long total, const void* ptr, int bytes,
                                          int site)
{
    const char* b = static_cast<const char*>(base);
    const char* q = static_cast<const char*>(ptr);
    if (q >= b && q + bytes <= b + total) return true;
    if (status) atomicCAS(status, 0, site);
    return false;
}
#define DS_X_OK(p, ptr, bytes) bounds_ok((p).chk_status, (p).x, (p).chk_x_bytes, ptr, bytes, 1)
#define DS_W_OK(p, ptr, bytes) bounds_ok((p).chk_status, (p).packed, (p).chk_w_bytes, ptr, bytes, 2)
#define DS_O_OK(p, base, ptr, bytes) bounds_ok((p).chk_status, base, (p).chk_o_bytes, ptr, bytes, 3)
#else
#define DS_X_OK(p, ptr, bytes) true
#define DS_W_OK(p, ptr, bytes) true
#define DS_O_OK(p, base, ptr, bytes) true
#endif
int* bounds_status_ptr();  // device address of the status word (ds_gemm_ws.cu), null on failure

__device__ __forceinline__ void red_shared_add(int* addr, int v)
{
    asm volatile("red.shared.add.s32 [%0], %1;" ::"r"((unsigned)__cvta_generic_to_shared(addr)), "r"(v)
                 : "memory");
}

__device__ __forceinline__ int magic_div(int k, unsigned magic) { return magic ? int(__umulhi(unsigned(k), magic)) : k; }


// Epilogue shared by both kernels: v = acc + bias (+ negative-weight count), optional residual
// add, ReLU, requantise clamp, then int32 or fp32 store.  Thread (tm, tn) owns rows
// 4*tm..4*tm+3 and BM/2 + the same, and columns 4*tn..4*tn+3 (and BN/2 + the same when TN == 8)
// of the CTA tile at (m0, n0).  `accv(i, j, o)` returns the finished integer sum of the element
// whose offset in the output is o, `colc(col)` the per-column constant added to it.
template <int TN, bool CONV, class AccFn, class ColFn>
__device__ __forceinline__ void store_tile(const GemmParams& p, int m0, int n0, int tm, int tn, int BM, int BN,
                                           AccFn accv, ColFn colc)
{
    auto ncol = [&](int j) { return (TN == 8 && j >= 4) ? (BN / 2 + 4 * tn + j - 4) : (4 * tn + j); };
    auto mrow = [&](int i) { return (i >= 4) ? (BM / 2 + 4 * tm + i - 4) : (4 * tm + i); };
    int addc[TN];
#pragma unroll
    for (int j = 0; j < TN; ++j) {
        const int n = n0 + ncol(j);
        int c = 0;
        if (n < p.N) {
            if (p.bias) c = __ldg(p.bias + n);
            c += colc(ncol(j));
        }
        addc[j] = c;
    }
    auto finish = [&](int v, long long oidx) -> int {
        if (p.residual) {
            // fp32 add of the two values as the reference's `out += identity` does it.
            const int r = DS_O_OK(p, p.residual, p.residual + oidx, 4) ? __ldg(p.residual + oidx) : 0;
            v = __float2int_rn(__int2float_rn(v) + __int2float_rn(r));
        }
        if (p.relu) v = max(v, 0);
        if (p.requant) v = min(max(v, p.rq_lo), p.rq_hi) * p.rq_mul + p.rq_add;
        if (p.round_f32) v = __float2int_rn(__int2float_rn(v));
        return v;
    };
    int32_t* oi = static_cast<int32_t*>(p.out);
    float* of = static_cast<float*>(p.out);

    if (CONV) {
        // 4 consecutive rows m of one column n are contiguous in NCHW when P % 4 == 0.
        const bool vec = (p.P % 4 == 0);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int m = m0 + mrow(4 * h);
            if (m >= p.M) continue;
            if (vec) {
                const int b = m / p.P, pp = m - b * p.P;
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    const int n = n0 + ncol(j);
                    if (n >= p.N) continue;
                    const long long o = ((long long)b * p.OC + n) * p.P + pp;
                    int v[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) v[i] = finish(accv(4 * h + i, j, o + i) + addc[j], o + i);
                    if (p.out_kind == DS_OUT_I32) {
                        if (DS_O_OK(p, oi, oi + o, 16)) *reinterpret_cast<int4*>(oi + o) = make_int4(v[0], v[1], v[2], v[3]);
                    } else if (DS_O_OK(p, of, of + o, 16)) {
                        *reinterpret_cast<float4*>(of + o) =
                            make_float4(__int2float_rn(v[0]) * p.inv_scale, __int2float_rn(v[1]) * p.inv_scale,
                                        __int2float_rn(v[2]) * p.inv_scale, __int2float_rn(v[3]) * p.inv_scale);
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int mi = m + i;
                    if (mi >= p.M) continue;
                    const int b = mi / p.P, pp = mi - b * p.P;
#pragma unroll
                    for (int j = 0; j < TN; ++j) {
                        const int n = n0 + ncol(j);
                        if (n >= p.N) continue;
                        const long long o = ((long long)b * p.OC + n) * p.P + pp;
                        const int v = finish(accv(4 * h + i, j, o) + addc[j], o);
                        if (p.out_kind == DS_OUT_I32) {
                            if (DS_O_OK(p, oi, oi + o, 4)) oi[o] = v;
                        } else if (DS_O_OK(p, of, of + o, 4)) {
                            of[o] = __int2float_rn(v) * p.inv_scale;
                        }
                    }
                }
            }
        }
    } else {
        const bool vec = (p.N % 4 == 0);
#pragma unroll
        for (int i = 0; i < kTM; ++i) {
            const int m = m0 + mrow(i);
            if (m >= p.M) continue;
#pragma unroll
            for (int h = 0; h < TN / 4; ++h) {
                const int n = n0 + ncol(4 * h);
                const long long o = (long long)m * p.N + n;
                if (vec && n + 3 < p.N) {
                    int v[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[j] = finish(accv(i, 4 * h + j, o + j) + addc[4 * h + j], o + j);
                    if (p.out_kind == DS_OUT_I32) {
                        if (DS_O_OK(p, oi, oi + o, 16)) *reinterpret_cast<int4*>(oi + o) = make_int4(v[0], v[1], v[2], v[3]);
                    } else if (DS_O_OK(p, of, of + o, 16)) {
                        *reinterpret_cast<float4*>(of + o) =
                            make_float4(__int2float_rn(v[0]) * p.inv_scale, __int2float_rn(v[1]) * p.inv_scale,
                                        __int2float_rn(v[2]) * p.inv_scale, __int2float_rn(v[3]) * p.inv_scale);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (n + j >= p.N) continue;
                        const int v = finish(accv(i, 4 * h + j, o + j) + addc[4 * h + j], o + j);
                        if (p.out_kind == DS_OUT_I32) {
                            if (DS_O_OK(p, oi, oi + o + j, 4)) oi[o + j] = v;
                        } else if (DS_O_OK(p, of, of + o + j, 4)) {
                            of[o + j] = __int2float_rn(v) * p.inv_scale;
                        }
                    }
                }
            }
        }
    }
}

// Split-K: adds this CTA's partial sums (plus `colc`, without bias or epilogue) into the output
// slots, which the host zeroed before the launch.  Integer adds commute, so the result does not
// depend on the order in which the splits arrive.  Same element mapping as store_tile.
template <int TN, bool CONV, class AccFn, class ColFn>
__device__ __forceinline__ void reduce_tile(const GemmParams& p, int m0, int n0, int tm, int tn, int BM, int BN,
                                            AccFn accv, ColFn colc)
{
    auto ncol = [&](int j) { return (TN == 8 && j >= 4) ? (BN / 2 + 4 * tn + j - 4) : (4 * tn + j); };
    auto mrow = [&](int i) { return (i >= 4) ? (BM / 2 + 4 * tm + i - 4) : (4 * tm + i); };
    int* oi = static_cast<int*>(p.out);
#pragma unroll
    for (int i = 0; i < kTM; ++i) {
        const int m = m0 + mrow(i);
        if (m >= p.M) continue;
        long long rowoff, nstride;
        if (CONV) {
            const int b = m / p.P, pp = m - b * p.P;
            rowoff = (long long)b * p.OC * p.P + pp;
            nstride = p.P;
        } else {
            rowoff = (long long)m * p.N;
            nstride = 1;
        }
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + ncol(j);
            if (n >= p.N) continue;
            if (DS_O_OK(p, oi, oi + rowoff + n * nstride, 4))
                atomicAdd(oi + rowoff + n * nstride, accv(i, j, 0) + colc(ncol(j)));
        }
    }
}

// Fixed-point value v (int32 bits, or fp32 bits for the fp32 input kinds) as the operand the
// kernels keep in shared memory: x + 0.5 as a float on the FP path, x as int bits otherwise.
// INK selects the input kind at compile time: INK_I32, INK_I32_CLAMP or INK_F32 (either fp32 kind).
constexpr int INK_I32 = 0, INK_F32 = 1, INK_I32_CLAMP = 2;

template <bool FP, int INK>
__device__ __forceinline__ float operand_of(const GemmParams& p, int v)
{
    if (INK == INK_I32_CLAMP) {
        const int c = min(max(v, p.rq_lo), p.rq_hi);
        if (FP) return __int_as_float(c * p.in_mul2 + p.in_add2) - kHalfMagic;
        return __int_as_float(c * p.rq_mul + p.rq_add);
    }
    if (INK != INK_F32) {
        // x + 0.5 without an int->float conversion: adding 2x+1 to the bits of 1.5*2^22
        // (ulp 0.5) gives 1.5*2^22 + x + 0.5 exactly for |x| < 2^20.
        return FP ? (__int_as_float(2 * v + (kHalfMagicBits + 1)) - kHalfMagic) : __int_as_float(v);
    }
    float f;  // the quantised value, an integer held in a float
    if (v == kPadMarker) f = 0.f;
    else if (p.in_kind == DS_IN_F32_CONV) f = quant_conv_f(__int_as_float(v), p.q);
    else f = truncf(__int_as_float(v) * p.q.scale);
    return FP ? (f + 0.5f) : __int_as_float(__float2int_rz(f));
}

// Calls fn(integral_constant<int, INK>) for the input kind of this launch.
template <class Fn>
__device__ __forceinline__ void with_input_kind(const GemmParams& p, Fn fn)
{
    if (p.in_kind == DS_IN_I32) fn(std::integral_constant<int, INK_I32>());
    else if (p.in_kind == DS_IN_I32_CLAMP) fn(std::integral_constant<int, INK_I32_CLAMP>());
    else fn(std::integral_constant<int, INK_F32>());
}

// Small-batch linear layer (ds_small.cu): M <= 64 rows.  Exact integer path, optional split along
// K with integer atomics when no epilogue is fused.
int launch_small_linear(const GemmParams& p, cudaStream_t st);

// Warp-specialised FP32-pipe kernel (ds_gemm_ws.cuh).  am: AM_LINEAR (K a multiple of 4 and x
// 16-byte aligned), AM_TABLE, AM_QUAD3, AM_PAIR3, AM_S2K7 or the window width of the row mode (1, 3, 5, 7).  Returns DS_ERR_UNSUPPORTED when no k-tile fits; the caller
// then falls back to the table mode or the integer path.  The per-width entry points are what
// launch_ws dispatches to; they expect GemmParams::err_flag to be set.
int launch_ws(const GemmParams& p, int am, cudaStream_t st);
int launch_ws_am1(const GemmParams& p, cudaStream_t st);
int launch_ws_am3(const GemmParams& p, cudaStream_t st);
int launch_ws_am5(const GemmParams& p, cudaStream_t st);
int launch_ws_am7(const GemmParams& p, cudaStream_t st);
int launch_ws_table(const GemmParams& p, cudaStream_t st);
int launch_ws_quad3(const GemmParams& p, cudaStream_t st);
int launch_ws_pair3(const GemmParams& p, cudaStream_t st);
int launch_ws_linear(const GemmParams& p, cudaStream_t st);
int launch_ws_s2k7(const GemmParams& p, cudaStream_t st);

}  // namespace ds
