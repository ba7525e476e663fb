// Shift-accumulate "GEMM" and implicit-im2col convolution for sm_100a.
//
// out[m,n] = bias[n] + sum_k term(x[m,k], w[n,k]),  term = sign * (x >> r)   (see the header)
//
// One tiled kernel serves both the linear layer (x is [M,K] row-major) and the convolution
// (x is unpadded NCHW; row m = (b,oh,ow), column k = (ic,kh,kw) is gathered on the fly, zero
// padding by predication -- the im2col matrix never exists).  Packed weight words are
// fetched from global memory and decoded once per CTA into shared memory; the decoded
// sign/shift never goes back to HBM.
//
// Two arithmetic paths, both bit-exact:
//   * integer path (FP == false): acc += (x >> sh) * mul, a funnel shift on the integer ALU
//     pipe plus an integer multiply-add on the FMA pipe.  Valid for every int32 input and
//     wraps modulo 2^32 like the reference.
//   * FP32-pipe path (FP == true): one FFMA with round-toward-minus-infinity per term.
//     With xh = x + 0.5 and w = +-2^-r, floor(xh * w) equals (x >> r) for w > 0 and
//     -(x >> r) - 1 for w < 0, because xh * w is never an integer.  Adding into an
//     accumulator of the form 1.5*2^23 + A (A an integer, |A| < 2^22) makes the FMA's single
//     rounding that floor.  The "-1" of every negative weight is a per-output constant that
//     the epilogue adds back, and the accumulator is drained into an int32 register often
//     enough that |A| stays below 2^22.  Needs base == 0 and a bound on |x| (act_bits).
#include "ds_common.cuh"

namespace ds {
namespace {

constexpr int kThreads = 256;
constexpr int kTM = 8;  // rows of x per thread
constexpr int kPadMarker = 0x7FC0DEAD;  // NaN pattern standing for "integer 0, do not quantise"

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
    // convolution geometry (CONV only)
    int C, H, W, OC, KH, KW, sh, sw, ph, pw, OH, OW, P;  // P = OH*OW
    // fused prologue / epilogue
    int in_kind, out_kind, relu, requant;
    Quant q;
    int rq_lo, rq_hi;
    float inv_scale;  // 2^-F
};

struct KEntry {
    int off;   // ic*H*W + kh*W + kw
    int khkw;  // kh | kw << 8; kh = 31 marks k >= K
};

template <int TMG, int TNG, int TN, int BKT, bool FP>
struct Smem {
    static constexpr int BM = TMG * kTM;
    static constexpr int BN = TNG * TN;
    static constexpr int AP = BM + 4;
    float a[2][BKT][AP];                 // FP: x + 0.5 as float; integer path: x as int bits
    float b[2][BKT][BN];                 // FP: +-2^-r; integer path: shift amounts (int bits)
    int bm[FP ? 1 : 2][FP ? 1 : BKT][FP ? 1 : BN];  // integer path: multipliers
    KEntry ktab[2][BKT];
    int negc[BN];                        // FP: number of negative weights per output column
};

template <int TN>
struct Frag {
    float v[TN];
};

// ---------------------------------------------------------------------------------------------
template <int TMG, int TNG, int TN, int BKT, bool FP, bool CONV>
__global__ void __launch_bounds__(kThreads, FP ? 1 : 2) gemm_kernel(const GemmParams p)
{
    using S = Smem<TMG, TNG, TN, BKT, FP>;
    constexpr int BM = S::BM, BN = S::BN;
    constexpr int EA = BM * BKT / kThreads;  // x elements staged per thread per tile
    constexpr int EW = (BN * BKT / 4 + kThreads - 1) / kThreads;  // words per thread (num >= 4)
    static_assert(TMG * TNG == kThreads, "256 threads");
    static_assert(TN == 4 || TN == 8, "TN");
    static_assert(EA >= 1 && EA <= 16, "staging registers");

    extern __shared__ __align__(16) unsigned char smem_raw[];
    S& s = *reinterpret_cast<S*>(smem_raw);

    const int t = threadIdx.x;
    const int m0 = blockIdx.x * BM;
    const int n0 = blockIdx.y * BN;
    // Threads that share n are adjacent in m for the convolution (NCHW output is contiguous in
    // m), and the other way round for the linear layer ([M,N] output is contiguous in n).
    const int tm = CONV ? (t % TMG) : (t / TNG);
    const int tn = CONV ? (t / TMG) : (t % TNG);

    // ---- per-thread staging geometry -------------------------------------------------------
    // CONV: thread stages column k_local = t / BM + (256 / BM) * e of row m_local = t % BM.
    // LINEAR: k_local = t % BKT, m_local = t / BKT + (256 / BKT) * e  (k is contiguous in x).
    const int a_m = CONV ? (t % BM) : (t / BKT);
    const int a_k = CONV ? (t / BM) : (t % BKT);
    constexpr int A_MSTEP = CONV ? 0 : (kThreads / BKT);
    constexpr int A_KSTEP = CONV ? ((kThreads >= BM) ? kThreads / BM : 1) : 0;
    constexpr int A_ELEMS = CONV ? (BKT / A_KSTEP) : EA;
    static_assert(A_ELEMS <= 16, "staging registers");
    static_assert(!CONV || kThreads >= BM || true, "");

    const int32_t* xi = static_cast<const int32_t*>(p.x);
    const float* xf = static_cast<const float*>(p.x);
    long long x_base = 0;       // CONV: element offset of (b, 0, ih0, iw0)
    uint32_t rowmask = 0, colmask = 0;
    if (CONV) {
        // BM can exceed 256 only if a thread owned several rows; not instantiated.
        const int m = m0 + a_m;
        if (m < p.M) {
            const int b = m / p.P, pp = m - b * p.P;
            const int oh = pp / p.OW, ow = pp - oh * p.OW;
            const int ih0 = oh * p.sh - p.ph, iw0 = ow * p.sw - p.pw;
            for (int kh = 0; kh < p.KH; ++kh)
                if (unsigned(ih0 + kh) < unsigned(p.H)) rowmask |= 1u << kh;
            for (int kw = 0; kw < p.KW; ++kw)
                if (unsigned(iw0 + kw) < unsigned(p.W)) colmask |= 1u << kw;
            x_base = (long long)b * p.C * p.H * p.W + (long long)ih0 * p.W + iw0;
        }
    }

    // ---- accumulators ----------------------------------------------------------------------
    int acc[kTM][TN];
    float accf[FP ? kTM : 1][FP ? TN : 1];
#pragma unroll
    for (int i = 0; i < kTM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            acc[i][j] = 0;
            if (FP) accf[i][j] = kMagic;
        }
    if (FP)
        for (int i = t; i < BN; i += kThreads) s.negc[i] = 0;

    // ---- staging helpers -------------------------------------------------------------------
    int a_reg[A_ELEMS];
    uint32_t w_reg[EW];

    auto fill_ktab = [&](int tile, int buf) {
        if (CONV && t < p.bk) {
            const int k = tile * p.bk + t;
            KEntry e;
            if (k < p.K) {
                const int khw = p.KH * p.KW;
                const int ic = k / khw, tap = k - ic * khw;
                const int kh = tap / p.KW, kw = tap - kh * p.KW;
                e.off = ic * p.H * p.W + kh * p.W + kw;
                e.khkw = kh | (kw << 8);
            } else {
                e.off = 0;
                e.khkw = 31;
            }
            s.ktab[buf][t] = e;
        }
    };

    // Raw fetch of tile `tile` into registers (x as int bits of the quantised value).
    auto fetch = [&](int tile, int buf) {
        const int k0 = tile * p.bk;
#pragma unroll
        for (int e = 0; e < A_ELEMS; ++e) {
            // fp32 inputs: positions outside the image or the matrix carry a marker (a NaN
            // pattern) so that stash() stores the integer 0 there without quantising it.
            int v = (p.in_kind == DS_IN_I32) ? 0 : kPadMarker;
            if (CONV) {
                const int kl = a_k + e * A_KSTEP;
                if (kl < p.bk) {
                    const KEntry ke = s.ktab[buf][kl];
                    const int kh = ke.khkw & 0xff, kw = ke.khkw >> 8;
                    if (((rowmask >> kh) & (colmask >> kw) & 1u) != 0u) {
                        const long long idx = x_base + ke.off;
                        if (p.in_kind == DS_IN_I32) v = __ldg(xi + idx);
                        else v = __float_as_int(__ldg(xf + idx));
                    }
                }
            } else {
                const int ml = a_m + e * A_MSTEP;
                const int m = m0 + ml, k = k0 + a_k;
                if (a_k < p.bk && m < p.M && k < p.K) {
                    const long long idx = (long long)m * p.K + k;
                    if (p.in_kind == DS_IN_I32) v = __ldg(xi + idx);
                    else v = __float_as_int(__ldg(xf + idx));
                }
            }
            a_reg[e] = v;
        }
        const int w0 = tile * p.kt_words;
        const int nwords = BN * p.kt_words;
#pragma unroll
        for (int e = 0; e < EW; ++e) {
            const int wi = t + e * kThreads;
            uint32_t w = 0;
            if (wi < nwords) {
                const int n = wi % BN, jw = wi / BN;
                if (n0 + n < p.N && w0 + jw < p.dec.row_len)
                    w = uint32_t(__ldg(p.packed + (long long)(n0 + n) * p.dec.row_len + w0 + jw));
            }
            w_reg[e] = w;
        }
    };

    // Convert and store the registers of tile `tile` into shared buffer `buf`.
    auto stash = [&](int tile, int buf) {
        const int k0 = tile * p.bk;
#pragma unroll
        for (int e = 0; e < A_ELEMS; ++e) {
            const int kl = CONV ? (a_k + e * A_KSTEP) : a_k;
            const int ml = CONV ? a_m : (a_m + e * A_MSTEP);
            if (kl < p.bk) {
                const int v = a_reg[e];
                float o;
                if (p.in_kind == DS_IN_I32) {
                    // x + 0.5 without an int->float conversion: adding 2x+1 to the bits of
                    // 1.5*2^22 (ulp 0.5) gives 1.5*2^22 + x + 0.5 exactly for |x| < 2^20.
                    o = FP ? (__int_as_float(2 * v + (kHalfMagicBits + 1)) - kHalfMagic) : __int_as_float(v);
                } else {
                    float f;  // the quantised value, an integer held in a float
                    if (v == kPadMarker) f = 0.f;
                    else if (p.in_kind == DS_IN_F32_CONV) f = quant_conv_f(__int_as_float(v), p.q);
                    else f = truncf(__int_as_float(v) * p.q.scale);
                    o = FP ? (f + 0.5f) : __int_as_float(__float2int_rz(f));
                }
                s.a[buf][kl][ml] = o;
            }
        }
        const int nwords = BN * p.kt_words;
#pragma unroll
        for (int e = 0; e < EW; ++e) {
            const int wi = t + e * kThreads;
            if (wi < nwords) {
                const int n = wi % BN, jw = wi / BN;
                uint32_t w = w_reg[e];
                const int kbase = jw * p.dec.num;
                int negs = 0;
                for (int i = 0; i < p.dec.num; ++i) {
                    const bool live = (k0 + kbase + i) < p.K;
                    if (FP) {
                        int neg;
                        s.b[buf][kbase + i][n] = decode_f32(w, p.dec, live, neg);
                        negs += neg;
                    } else {
                        int shv, mul;
                        decode_int(w, p.dec, live, shv, mul);
                        s.b[buf][kbase + i][n] = __int_as_float(shv);
                        s.bm[buf][kbase + i][n] = mul;
                    }
                    w >>= p.dec.fw;
                }
                if (FP && negs) atomicAdd(&s.negc[n], negs);
            }
        }
    };

    auto compute = [&](int buf) {
#pragma unroll 4
        for (int k = 0; k < p.bk; ++k) {
            float a[kTM];
            *reinterpret_cast<float4*>(&a[0]) = *reinterpret_cast<const float4*>(&s.a[buf][k][4 * tm]);
            *reinterpret_cast<float4*>(&a[4]) =
                *reinterpret_cast<const float4*>(&s.a[buf][k][BM / 2 + 4 * tm]);
            float b[TN];
            *reinterpret_cast<float4*>(&b[0]) = *reinterpret_cast<const float4*>(&s.b[buf][k][4 * tn]);
            if (TN == 8)
                *reinterpret_cast<float4*>(&b[TN - 4]) =
                    *reinterpret_cast<const float4*>(&s.b[buf][k][BN / 2 + 4 * tn]);
            if (FP) {
#pragma unroll
                for (int i = 0; i < kTM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j) accf[i][j] = __fmaf_rd(a[i], b[j], accf[i][j]);
            } else {
                int mu[TN];
                *reinterpret_cast<int4*>(&mu[0]) = *reinterpret_cast<const int4*>(&s.bm[buf][k][4 * tn]);
                if (TN == 8)
                    *reinterpret_cast<int4*>(&mu[TN - 4]) =
                        *reinterpret_cast<const int4*>(&s.bm[buf][k][BN / 2 + 4 * tn]);
#pragma unroll
                for (int i = 0; i < kTM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j)
                        acc[i][j] += (__float_as_int(a[i]) >> __float_as_int(b[j])) * mu[j];
            }
        }
    };

    auto drain = [&]() {
#pragma unroll
        for (int i = 0; i < kTM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                acc[i][j] += __float_as_int(accf[i][j]) - kMagicBits;
                accf[i][j] = kMagic;
            }
    };

    // ---- main loop: two shared buffers, register prefetch, one barrier per tile --------------
    fill_ktab(0, 0);
    __syncthreads();
    fetch(0, 0);
    fill_ktab(1, 1);
    stash(0, 0);
    __syncthreads();
    int since = 0;
    for (int tile = 0; tile < p.ntiles; ++tile) {
        const int buf = tile & 1;
        const bool more = tile + 1 < p.ntiles;
        if (more) fetch(tile + 1, buf ^ 1);
        compute(buf);
        if (FP && ++since == p.flush_tiles) {
            drain();
            since = 0;
        }
        if (more) {
            stash(tile + 1, buf ^ 1);
            fill_ktab(tile + 2, buf);
        }
        __syncthreads();
    }
    if (FP) drain();

    // ---- epilogue -----------------------------------------------------------------------------
    // Column index of accumulator j and row index of accumulator i inside the CTA tile.
    auto ncol = [&](int j) { return (TN == 8 && j >= 4) ? (BN / 2 + 4 * tn + j - 4) : (4 * tn + j); };
    auto mrow = [&](int i) { return (i >= 4) ? (BM / 2 + 4 * tm + i - 4) : (4 * tm + i); };

    int addc[TN];
#pragma unroll
    for (int j = 0; j < TN; ++j) {
        const int n = n0 + ncol(j);
        int c = 0;
        if (n < p.N) {
            if (p.bias) c = __ldg(p.bias + n);
            if (FP) c += s.negc[ncol(j)];
        }
        addc[j] = c;
    }

    auto finish = [&](int v, long long oidx) -> int {
        if (p.residual) {
            // fp32 add of the two values as the reference's `out += identity` does it.
            v = __float2int_rn(__int2float_rn(v) + __int2float_rn(__ldg(p.residual + oidx)));
        }
        if (p.relu) v = max(v, 0);
        if (p.requant) v = min(max(v, p.rq_lo), p.rq_hi);
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
                    for (int i = 0; i < 4; ++i) v[i] = finish(acc[4 * h + i][j] + addc[j], o + i);
                    if (p.out_kind == DS_OUT_I32) {
                        *reinterpret_cast<int4*>(oi + o) = make_int4(v[0], v[1], v[2], v[3]);
                    } else {
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
                        const int v = finish(acc[4 * h + i][j] + addc[j], o);
                        if (p.out_kind == DS_OUT_I32) oi[o] = v;
                        else of[o] = __int2float_rn(v) * p.inv_scale;
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
                    for (int j = 0; j < 4; ++j) v[j] = finish(acc[i][4 * h + j] + addc[4 * h + j], o + j);
                    if (p.out_kind == DS_OUT_I32) {
                        *reinterpret_cast<int4*>(oi + o) = make_int4(v[0], v[1], v[2], v[3]);
                    } else {
                        *reinterpret_cast<float4*>(of + o) =
                            make_float4(__int2float_rn(v[0]) * p.inv_scale, __int2float_rn(v[1]) * p.inv_scale,
                                        __int2float_rn(v[2]) * p.inv_scale, __int2float_rn(v[3]) * p.inv_scale);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (n + j >= p.N) continue;
                        const int v = finish(acc[i][4 * h + j] + addc[4 * h + j], o + j);
                        if (p.out_kind == DS_OUT_I32) oi[o + j] = v;
                        else of[o + j] = __int2float_rn(v) * p.inv_scale;
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
template <int TMG, int TNG, int TN, int BKT, bool FP, bool CONV>
int launch_cfg(GemmParams& p, cudaStream_t st)
{
    using S = Smem<TMG, TNG, TN, BKT, FP>;
    constexpr int BM = S::BM, BN = S::BN;
    p.kt_words = BKT / p.dec.num;
    if (p.kt_words < 1) return DS_ERR_UNSUPPORTED;
    p.bk = p.kt_words * p.dec.num;
    p.ntiles = (p.dec.row_len + p.kt_words - 1) / p.kt_words;
    auto kern = gemm_kernel<TMG, TNG, TN, BKT, FP, CONV>;
    const size_t smem = sizeof(S);
    static bool attr_done = false;  // per instantiation
    if (!attr_done) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) {
            cudaGetLastError();
            return DS_ERR_CUDA;
        }
        attr_done = true;
    }
    const long long gx = ((long long)p.M + BM - 1) / BM, gy = (p.N + BN - 1) / BN;
    if (gx > 2147483647LL || gy > 65535) return DS_ERR_RANGE;
    kern<<<dim3((unsigned)gx, (unsigned)gy), kThreads, smem, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
}

template <bool FP, bool CONV>
int launch_path(GemmParams& p, cudaStream_t st)
{
    // Tile shape by output width: 128x128 for wide layers, 256x64 for 64-channel layers,
    // 256x32 below that; 64x128 when there are few rows (small-batch linear layers).
    if (!CONV && p.M <= 64) return launch_cfg<8, 32, 4, 32, FP, CONV>(p, st);
    if (p.N > 64) return launch_cfg<16, 16, 8, 32, FP, CONV>(p, st);
    if (p.N > 32) return launch_cfg<32, 8, 8, 16, FP, CONV>(p, st);
    return launch_cfg<32, 8, 4, 16, FP, CONV>(p, st);
}

int setup_common(GemmParams& p, int bits, int base, const ds_fuse_t* fuse, bool& use_fp)
{
    if (bits < 1 || bits > 7) return DS_ERR_UNSUPPORTED;  // the reference's range, shift.cu:194-385
    if (base > 0) return DS_ERR_UNSUPPORTED;
    p.dec.bits = bits;
    p.dec.fw = bits + 1;
    p.dec.num = 32 / (bits + 1);
    p.dec.base = base;
    p.dec.row_len = (p.K + p.dec.num - 1) / p.dec.num;
    ds_fuse_t f = {};
    if (fuse) f = *fuse;
    if (f.in_kind < 0 || f.in_kind > 2 || f.out_kind < 0 || f.out_kind > 1) return DS_ERR_BAD_ARG;
    const int I = f.act_integer_bits, F = f.act_fraction_bits;
    const bool needs_if = f.in_kind != DS_IN_I32 || f.out_kind != DS_OUT_I32 || f.requant;
    if (needs_if && (F < 0 || F > 30)) return DS_ERR_BAD_ARG;
    if ((f.in_kind == DS_IN_F32_CONV || f.requant) && (I < 1 || I + F > 31)) return DS_ERR_BAD_ARG;
    p.in_kind = f.in_kind;
    p.out_kind = f.out_kind;
    p.relu = f.relu;
    p.requant = f.requant;
    p.residual = f.residual;
    p.q.scale = float(1ll << (needs_if ? F : 0));
    p.inv_scale = 1.0f / p.q.scale;
    p.q.sign_mode = (f.in_kind == DS_IN_F32_CONV && I == 1);
    p.q.lo = p.q.hi = 0.f;
    p.rq_lo = p.rq_hi = 0;
    if (f.in_kind == DS_IN_F32_CONV || f.requant) {
        const long long lo = -(1ll << (I - 1 + F)), hi = ((1ll << (I - 1)) - 1) * (1ll << F);
        p.q.lo = float(lo);
        p.q.hi = float(hi);
        p.rq_lo = int(lo);
        p.rq_hi = int(hi);
    }
    // FP32-pipe path: needs base == 0 and every |x| <= 2^(act_bits-1) <= 2^19, and at least
    // one k-tile (<= 32 terms of magnitude <= 2^(act_bits-1) + 1) between drains.
    int ab = f.act_bits;
    if (f.in_kind == DS_IN_F32_CONV) ab = p.q.sign_mode ? F + 2 : I + F;
    if (f.in_kind == DS_IN_F32_LINEAR) ab = 0;
    use_fp = (base == 0 && ab >= 1 && ab <= 18);
    if (use_fp) {
        const long long per_term = (1ll << (ab - 1)) + 1;
        const long long terms = ((1ll << 22) - 1) / per_term;  // terms that cannot overflow
        p.flush_tiles = int(terms / 32 > 1024 ? 1024 : terms / 32);  // tiles of <= 32 terms
        if (p.flush_tiles < 1) use_fp = false;
    }
    return DS_OK;
}

int check_ptrs(const void* x, const void* packed, const void* out)
{
    if (!x || !packed || !out) return DS_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(out) & 15u) != 0) return DS_ERR_ALIGN;
    return DS_OK;
}

}  // namespace
}  // namespace ds

using namespace ds;

extern "C" int ds_linear_ex(const void* x, const int32_t* packed, const int32_t* bias, void* out, int M,
                            int K, int N, int bits, int base, const ds_fuse_t* fuse, void* stream)
{
    if (M < 0 || K <= 0 || N <= 0) return DS_ERR_BAD_ARG;
    if (M == 0) return DS_OK;
    int rc = check_ptrs(x, packed, out);
    if (rc) return rc;
    GemmParams p = {};
    p.x = x; p.packed = packed; p.bias = bias; p.out = out;
    p.M = M; p.K = K; p.N = N;
    bool fp = false;
    rc = setup_common(p, bits, base, fuse, fp);
    if (rc) return rc;
    if (p.residual && (reinterpret_cast<uintptr_t>(p.residual) & 3u)) return DS_ERR_ALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return fp ? launch_path<true, false>(p, st) : launch_path<false, false>(p, st);
}

extern "C" int ds_conv2d_ex(const void* x, const int32_t* packed, const int32_t* bias, void* out, int B,
                            int C, int H, int W, int OC, int KH, int KW, int sh, int sw, int ph, int pw,
                            int bits, int base, const ds_fuse_t* fuse, void* stream)
{
    if (B < 0 || C <= 0 || H <= 0 || W <= 0 || OC <= 0 || KH <= 0 || KW <= 0 || sh <= 0 || sw <= 0 ||
        ph < 0 || pw < 0)
        return DS_ERR_BAD_ARG;
    if (KH > 31 || KW > 31) return DS_ERR_UNSUPPORTED;
    if (H + 2 * ph < KH || W + 2 * pw < KW) return DS_ERR_BAD_ARG;
    if (B == 0) return DS_OK;
    int rc = check_ptrs(x, packed, out);
    if (rc) return rc;
    const int OH = (H + 2 * ph - KH) / sh + 1, OW = (W + 2 * pw - KW) / sw + 1;
    const long long M = (long long)B * OH * OW, Kll = (long long)C * KH * KW;
    if (M > 2147483647LL || Kll > 2147483647LL || (long long)C * H * W > 2147483647LL) return DS_ERR_RANGE;
    GemmParams p = {};
    p.x = x; p.packed = packed; p.bias = bias; p.out = out;
    p.M = int(M); p.K = int(Kll); p.N = OC;
    p.C = C; p.H = H; p.W = W; p.OC = OC; p.KH = KH; p.KW = KW;
    p.sh = sh; p.sw = sw; p.ph = ph; p.pw = pw; p.OH = OH; p.OW = OW; p.P = OH * OW;
    bool fp = false;
    rc = setup_common(p, bits, base, fuse, fp);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return fp ? launch_path<true, true>(p, st) : launch_path<false, true>(p, st);
}

extern "C" int ds_linear_i32(const int32_t* x, const int32_t* packed, const int32_t* bias, int32_t* out,
                             int M, int K, int N, int bits, int base, int act_bits, void* stream)
{
    ds_fuse_t f = {};
    f.act_bits = act_bits;
    return ds_linear_ex(x, packed, bias, out, M, K, N, bits, base, &f, stream);
}

extern "C" int ds_conv2d_i32(const int32_t* x, const int32_t* packed, const int32_t* bias, int32_t* out,
                             int B, int C, int H, int W, int OC, int KH, int KW, int sh, int sw, int ph,
                             int pw, int bits, int base, int act_bits, void* stream)
{
    ds_fuse_t f = {};
    f.act_bits = act_bits;
    return ds_conv2d_ex(x, packed, bias, out, B, C, H, W, OC, KH, KW, sh, sw, ph, pw, bits, base, &f, stream);
}
