// Shift-accumulate "GEMM" and implicit-im2col convolution for sm_100a.
//
// out[m,n] = bias[n] + sum_k term(x[m,k], w[n,k]),  term = sign * (x >> r)   (see the header)
//
// One tiled kernel serves both the linear layer (x is [M,K] row-major) and the convolution
// (x is unpadded NCHW; row m = (b,oh,ow), column k = (ic,kh,kw) is gathered on the fly, zero
// padding by predication -- the im2col matrix never exists).  Packed weight words are
// fetched from global memory and decoded once per CTA into shared memory through a small
// lookup table; the decoded sign/shift never goes back to HBM.
//
// Two arithmetic paths, both bit-exact:
//   * integer path (MODE_INT): acc += (x >> sh) * mul, a funnel shift on the integer ALU pipe
//     plus an integer multiply-add.  Valid for every int32 input, any base <= 0, and wraps
//     modulo 2^32 like the reference.  256 threads, 8x8 outputs per thread in registers.
//   * FP32-pipe path (MODE_FP): one FFMA with round-toward-minus-infinity per term.  With
//     xh = x + 0.5 and w = +-2^-r, floor(xh * w) equals (x >> r) for w > 0 and -(x >> r) - 1
//     for w < 0, because xh * w is never an integer.  Adding into an accumulator of the form
//     1.5*2^23 + A (A an integer, |A| < 2^22) makes the FMA's single rounding exactly that
//     floor.  The "-1" of every negative weight is a per-output constant that the epilogue
//     adds back.  Before |A| can reach 2^22 the accumulators are drained into per-thread
//     int32 slots in shared memory (red.shared.add), so registers hold only the float
//     accumulators.  Needs base == 0 and a bound on |x| (act_bits).  512 threads, one CTA per
//     SM, 256 output rows per CTA.
//
// Staging of x (template parameter AM):
//   AM_LINEAR    x is [M,K]; a warp reads runs of consecutive k.
//   AM_TABLE     convolution, any window: a per-tile table maps k -> (offset, kh, kw).
//   AM_ROW + KW  convolution with a KW-wide window and a k-tile made of whole (ic,kh) rows:
//                one table entry and one validity test per row, KW loads at constant
//                offsets.  This is the cheap path used by 1x1, 3x3, 5x5 and 7x7 windows.
#include "ds_gemm_common.cuh"

namespace ds {
namespace {

template <int NT, int TMG, int TNG, int TN, int BKT, int MODE>
struct Smem {
    static constexpr bool FP = MODE == MODE_FP;
    static constexpr int BM = TMG * kTM;
    static constexpr int BN = TNG * TN;
    static constexpr int AP = BM + 4;
    // Every member that is read with 8- or 16-byte loads sits at a multiple of 16 bytes.
    alignas(16) float a[2][BKT][AP];  // FP: x + 0.5 as float; integer path: x (int bits)
    alignas(16) float b[2][BKT][BN];  // FP: +-2^-r; integer path: shift amounts (int bits)
    alignas(16) KEntry ktab[2][BKT];
    alignas(16) int bm[FP ? 1 : 2][FP ? 1 : BKT][FP ? 1 : BN];  // integer path: multipliers
    int lut0[256];           // decoded weight per field value: FP float bits / integer shift
    int lut1[FP ? 1 : 256];  // integer path: multiplier
    int negc[BN];            // FP: negative weights per output column
    int accs[FP ? kTM * TN * NT : 1];  // FP: drained accumulators, [slot][thread]
};

// ---------------------------------------------------------------------------------------------
template <int NT, int TMG, int TNG, int TN, int BKT, int MODE, int AM>
__global__ void __launch_bounds__(NT, MODE == MODE_FP ? 1 : 2) gemm_kernel(const GemmParams p)
{
    using S = Smem<NT, TMG, TNG, TN, BKT, MODE>;
    constexpr bool FP = MODE == MODE_FP;
    constexpr bool CONV = AM != AM_LINEAR;
    constexpr bool ROW = AM >= 1;
    constexpr int KW = ROW ? AM : 1;
    constexpr int BM = S::BM, BN = S::BN;
    constexpr int EW = (BN * (BKT / 4) + NT - 1) / NT;  // words per thread (num >= 4)
    static_assert(TMG * TNG == NT, "thread grid");
    static_assert(TN == 4 || TN == 8, "TN");
    static_assert((BN & (BN - 1)) == 0, "BN power of two");
    static_assert(TMG % 8 == 0 && TNG % 8 == 0, "warp footprint");
    static_assert(offsetof(S, ktab) % 16 == 0 && offsetof(S, b) % 16 == 0 && offsetof(S, bm) % 16 == 0, "alignment");

    extern __shared__ __align__(16) unsigned char smem_raw[];
    S& s = *reinterpret_cast<S*>(smem_raw);

    const int t = threadIdx.x;
    const int m0 = blockIdx.x * BM;
    const int n0 = blockIdx.y * BN;
    if (p.gate && *p.gate != p.gate_want) return;  // the other arithmetic path serves this input
    // A warp covers 8 x 4 thread tiles: 8 along the direction in which the output is contiguous
    // (m for the NCHW convolution output, n for the [M,N] linear output), so that both operand
    // fragments come from few shared-memory wavefronts and stores fill whole sectors.
    const int lane = t & 31, warp = t >> 5;
    int tm, tn;
    if (CONV) {
        constexpr int WMG = TMG / 8;
        tm = (warp % WMG) * 8 + (lane & 7);
        tn = (warp / WMG) * 4 + (lane >> 3);
    } else {
        constexpr int WNG = TNG / 8;
        tn = (warp % WNG) * 8 + (lane & 7);
        tm = (warp / WNG) * 4 + (lane >> 3);
    }

    // ---- per-thread staging geometry -------------------------------------------------------
    // CONV: one row m_local = t % BM of the tile; `a_k` = t / BM picks every (NT / BM)-th column
    //       (table mode) or (ic,kh) row (row mode) of the k-tile.
    // LINEAR: one column k_local = t % KL, rows m_local = t / KL + (NT / KL) * e, KL = 32 or 16
    //         (k is contiguous in x, so a warp reads whole sectors).
    constexpr int KL = (BKT > 16) ? 32 : 16;
    constexpr int A_MSTEP = NT / KL;
    constexpr int A_KSTEP = (NT >= BM) ? NT / BM : 1;
    // row mode: a k-tile holds a multiple of A_KSTEP rows; UNITS rows per thread per tile
    constexpr int UNITS = (BKT / (KW * A_KSTEP)) > 0 ? (BKT / (KW * A_KSTEP)) : 1;
    constexpr int A_ELEMS = ROW ? UNITS * KW : (CONV ? (BKT + A_KSTEP - 1) / A_KSTEP : (BM + A_MSTEP - 1) / A_MSTEP);
    static_assert(A_ELEMS <= 16, "staging registers");
    static_assert(!CONV || NT >= BM, "one staging thread per row");
    const int a_m = CONV ? (t % BM) : (t / KL);
    const int a_k = CONV ? (t / BM) : (t % KL);

    const int32_t* xi = static_cast<const int32_t*>(p.x);
    long long x_base = 0;   // LINEAR: element offset of (m0 + a_m, a_k)
    const char* x_pix = reinterpret_cast<const char*>(p.x);  // CONV: address of (b, 0, ih0, iw0); may lie
                                                             // outside the tensor, only valid taps are read
    uint32_t rowmask = 0, colmask = 0;  // CONV: valid kh / kw; LINEAR: rowmask bit e = row valid
    if (CONV) {
        const int m = m0 + a_m;
        if (m < p.M) {
            const int b = m / p.P, pp = m - b * p.P;
            const int oh = pp / p.OW, ow = pp - oh * p.OW;
            const int ih0 = oh * p.sh - p.ph, iw0 = ow * p.sw - p.pw;
            for (int kh = 0; kh < p.KH; ++kh)
                if (unsigned(ih0 + kh) < unsigned(p.H)) rowmask |= 1u << kh;
            for (int kw = 0; kw < p.KW; ++kw)
                if (unsigned(iw0 + kw) < unsigned(p.W)) colmask |= 1u << kw;
            x_pix += ((long long)b * p.C * p.H * p.W + (long long)ih0 * p.W + iw0) * 4;
        }
    } else {
        x_base = (long long)(m0 + a_m) * p.K + a_k;
#pragma unroll
        for (int e = 0; e < A_ELEMS; ++e)
            if (a_m + e * A_MSTEP < BM && m0 + a_m + e * A_MSTEP < p.M) rowmask |= 1u << e;
        if (a_k >= p.bk) rowmask = 0;
    }

    // ---- decode table, accumulators ------------------------------------------------------------
    for (int f = t; f < (1 << p.dec.fw); f += NT) {
        if (FP) {
            int neg;
            s.lut0[f] = __float_as_int(decode_f32(uint32_t(f), p.dec, true, neg));
        } else {
            int shv, mul;
            decode_int(uint32_t(f), p.dec, true, shv, mul);
            s.lut0[f] = shv;
            s.lut1[f] = mul;
        }
    }
    int acc[FP ? 1 : kTM][FP ? 1 : TN];
    float accf[FP ? kTM : 1][FP ? TN : 1];
    if (FP) {
#pragma unroll
        for (int i = 0; i < kTM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                accf[i][j] = kMagic;
                s.accs[(i * TN + j) * NT + t] = 0;
            }
        for (int i = t; i < BN; i += NT) s.negc[i] = 0;
    } else {
#pragma unroll
        for (int i = 0; i < kTM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) acc[i][j] = 0;
    }

    // ---- staging helpers -------------------------------------------------------------------
    int a_reg[A_ELEMS];
    uint32_t w_reg[EW];
    const int nwords = BN * p.kt_words;
    // Word e of this thread: column n = wi % BN, word jw = wi / BN of the k-tile.
    const int32_t* w_ptr[EW];  // address of word jw of tile 0, null if the thread has no such word
    int w_jw[EW];
#pragma unroll
    for (int e = 0; e < EW; ++e) {
        const int wi = t + e * NT;
        const int n = wi & (BN - 1);
        w_jw[e] = wi / BN;
        w_ptr[e] = (wi < nwords && n0 + n < p.N) ? p.packed + (long long)(n0 + n) * p.dec.row_len + w_jw[e] : nullptr;
    }

    auto fill_ktab = [&](int tile, int buf) {
        if (!CONV || t >= BKT) return;
        KEntry e;
        e.pad = 0;
        e.off = 0;
        e.kh = 31;
        e.kw = 0;
        if (ROW) {
            const int row = tile * p.rows_per_tile + t;  // global (ic,kh) row index
            if (t < p.rows_per_tile && row < p.C * p.KH) {
                const int ic = magic_div(row, p.magic_kh);
                e.kh = row - ic * p.KH;
                e.off = (ic * p.H * p.W + e.kh * p.W) * 4;
            }
        } else {
            const int k = tile * p.bk + t;
            if (t < p.bk && k < p.K) {
                const int ic = magic_div(k, p.magic_khw);
                const int tap = k - ic * (p.KH * p.KW);
                e.kh = magic_div(tap, p.magic_kw);
                e.kw = tap - e.kh * p.KW;
                e.off = (ic * p.H * p.W + e.kh * p.W + e.kw) * 4;
            }
        }
        s.ktab[buf][t] = e;
    };

    // Raw fetch of tile `tile` into registers.  fp32 inputs keep their bits; positions outside
    // the image or the matrix carry a marker so that stash() stores the integer 0 there
    // without quantising it.
    auto fetch = [&](int tile, int buf) {
        const int padv = p.pad_raw;
        if (ROW) {
#pragma unroll
            for (int u = 0; u < UNITS; ++u) {
                const int r = a_k + u * A_KSTEP;  // < BKT / KW by construction of UNITS
                const int2 e = *reinterpret_cast<const int2*>(&s.ktab[buf][r]);
                const bool rv = (rowmask >> e.y) & 1u;
                const int* rowp = reinterpret_cast<const int*>(x_pix + e.x);
#pragma unroll
                for (int kw = 0; kw < KW; ++kw) {
                    int v = padv;
                    if (rv && (colmask & (1u << kw)) && DS_X_OK(p, rowp + kw, 4)) v = __ldg(rowp + kw);
                    a_reg[u * KW + kw] = v;
                }
            }
        } else if (CONV) {
#pragma unroll
            for (int e = 0; e < A_ELEMS; ++e) {
                const int kl = a_k + e * A_KSTEP;
                int v = padv;
                if (kl < BKT) {
                    const int4 ke = *reinterpret_cast<const int4*>(&s.ktab[buf][kl]);
                    if (((rowmask >> ke.y) & (colmask >> ke.z) & 1u) != 0u && DS_X_OK(p, x_pix + ke.x, 4))
                        v = __ldg(reinterpret_cast<const int*>(x_pix + ke.x));
                }
                a_reg[e] = v;
            }
        } else {
            const int32_t* src = xi + (x_base + (long long)tile * p.bk);
            const bool ktail = (tile * p.bk + a_k) >= p.K;
#pragma unroll
            for (int e = 0; e < A_ELEMS; ++e) {
                int v = padv;
                if (((rowmask >> e) & 1u) && !ktail && DS_X_OK(p, src + (long long)e * A_MSTEP * p.K, 4)) v = __ldg(src + (long long)e * A_MSTEP * p.K);
                a_reg[e] = v;
            }
        }
        const int w0 = tile * p.kt_words;
#pragma unroll
        for (int e = 0; e < EW; ++e) {
            uint32_t w = 0;
            if (w_ptr[e] && w0 + w_jw[e] < p.dec.row_len && DS_W_OK(p, w_ptr[e] + w0, 4)) w = uint32_t(__ldg(w_ptr[e] + w0));
            w_reg[e] = w;
        }
    };

    // Convert and store the x registers into shared buffer `buf`.  LAST: the tile may reach past
    // K, where x is stored as 0 (see decode_word).
    auto stash_a = [&](auto ink_tag, auto last_tag, int tile, int buf) {
        constexpr int INK = decltype(ink_tag)::value;
        constexpr bool LAST = decltype(last_tag)::value;
        const int k0 = tile * p.bk;
        if (ROW) {
#pragma unroll
            for (int u = 0; u < UNITS; ++u) {
                const int r = a_k + u * A_KSTEP;
#pragma unroll
                for (int kw = 0; kw < KW; ++kw) {
                    const int kl = r * KW + kw;
                    float o = operand_of<FP, INK>(p, a_reg[u * KW + kw]);
                    if (LAST && k0 + kl >= p.K) o = 0.f;
                    s.a[buf][kl][a_m] = o;
                }
            }
        } else {
#pragma unroll
            for (int e = 0; e < A_ELEMS; ++e) {
                const int kl = CONV ? (a_k + e * A_KSTEP) : a_k;
                const int ml = CONV ? a_m : (a_m + e * A_MSTEP);
                if (kl < BKT && ml < BM) {
                    float o = operand_of<FP, INK>(p, a_reg[e]);
                    if (LAST && k0 + kl >= p.K) o = 0.f;
                    s.a[buf][kl][ml] = o;
                }
            }
        }
    };

    // Decode the NUM fields of each of this thread's words into the weight tile.  Tail slots
    // (k >= K) of the last word decode like any field; the matching x values are stored as 0 so
    // they add nothing, and the epilogue takes their share out of the negative-weight count.
    const uint32_t fmask = (1u << p.dec.fw) - 1u;
    auto decode_words = [&](auto num_tag, int buf) {
        constexpr int NUM = decltype(num_tag)::value;
#pragma unroll
        for (int e = 0; e < EW; ++e) {
            if (!w_ptr[e]) continue;
            const int n = (t + e * NT) & (BN - 1);
            float* dst = &s.b[buf][w_jw[e] * NUM][n];
            int* dstm = &s.bm[FP ? 0 : buf][FP ? 0 : w_jw[e] * NUM][FP ? 0 : n];
            uint32_t w = w_reg[e];
            int negs = 0;
#pragma unroll
            for (int i = 0; i < NUM; ++i) {
                const uint32_t f = w & fmask;
                w >>= p.dec.fw;
                const int v0 = s.lut0[f];
                dst[i * BN] = __int_as_float(v0);
                if (FP) negs += int(uint32_t(v0) >> 31);
                else dstm[i * BN] = s.lut1[f];
            }
            if (FP && negs) atomicAdd(&s.negc[n], negs);
        }
    };

    auto stash = [&](int tile, int buf) {
        const bool last = tile + 1 >= p.ntiles;
        with_input_kind(p, [&](auto ink_tag) {
            if (last) stash_a(ink_tag, std::true_type(), tile, buf);
            else stash_a(ink_tag, std::false_type(), tile, buf);
        });
        switch (p.dec.num) {
            case 4: decode_words(std::integral_constant<int, 4>(), buf); break;
            case 5: decode_words(std::integral_constant<int, 5>(), buf); break;
            case 6: decode_words(std::integral_constant<int, 6>(), buf); break;
            case 8: decode_words(std::integral_constant<int, 8>(), buf); break;
            case 10: decode_words(std::integral_constant<int, 10>(), buf); break;
            default: decode_words(std::integral_constant<int, 16>(), buf); break;
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

    // FP path: move the float accumulators (raw bits, kMagicBits + A) into this thread's
    // shared int32 slots and restart them; the epilogue removes ndrains * kMagicBits.
    int ndrains = 0;
    auto drain = [&]() {
#pragma unroll
        for (int i = 0; i < kTM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                red_shared_add(&s.accs[(i * TN + j) * NT + t], __float_as_int(accf[i][j]));
                accf[i][j] = kMagic;
            }
        ++ndrains;
    };

    // ---- main loop: two shared buffers, register prefetch, one barrier per tile --------------
    // gridDim.z > 1 (linear layers, plain epilogue only): CTA z takes k-tiles [t_begin, t_end)
    const int t_begin = blockIdx.z * p.tiles_per_split;
    const int t_end = min(p.ntiles, t_begin + p.tiles_per_split);
    fill_ktab(t_begin, 0);
    __syncthreads();
    fetch(t_begin, 0);
    fill_ktab(t_begin + 1, 1);
    stash(t_begin, 0);
    __syncthreads();
    int since = 0;
    for (int tile = t_begin; tile < t_end; ++tile) {
        const int buf = (tile - t_begin) & 1;
        const bool more = tile + 1 < t_end;
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
    if (FP) drain();  // each thread reads back only its own slots below

    // ---- epilogue -----------------------------------------------------------------------------
    if (gridDim.z > 1) {
        // split along K: integer adds into the zeroed output commute, the bias goes in once; on the
        // FP32-pipe path every CTA adds the count of the negative weights it decoded (the slots
        // past K belong to the range that holds the last k-tile)
        reduce_tile<TN, CONV>(
            p, m0, n0, tm, tn, BM, BN,
            [&](int i, int j, long long) -> int {
                if (FP) return s.accs[(i * TN + j) * NT + t] - ndrains * kMagicBits;
                return acc[FP ? 0 : i][FP ? 0 : j];
            },
            [&](int col) -> int {
                int c = (blockIdx.z == 0 && p.bias && n0 + col < p.N) ? __ldg(p.bias + n0 + col) : 0;
                if (FP) c += s.negc[col] - (t_end == p.ntiles ? p.tail_neg : 0);
                return c;
            });
        return;
    }
    store_tile<TN, CONV>(
        p, m0, n0, tm, tn, BM, BN,
        [&](int i, int j, long long) -> int {
            if (FP) return s.accs[(i * TN + j) * NT + t] - ndrains * kMagicBits;
            return acc[FP ? 0 : i][FP ? 0 : j];
        },
        [&](int col) -> int { return FP ? (s.negc[col] - p.tail_neg) : 0; });
}

// ---------------------------------------------------------------------------------------------
// Chooses the k-tile: `bk` values of k per tile, a multiple of num (whole packed words) and, in
// row mode, of A_KSTEP*KW (whole rows, split evenly over the staging threads of one x row).
template <int BKT, int AM, int A_KSTEP>
bool choose_tile(GemmParams& p)
{
    constexpr int KW = AM >= 1 ? AM : 1;
    int best = 0;
    for (int bk = BKT; bk >= 2 && !best; --bk) {
        if (bk % p.dec.num) continue;
        if (AM >= 1 && bk % (A_KSTEP * KW)) continue;
        best = bk;
    }
    if (!best) return false;
    p.bk = best;
    p.kt_words = best / p.dec.num;
    p.rows_per_tile = best / KW;
    p.ntiles = (p.dec.row_len + p.kt_words - 1) / p.kt_words;
    // Every slot from K to the end of the last tile decodes from a zero field, i.e. as -2^0.
    p.tail_neg = p.ntiles * p.bk - p.K;
    return true;
}

template <int NT, int TMG, int TNG, int TN, int BKT, int MODE, int AM>
int launch_cfg(GemmParams p, cudaStream_t st)
{
    using S = Smem<NT, TMG, TNG, TN, BKT, MODE>;
    constexpr int BM = S::BM, BN = S::BN;
    if (!choose_tile<BKT, AM, (NT >= BM ? NT / BM : 1)>(p)) return DS_ERR_UNSUPPORTED;
    if (MODE == MODE_FP) {
        p.flush_tiles /= p.bk;  // setup_common left the number of terms that cannot overflow
        if (p.flush_tiles < 1) return DS_ERR_UNSUPPORTED;
        if (p.flush_tiles > 4096) p.flush_tiles = 4096;
    }
    if (p.prepare_only) return DS_OK;  // this kernel decodes the packed words itself
    auto kern = gemm_kernel<NT, TMG, TNG, TN, BKT, MODE, AM>;
    const size_t smem = sizeof(S);
    static bool done[kMaxDevices];  // per instantiation and device
    const int dev = device_slot();
    if (dev < 0) return DS_ERR_CUDA;
    bool& attr_done = done[dev];
    if (!attr_done) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) {
            cudaGetLastError();
            return DS_ERR_CUDA;
        }
        attr_done = true;
    }
    const long long gx = ((long long)p.M + BM - 1) / BM, gy = (p.N + BN - 1) / BN;
    if (gx > 2147483647LL || gy > 65535) return DS_ERR_RANGE;
    p.splits = 1;
    p.tiles_per_split = p.ntiles;
    const bool plain = p.out_kind == DS_OUT_I32 && !p.relu && !p.requant && !p.round_f32 && !p.residual;
    if (AM == AM_LINEAR && plain && !p.gate && gx * gy < 148) {
        // Few output tiles (small batch): split K across gridDim.z until two CTAs per SM have work;
        // the partial sums meet through integer atomics in the zeroed output.
        int splits = 1;
        while (splits < 16 && gx * gy * splits < 2 * 148 && p.ntiles / (splits * 2) >= 4) splits *= 2;
        p.tiles_per_split = (p.ntiles + splits - 1) / splits;
        p.splits = (p.ntiles + p.tiles_per_split - 1) / p.tiles_per_split;
        if (p.splits > 1 && cudaMemsetAsync(p.out, 0, size_t(p.M) * size_t(p.N) * 4, st) != cudaSuccess) return DS_ERR_CUDA;
    }
    kern<<<dim3((unsigned)gx, (unsigned)gy, (unsigned)p.splits), NT, smem, st>>>(p);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
}

// Few output channels and enough rows to fill the GPU with 512-row tiles: the 512 x 32 tile of
// the block kernel beats the 256 x 64 tile of the warp-specialised one, half of which would be idle.
inline bool narrow_tile(const GemmParams& p) { return p.N <= 32 && p.M >= 148 * 512; }

// Tile shape by output width.  FP path: 256 rows x 128 or 64 columns, 512 threads.
// Integer path: 128 x 128, 256 x 64 or 256 x 32, 256 threads.
template <int AM>
int launch_am(const GemmParams& p, bool fp, cudaStream_t st)
{
    if (fp) {
        // The warp-specialised kernel takes convolutions and, through 16-byte loads along k, linear
        // layers whose rows are whole 16-byte groups; other linear layers stay on the block kernel.
        if (AM == AM_LINEAR) {
            if (p.K % 4 == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15u) == 0 && p.N > 32) {
                const int rc = launch_ws(p, AM_LINEAR, st);
                if (rc != DS_ERR_UNSUPPORTED) return rc;
            }
        } else {
            // Few output channels: a 512 x 32 tile wastes no columns where the warp-specialised
            // kernel would compute 64.
            if (narrow_tile(p)) {
                const int rc = launch_cfg<512, 64, 8, 4, 16, MODE_FP, AM>(p, st);
                if (rc != DS_ERR_UNSUPPORTED) return rc;
            }
            const int rc = launch_ws(p, AM, st);
            if (rc != DS_ERR_UNSUPPORTED) return rc;
        }
        if (p.N > 64) return launch_cfg<512, 32, 16, 8, 28, MODE_FP, AM>(p, st);
        return launch_cfg<512, 32, 16, 4, 28, MODE_FP, AM>(p, st);
    }
    if (p.N > 64) return launch_cfg<256, 16, 16, 8, 20, MODE_INT, AM>(p, st);
    if (p.N > 32) return launch_cfg<256, 32, 8, 8, 16, MODE_INT, AM>(p, st);
    return launch_cfg<256, 32, 8, 4, 16, MODE_INT, AM>(p, st);
}

int launch_conv(const GemmParams& p, bool fp, cudaStream_t st)
{
    int rc = DS_ERR_UNSUPPORTED;
    switch (p.KW) {  // row mode where the window width has an instantiation and a k-tile exists
        case 1: rc = launch_am<1>(p, fp, st); break;
        case 3:
            // stride 1 and padding 1 along W, rows of whole 16-byte groups: four pixels per load
            if (fp && !narrow_tile(p) && p.sw == 1 && p.pw == 1 && p.W % 4 == 0 &&
                (reinterpret_cast<uintptr_t>(p.x) & 15u) == 0) {
                rc = launch_ws(p, AM_QUAD3, st);
                if (rc != DS_ERR_UNSUPPORTED) break;
            }
            if (fp && !narrow_tile(p) && p.sw == 1 && p.pw == 1 && p.W % 2 == 0 &&
                (reinterpret_cast<uintptr_t>(p.x) & 7u) == 0) {  // two pixels per 8-byte load
                rc = launch_ws(p, AM_PAIR3, st);
                if (rc != DS_ERR_UNSUPPORTED) break;
            }
            rc = launch_am<3>(p, fp, st);
            break;
        case 5: rc = launch_am<5>(p, fp, st); break;
        case 7:
            // stride 2 and padding 3 along W, rows of whole 32-byte groups: four output pixels per thread
            if (fp && !narrow_tile(p) && p.sw == 2 && p.pw == 3 && p.W % 8 == 0 && p.OW * 2 == p.W &&
                (reinterpret_cast<uintptr_t>(p.x) & 15u) == 0) {
                rc = launch_ws(p, AM_S2K7, st);
                if (rc != DS_ERR_UNSUPPORTED) break;
            }
            rc = launch_am<7>(p, fp, st);
            break;
        default: break;
    }
    if (rc == DS_ERR_UNSUPPORTED) rc = launch_am<AM_TABLE>(p, fp, st);
    return rc;
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
    if (f.in_kind < 0 || f.in_kind > 3 || f.out_kind < 0 || f.out_kind > 1) return DS_ERR_BAD_ARG;
    const int I = f.act_integer_bits, F = f.act_fraction_bits;
    const bool in_clamp = f.in_kind == DS_IN_I32_CLAMP;
    const bool needs_if = f.in_kind != DS_IN_I32 || f.out_kind != DS_OUT_I32 || f.requant;
    if (needs_if && (F < 0 || F > 30)) return DS_ERR_BAD_ARG;
    if ((f.in_kind == DS_IN_F32_CONV || f.requant || in_clamp) && (I < 1 || I + F > 32)) return DS_ERR_BAD_ARG;
    p.in_kind = f.in_kind;
    p.out_kind = f.out_kind;
    p.relu = f.relu;
    p.requant = f.requant;
    p.round_f32 = f.round_f32;
    p.splits = 1;
    // workspace: kWorkspaceCounters arrival counters, then (optionally) room for partial sums
    p.counters = static_cast<int*>(f.workspace);
    p.counter_slots = f.workspace ? f.workspace_bytes / 4 : 0;
    p.partials = nullptr;
    p.partial_bytes = 0;
    if (p.counter_slots > kWorkspaceCounters) {
        p.partials = p.counters + kWorkspaceCounters;
        p.partial_bytes = f.workspace_bytes - (long long)kWorkspaceCounters * 4;
        p.counter_slots = kWorkspaceCounters;
    }
    if (p.counter_slots > kWorkspaceGateSlot) p.counter_slots = kWorkspaceGateSlot;  // the last word is the range flag
    p.wd = nullptr;
    p.negpre = nullptr;
    p.npad = 0;
    p.prepared = f.prepared;
    p.prepared_bytes = f.prepared ? f.prepared_bytes : 0;
    if (f.prepared && ((reinterpret_cast<uintptr_t>(f.prepared) & 15u) || f.prepared_bytes < 0)) return DS_ERR_BAD_ARG;
    p.full_units = p.tail_first = p.tail_items = 0;
    p.tail_splits = 1;
    p.tail_tps = 0;
    if (f.workspace && ((reinterpret_cast<uintptr_t>(f.workspace) & 3u) || f.workspace_bytes < 0)) return DS_ERR_BAD_ARG;
    p.residual = f.residual;
    p.q.scale = float(1ll << (needs_if ? F : 0));
    p.inv_scale = 1.0f / p.q.scale;
    const bool uses_rtf = f.in_kind == DS_IN_F32_CONV || f.requant || in_clamp;
    const bool sign_mode = uses_rtf && I == 1;  // round_to_fixed(x, 1, F) = sign(x) - 1
    p.q.sign_mode = sign_mode ? 1 : 0;
    p.q.lo = p.q.hi = 0.f;
    p.rq_lo = p.rq_hi = p.rq_add = 0;
    p.rq_mul = 1;
    if (sign_mode) {
        // codes {-2^(F+1), -2^F, 0} for x < 0, x == 0, x > 0
        p.q.lo = -float(2ll << F);
        p.rq_lo = -1;
        p.rq_hi = 1;
        p.rq_mul = int(1u << F);
        p.rq_add = -p.rq_mul;
    } else if (uses_rtf) {
        const long long lo = -(1ll << (I - 1 + F)), hi = ((1ll << (I - 1)) - 1) * (1ll << F);
        p.q.lo = float(lo);
        p.q.hi = float(hi);
        p.rq_lo = int(lo);
        p.rq_hi = int(hi);
    }
    p.pad_raw = (f.in_kind == DS_IN_I32) ? 0 : (in_clamp ? (sign_mode ? 1 : 0) : kPadMarker);
    p.in_mul2 = int(2u * unsigned(p.rq_mul));
    p.in_add2 = int(2u * unsigned(p.rq_add) + unsigned(kHalfMagicBits + 1));
    // FP32-pipe path: needs base == 0, every |x| <= 2^(act_bits-1) <= 2^17, and room for at
    // least one k-tile of terms (each of magnitude <= 2^(act_bits-1) + 1) between drains.
    int ab = f.act_bits == DS_ACT_BITS_AUTO ? 0 : f.act_bits;
    if (f.in_kind == DS_IN_F32_CONV || in_clamp) ab = sign_mode ? F + 2 : I + F;
    if (f.in_kind == DS_IN_F32_LINEAR) ab = 0;
    use_fp = (base == 0 && ab >= 1 && ab <= 18);
    p.flush_tiles = 0;
    if (use_fp) {
        const long long per_term = (1ll << (ab - 1)) + 1;
        const long long terms = ((1ll << 22) - 1) / per_term;  // terms that cannot overflow
        p.flush_tiles = int(terms > (1 << 20) ? (1 << 20) : terms);  // divided by bk at launch
        if (terms < 28) use_fp = false;
    }
    return DS_OK;
}

// Sets *flag to 1 if any |x| exceeds `limit` (the flag was zeroed before).  One pass, 16-byte loads
// for the aligned bulk.
__global__ void __launch_bounds__(256) range_kernel(const int* __restrict__ x, long long n, int limit, int* flag)
{
    bool over = false;
    const long long n4 = ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) ? n / 4 : 0;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
        const int4 v = __ldg(reinterpret_cast<const int4*>(x) + i);
        over |= (v.x > limit) | (v.x < -limit) | (v.y > limit) | (v.y < -limit) | (v.z > limit) | (v.z < -limit) |
                (v.w > limit) | (v.w < -limit);
    }
    for (long long i = 4 * n4 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int v = __ldg(x + i);
        over |= (v > limit) | (v < -limit);
    }
    if (over) *flag = 1;
}

// act_bits = DS_ACT_BITS_AUTO: can this call be served by the two gated launches?  It needs int32
// input without a promise, right shifts only and a workspace (whose last counter word is the flag).
bool auto_range(const ds_fuse_t* fuse, int base)
{
    return fuse && fuse->act_bits == DS_ACT_BITS_AUTO && fuse->in_kind == DS_IN_I32 && base == 0 && fuse->workspace &&
           fuse->workspace_bytes >= (long long)kWorkspaceCounters * 4;
}

// Zeroes the flag and measures the range of x on `st`; returns the flag's device address.
int* launch_range(const void* x, long long n, const ds_fuse_t* fuse, cudaStream_t st)
{
    int* flag = static_cast<int*>(fuse->workspace) + kWorkspaceGateSlot;
    if (cudaMemsetAsync(flag, 0, sizeof(int), st) != cudaSuccess) return nullptr;
    const long long want = (n / 4 + 255) / 256 + 1;
    range_kernel<<<unsigned(want > 148 * 16 ? 148 * 16 : want), 256, 0, st>>>(static_cast<const int*>(x), n, 1 << 15, flag);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? flag : nullptr;
}

// Checked build: the extents the kernels test their addresses against.
long long g_check_shrink_x = 0;  // ds_bounds_debug_shrink_x: bytes taken off the declared extent of x

void set_check_extents(GemmParams& p, long long x_elems)
{
    p.chk_x_bytes = x_elems * 4 - g_check_shrink_x;
    p.chk_w_bytes = (long long)p.N * p.dec.row_len * 4;
    p.chk_o_bytes = (long long)p.M * p.N * 4;
    p.chk_status = bounds_status_ptr();
}

int check_ptrs(const void* x, const void* packed, const void* out)
{
    if (!x || !packed || !out) return DS_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(out) & 15u) != 0) return DS_ERR_ALIGN;
    return DS_OK;
}

unsigned magic_of(int d) { return d == 1 ? 0u : unsigned(((1ull << 32) + unsigned(d) - 1) / unsigned(d)); }

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
    if (auto_range(fuse, base) && M > 64) {
        // measure the range once, then launch both arithmetic paths gated on the result
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        int* flag = launch_range(x, (long long)M * K, fuse, st);
        if (!flag) return DS_ERR_CUDA;
        ds_fuse_t f = *fuse;
        for (int pass = 0; pass < 2; ++pass) {
            f.act_bits = pass == 0 ? 16 : 0;
            GemmParams g = {};
            g.x = x; g.packed = packed; g.bias = bias; g.out = out;
            g.M = M; g.K = K; g.N = N;
            bool gfp = false;
            rc = setup_common(g, bits, base, &f, gfp);
            if (rc) return rc;
            if (g.residual && (reinterpret_cast<uintptr_t>(g.residual) & 3u)) return DS_ERR_ALIGN;
            g.prepared = nullptr;
            g.prepared_bytes = 0;
            g.gate = flag;
            g.gate_want = pass;
            set_check_extents(g, (long long)M * K);
            rc = launch_am<AM_LINEAR>(g, gfp, st);
            if (rc) return rc;
        }
        return DS_OK;
    }
    GemmParams p = {};
    p.x = x; p.packed = packed; p.bias = bias; p.out = out;
    p.M = M; p.K = K; p.N = N;
    bool fp = false;
    rc = setup_common(p, bits, base, fuse, fp);
    if (rc) return rc;
    if (p.residual && (reinterpret_cast<uintptr_t>(p.residual) & 3u)) return DS_ERR_ALIGN;
    p.prepared = nullptr;  // weights expanded ahead of time exist for convolutions only
    p.prepared_bytes = 0;
    set_check_extents(p, (long long)M * K);
    // Small batches run on the integer pipe: up to 16 rows on the kernel that splits K across the
    // lanes of a warp, up to 64 rows on the block kernel with a 64-row tile (K split across CTAs
    // when nothing is fused into the epilogue).
    // The 64-row tile also serves larger batches on the integer path while 128-row tiles would leave
    // more than half of the SMs without one (a 256 x 512 -> 1000 classifier: 32 CTAs instead of 16).
    const long long tiles128 = ((long long)(M + 127) / 128) * ((N + 127) / 128);
    if (M <= 16) return launch_small_linear(p, static_cast<cudaStream_t>(stream));
    const long long tiles256 = ((long long)(M + 255) / 256) * ((N + 127) / 128);
    if (fp && (M <= 64 || tiles256 * 4 < 148)) {
        // a caller that bounds its activations gets the same tile on the FP32 pipe (also larger
        // batches whose 256-row tiles would cover less than a quarter of the SMs)
        const int rc = launch_cfg<256, 8, 32, 4, 16, MODE_FP, AM_LINEAR>(p, static_cast<cudaStream_t>(stream));
        if (rc != DS_ERR_UNSUPPORTED) return rc;
    }
    if (M <= 64 || (!fp && tiles128 * 2 < 148)) {
        const int rc = launch_cfg<256, 8, 32, 4, 16, MODE_INT, AM_LINEAR>(p, static_cast<cudaStream_t>(stream));
        if (rc != DS_ERR_UNSUPPORTED) return rc;
    }
    return launch_am<AM_LINEAR>(p, fp, static_cast<cudaStream_t>(stream));
}

namespace ds {
namespace {

// Shared body of ds_conv2d_ex and ds_conv2d_prepare.
int conv2d_run(const void* x, const int32_t* packed, const int32_t* bias, void* out, int B, int C, int H, int W,
               int OC, int KH, int KW, int sh, int sw, int ph, int pw, int bits, int base, const ds_fuse_t* fuse,
               void* stream, long long* needed_out)
{
    const bool prepare = needed_out != nullptr;
    if (B < 0 || C <= 0 || H <= 0 || W <= 0 || OC <= 0 || KH <= 0 || KW <= 0 || sh <= 0 || sw <= 0 ||
        ph < 0 || pw < 0)
        return DS_ERR_BAD_ARG;
    if (KH > 31 || KW > 31) return DS_ERR_UNSUPPORTED;
    if (H + 2 * ph < KH || W + 2 * pw < KW) return DS_ERR_BAD_ARG;
    if (B == 0) return DS_OK;
    if (prepare) {
        if (!packed || (reinterpret_cast<uintptr_t>(packed) & 3u)) return DS_ERR_BAD_ARG;
    } else {
        const int rc = check_ptrs(x, packed, out);
        if (rc) return rc;
    }
    const int OH = (H + 2 * ph - KH) / sh + 1, OW = (W + 2 * pw - KW) / sw + 1;
    const long long M = (long long)B * OH * OW, Kll = (long long)C * KH * KW;
    if (M > 2147483647LL || Kll > 2147483647LL || (long long)C * H * W > 2147483647LL) return DS_ERR_RANGE;
    if ((long long)C * H * W * 4 >= (1ll << 31)) return DS_ERR_RANGE;  // int byte offsets inside one image
    if (Kll * KH * KW >= (1ll << 32)) return DS_ERR_RANGE;                 // exactness of the magic division
    GemmParams p = {};
    p.x = x; p.packed = packed; p.bias = bias; p.out = out;
    p.M = int(M); p.K = int(Kll); p.N = OC;
    p.C = C; p.H = H; p.W = W; p.OC = OC; p.KH = KH; p.KW = KW;
    p.sh = sh; p.sw = sw; p.ph = ph; p.pw = pw; p.OH = OH; p.OW = OW; p.P = OH * OW;
    p.magic_khw = magic_of(KH * KW);
    p.magic_kw = magic_of(KW);
    p.magic_kh = magic_of(KH);
    if (!prepare && auto_range(fuse, base)) {
        // measure the range once, then launch both arithmetic paths gated on the result
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        int* flag = launch_range(x, (long long)B * C * H * W, fuse, st);
        if (!flag) return DS_ERR_CUDA;
        ds_fuse_t f = *fuse;
        for (int pass = 0; pass < 2; ++pass) {
            f.act_bits = pass == 0 ? 16 : 0;
            f.prepared = nullptr;   // expanded ahead of time for one path only: not used here
            f.prepared_bytes = 0;
            GemmParams g = p;
            bool gfp = false;
            const int rc = setup_common(g, bits, base, &f, gfp);
            if (rc) return rc;
            g.gate = flag;
            g.gate_want = pass;
            set_check_extents(g, (long long)B * C * H * W);
            const int rl = launch_conv(g, gfp, st);
            if (rl) return rl;
        }
        return DS_OK;
    }
    bool fp = false;
    const int rc = setup_common(p, bits, base, fuse, fp);
    if (rc) return rc;
    p.prepare_only = prepare ? 1 : 0;
    p.needed_out = needed_out;
    set_check_extents(p, (long long)B * C * H * W);
    return launch_conv(p, fp, static_cast<cudaStream_t>(stream));
}

}  // namespace
}  // namespace ds

extern "C" int ds_conv2d_ex(const void* x, const int32_t* packed, const int32_t* bias, void* out, int B,
                            int C, int H, int W, int OC, int KH, int KW, int sh, int sw, int ph, int pw,
                            int bits, int base, const ds_fuse_t* fuse, void* stream)
{
    return ds::conv2d_run(x, packed, bias, out, B, C, H, W, OC, KH, KW, sh, sw, ph, pw, bits, base, fuse, stream,
                          nullptr);
}

extern "C" int ds_conv2d_prepare(const int32_t* packed, int B, int C, int H, int W, int OC, int KH, int KW,
                                 int sh, int sw, int ph, int pw, int bits, int base, const ds_fuse_t* fuse,
                                 long long* bytes_needed, void* stream)
{
    if (!bytes_needed) return DS_ERR_BAD_ARG;
    *bytes_needed = 0;
    return ds::conv2d_run(nullptr, packed, nullptr, nullptr, B, C, H, W, OC, KH, KW, sh, sw, ph, pw, bits, base,
                          fuse, stream, bytes_needed);
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

// ---------------------------------------------------------------------------------------------
// Convolution entry point that allocates nothing, for callers that cannot call cudaMalloc.
namespace {

constexpr int kNoAllocMaxTiles = 16384;  // output tiles (256 rows x 128 or 64 columns) per call
constexpr int kNoAllocMaxDevices = 64;

// The split-K arrival counters of ds_conv2d_noalloc.  The array lives in the library image: every
// GPU that loads the library holds these 64 KiB until the process exits.  In host code this name is
// only a handle; the kernels need the device address, which cudaGetSymbolAddress gives per device.
static __device__ __align__(256) int g_noalloc_counters[kNoAllocMaxTiles];

int* g_noalloc_dev_ptr[kNoAllocMaxDevices];  // device address of the array, per device ordinal

}  // namespace

extern "C" int ds_conv2d_noalloc(const void* x, const int32_t* packed, const int32_t* bias, void* out, int B,
                                 int C, int H, int W, int OC, int KH, int KW, int sh, int sw, int ph, int pw,
                                 int bits, int base, const ds_fuse_t* fuse, void* stream)
{
    if (B < 0 || C <= 0 || H <= 0 || W <= 0 || OC <= 0 || KH <= 0 || KW <= 0 || sh <= 0 || sw <= 0 ||
        ph < 0 || pw < 0 || H + 2 * ph < KH || W + 2 * pw < KW)
        return DS_ERR_BAD_ARG;
    if (B == 0) return DS_OK;
    const long long OH = (H + 2 * ph - KH) / sh + 1, OW = (W + 2 * pw - KW) / sw + 1;
    const long long tiles = ((B * OH * OW + 255) / 256) * ((OC + (OC > 64 ? 127 : 63)) / (OC > 64 ? 128 : 64));
    if (tiles > kNoAllocMaxTiles) return DS_ERR_SCRATCH;

    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return DS_ERR_CUDA;
    if (dev < 0 || dev >= kNoAllocMaxDevices) return DS_ERR_UNSUPPORTED;
    if (!g_noalloc_dev_ptr[dev]) {  // set-up: once per device, with that device current
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_noalloc_counters) != cudaSuccess || !ptr) {
            cudaGetLastError();
            return DS_ERR_CUDA;
        }
        g_noalloc_dev_ptr[dev] = static_cast<int*>(ptr);
    }
    int* counters = g_noalloc_dev_ptr[dev];
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call (or an aborted one) left; the counters must start at 0.
    if (cudaMemsetAsync(counters, 0, size_t(tiles) * sizeof(int), st) != cudaSuccess) return DS_ERR_CUDA;
    ds_fuse_t f = {};
    if (fuse) f = *fuse;
    f.workspace = counters;
    f.workspace_bytes = (long long)kNoAllocMaxTiles * (long long)sizeof(int);
    return ds_conv2d_ex(x, packed, bias, out, B, C, H, W, OC, KH, KW, sh, sw, ph, pw, bits, base, &f, stream);
}

// Checked build only: declares the activations `bytes` shorter than they are for the calls that
// follow (0 restores the truth), so that a test can watch the checks catch loads beyond the declared
// end without any access leaving the real buffer.  DS_ERR_UNSUPPORTED in a normal build.
extern "C" int ds_bounds_debug_shrink_x(long long bytes)
{
#ifdef DS_BOUNDS_CHECK
    if (bytes < 0) return DS_ERR_BAD_ARG;
    ds::g_check_shrink_x = bytes;
    return DS_OK;
#else
    (void)bytes;
    return DS_ERR_UNSUPPORTED;
#endif
}
