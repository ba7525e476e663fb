// Warp-specialised FP32-pipe shift "GEMM" / convolution for sm_100a.
//
// Arithmetic: see ds_gemm.cu (one FFMA with round-toward-minus-infinity per term, magic-offset
// accumulators drained into shared int32 slots).  This file changes how the work is divided:
//
//   * 16 consumer warps (512 threads) own a 256 x BN output tile, 8 x TN outputs per thread.
//     Their loop is nothing but shared-memory fragment loads and FFMAs; they never touch
//     global memory before the epilogue and never wait on another consumer warp.
//   * 8 producer warps (256 threads) gather x (implicit im2col, zero padding by predication,
//     int32 -> x + 0.5 conversion or the fused fp32 quantiser), fetch the packed weight words
//     and decode them through the lookup table, one k-tile ahead of the consumers.  For a
//     linear layer (x is [M,K]) a producer thread owns one row and reads its k-tile with
//     16-byte loads; its stores into the k-major stage are conflict-free.
//   * The two groups meet only at mbarriers: full[s] (one arrival per producer warp, plus one per
//     producer thread when its asynchronous weight copies land) and empty[s] (one per consumer
//     warp) for each stage of the ring (two, or three on the 64-column tile).  Global-load latency, the decode chains
//     and the stores of a stage all overlap the FFMA stream of the previous stage, so the
//     FMA pipe no longer idles while "everybody stages".
//
// Every wait is bounded: a wait that runs out records an error and lets the thread continue,
// so the kernel always terminates; the host can read the flag with ds_last_kernel_error().
#pragma once
#include "ds_gemm_common.cuh"

// -DDS_WS_TIMING (the "timing" flavour of the library): every warp of CTA 1 counts the cycles it
// spends waiting at the hand-shake, staging and in the epilogue, and prints them when the kernel
// ends.  A diagnostic build; the normal build contains none of it.
#ifdef DS_WS_TIMING
#include <cstdio>
#define WS_T(...) __VA_ARGS__
#else
#define WS_T(...)
#endif

namespace ds {
namespace {

constexpr int WS_CONS = 512;   // consumer threads
constexpr int WS_PROD = 256;   // producer threads
constexpr int WS_NT = WS_CONS + WS_PROD;
constexpr int WS_BM = 256;     // rows of x per CTA
constexpr int WS_BKT = 28;     // largest k-tile
// Stages of the ring: two on the 128-column tile (the accumulator slots take 128 KiB of shared
// memory there), three on the 64-column tile, where the slots are half as large and the producers'
// chain per k-tile is as long as the consumers' k-tile: with a third stage they never wait for `empty`.
template <int TN>
struct WsStages {
    static constexpr int N = (TN == 4) ? 3 : 2;
};
// Register split after the roles part.  The CTA starts with 768 * 80 registers; what the
// producers give back is all the consumers can take: a larger request would wait for registers
// that never come.  Usual split 56 / 88 (256 * 24 >= 512 * 8).  The four-pixel staging mode and
// the linear layer need fewer producer registers, so their split is 48 / 96 (256 * 32 = 512 * 16): with 96 registers the
// compiler has room to fetch the next fragments early, and a consumer warp running without its
// neighbours (which wait at the hand-shake) keeps the FMA pipe busier.
constexpr int WS_LAUNCH_REGS = 80;
template <int AM>
struct WsRegs {
    static constexpr int PROD = (AM == AM_QUAD3 || AM == AM_LINEAR || AM == AM_S2K7) ? 48 : 56;
    static constexpr int CONS = (AM == AM_QUAD3 || AM == AM_LINEAR || AM == AM_S2K7) ? 96 : 88;
    static_assert(WS_CONS * (CONS - WS_LAUNCH_REGS) <= WS_PROD * (WS_LAUNCH_REGS - PROD), "register pool");
};
constexpr int WS_WAIT_LIMIT = 1 << 12;  // rounds of one mbarrier wait before giving up
constexpr unsigned WS_WAIT_NS = 1000000;  // suspend-time hint of one round, nanoseconds


template <int TN>
struct WsSmem {
    static constexpr int BN = 16 * TN;
    static constexpr int AP = WS_BM + 4;
    static constexpr int STAGES = WsStages<TN>::N;
    alignas(16) float a[STAGES][WS_BKT][AP];  // x + 0.5
    alignas(16) float b[STAGES][WS_BKT][BN];  // +-2^-r
    alignas(16) KEntry ktab[2][WS_BKT];       // by k-tile parity: written one k-tile ahead of its use
    alignas(8) unsigned long long full[STAGES];
    alignas(8) unsigned long long empty[STAGES];
    int lut0[256];  // float bits of the decoded weight per field value
    // Negative weights per output column.  NEGSETS sets, used round-robin by item: the producers can
    // be STAGES items ahead of the consumers (items of a single k-tile), and a set is cleared by the
    // consumers only after their epilogue.
    static constexpr int NEGSETS = (STAGES == 2) ? 4 : 8;
    int negc[NEGSETS][BN];
    int err;
    int last_flag;  // split-K: this CTA arrived last at its tile's counter
    int accs[kTM * TN * WS_CONS];  // drained accumulators, [slot][consumer thread]
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar)
{
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}

// One arrival for the whole warp: 32 arrivals on the same word would be served one after the
// other.  __syncwarp orders every lane's shared-memory accesses before the elected lane's arrive.
__device__ __forceinline__ void warp_arrive(unsigned long long* bar)
{
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}

// Bounded wait for the phase with the given parity to complete.  Each try_wait lets the hardware
// suspend the thread for up to WS_WAIT_NS before it reports "not yet", so a waiting warp issues
// almost nothing.  Returns false after WS_WAIT_LIMIT such rounds (seconds; a correct run waits
// microseconds).
__device__ __forceinline__ bool mbar_try_once(unsigned addr, unsigned parity)
{
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity), "r"(WS_WAIT_NS)
        : "memory");
    return ok != 0;
}

// Bounded wait.  `err` is the CTA's error word in shared memory: whoever gives up sets it, and every
// wait that finds it set after a failed round gives up at once, so that a launch in which something
// went wrong ends within seconds instead of one full limit per wait.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* err)
{
    const unsigned addr = smem_u32(bar);
    for (int i = 0; i < WS_WAIT_LIMIT; ++i) {
        if (mbar_try_once(addr, parity)) return true;
        if (*err) return false;
    }
    *err = 1;
    return false;
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}

// One arrival on `bar` once every cp.async this thread has issued so far has landed.  The thread
// does not wait; the barrier's expected count must include this arrival (.noinc).
__device__ __forceinline__ void cp_async_arrive_on(unsigned long long* bar)
{
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 2, %0;" ::"n"(WS_CONS) : "memory"); }

__device__ __forceinline__ void producer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(WS_PROD) : "memory"); }

// ---------------------------------------------------------------------------------------------
// Work unit = (output tile, K range).  Units are numbered with the row tile fastest, so CTAs that
// run side by side share weight tiles in L2.  Units [0, full_units) cover every output tile
// `splits` times (1 = each tile whole); the units after them are the tail: the last tail_items
// tiles, each cut into tail_splits K ranges so that the last wave of CTAs is short instead of
// mostly empty.
struct WsItem {
    int m0, n0, t_begin, t_end, tile_id;
    int tail_idx;  // >= 0: tail unit of that tail tile, partial sums go through the workspace
    int sp;
};

__device__ __forceinline__ WsItem ws_item(const GemmParams& p, int unit, int BM, int BN)
{
    WsItem w;
    int tile, tps;
    if (unit < p.full_units) {
        const int tiles = p.grid_m * p.grid_n;
        w.sp = unit / tiles;
        tile = unit - w.sp * tiles;
        tps = p.tiles_per_split;
        w.tail_idx = -1;
    } else {
        const int v = unit - p.full_units;
        w.sp = v / p.tail_items;
        w.tail_idx = v - w.sp * p.tail_items;
        tile = p.tail_first + w.tail_idx;
        tps = p.tail_tps;
    }
    const int nt = tile / p.grid_m, mt = tile - nt * p.grid_m;
    w.m0 = mt * BM;
    w.n0 = nt * BN;
    w.t_begin = w.sp * tps;
    w.t_end = min(p.ntiles, w.t_begin + tps);
    w.tile_id = tile;
    return w;
}

template <int TN, int AM, bool PRE>
__global__ void __launch_bounds__(WS_NT, 1) ws_kernel(const GemmParams p)
{
    using S = WsSmem<TN>;
    constexpr bool CONV = AM != AM_LINEAR;
    constexpr bool QUAD = AM == AM_QUAD3;
    constexpr bool PAIR = AM == AM_PAIR3;
    constexpr bool S2K7 = AM == AM_S2K7;
    constexpr bool ROW = AM >= 1;
    constexpr int KW = (QUAD || PAIR) ? 3 : (S2K7 ? 7 : (ROW ? AM : 1));
    constexpr int BM = WS_BM, BN = S::BN;
    constexpr int TMG = 32, TNG = 16;
    static_assert(offsetof(S, b) % 16 == 0 && offsetof(S, ktab) % 16 == 0 && offsetof(S, full) % 8 == 0, "alignment");

    extern __shared__ __align__(16) unsigned char smem_raw[];
    S& s = *reinterpret_cast<S*>(smem_raw);

    const int t = threadIdx.x;
    const int total_items = p.full_units + p.tail_items * p.tail_splits;
    if (p.gate && *p.gate != p.gate_want) return;  // the other arithmetic path serves this input

    // ---- set-up by all threads ------------------------------------------------------------------
    for (int f = t; f < (1 << p.dec.fw); f += WS_NT) {
        int neg;
        s.lut0[f] = __float_as_int(decode_f32(uint32_t(f), p.dec, true, neg));
    }
    for (int i = t; i < S::NEGSETS * BN; i += WS_NT) (&s.negc[0][0])[i] = 0;
    if (t == 0) {
        for (int i = 0; i < S::STAGES; ++i) {
            // one arrival per producer warp (x stored) and, with expanded weights, one per producer
            // thread when its asynchronous weight copies have landed
            mbar_init(&s.full[i], WS_PROD / 32 + (PRE ? WS_PROD : 0));
            mbar_init(&s.empty[i], WS_CONS / 32);
        }
        s.err = 0;
    }
    __syncthreads();

    if (t >= WS_CONS) {
        // =========================== producers ==================================================
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(WsRegs<AM>::PROD));
        const int pt = t - WS_CONS;
        constexpr int PIX = BM / WS_PROD;  // rows of the x tile per producer thread (conv)
        const char* x_pix[PIX];
        uint32_t rowmask[PIX], colmask[PIX];
        // weight words: column n = wi % BN, word jw = wi / BN of the k-tile, wi = pt + WS_PROD * e
        constexpr int EW = (BN * (WS_BKT / 4) + WS_PROD - 1) / WS_PROD;
        const int wn = pt & (BN - 1);
        const int32_t* wrow = nullptr;
        const uint32_t fmask = (1u << p.dec.fw) - 1u;

        // Registers that hold one k-tile of this thread's x values and weight words between the
        // global loads (issued one tile ahead) and their conversion into shared memory.
        constexpr int RMAX = (KW == 1) ? 28 : (KW == 3 ? 8 : 4);  // rows of the largest k-tile, row mode
        constexpr int XN = ROW ? RMAX * KW : WS_BKT;      // x values per thread per tile (conv)
        // linear: a thread owns one row of x and reads its k-tile with 16-byte loads
        static_assert(CONV || (PIX == 1 && WS_BKT % 4 == 0), "linear staging: one row per producer thread");
        constexpr int XREG = CONV ? XN * PIX : WS_BKT;
        int xr[XREG];
        uint32_t w_reg[EW];
        static_assert(XREG <= 32, "producer registers");

        // Per-item state of this thread: the x rows it gathers and the weight row it decodes.
        auto setup_item = [&](const WsItem& w) {
            wrow = (w.n0 + wn < p.N) ? p.packed + (long long)(w.n0 + wn) * p.dec.row_len : nullptr;
            if (QUAD) {
                // this thread's four pixels: same image, same output row, ow a multiple of 4
                const int m = w.m0 + 4 * (pt & 63);
                x_pix[0] = reinterpret_cast<const char*>(p.x);
                rowmask[0] = colmask[0] = 0;
                if (m < p.M) {
                    const int b = m / p.P, pp = m - b * p.P;
                    const int oh = pp / p.OW, ow = pp - oh * p.OW;
                    const int ih0 = oh * p.sh - p.ph;
                    for (int kh = 0; kh < p.KH; ++kh)
                        if (unsigned(ih0 + kh) < unsigned(p.H)) rowmask[0] |= 1u << kh;
                    colmask[0] = (ow > 0 ? 1u : 0u) | (ow + 4 < p.W ? 2u : 0u);  // value left / right of the four
                    // address of (b, 0, ih0, ow): the centre tap of the first pixel
                    x_pix[0] += ((long long)b * p.C * p.H * p.W + (long long)ih0 * p.W + ow) * 4;
                }
            } else if (S2K7) {
                // this thread's four output pixels: same image, same output row, ow a multiple of 4;
                // the sixteen inputs iw = 2*ow - 4 .. 2*ow + 11 cover their windows (iw0 = 2*ow - 3)
                const int m = w.m0 + 4 * (pt & 63);
                x_pix[0] = reinterpret_cast<const char*>(p.x);
                rowmask[0] = colmask[0] = 0;
                if (m < p.M) {
                    const int b = m / p.P, pp = m - b * p.P;
                    const int oh = pp / p.OW, ow = pp - oh * p.OW;
                    const int ih0 = oh * p.sh - p.ph, iwb = 2 * ow - 4;
                    for (int kh = 0; kh < p.KH; ++kh)
                        if (unsigned(ih0 + kh) < unsigned(p.H)) rowmask[0] |= 1u << kh;
                    for (int v = 0; v < 4; ++v)  // whole 16-byte groups lie inside or outside the row
                        if (unsigned(iwb + 4 * v) < unsigned(p.W)) colmask[0] |= 1u << v;
                    x_pix[0] += ((long long)b * p.C * p.H * p.W + (long long)ih0 * p.W + iwb) * 4;
                }
            } else if (PAIR) {
                // this thread's two pixels: same image, same output row, ow even
                const int m = w.m0 + 2 * (pt & 127);
                x_pix[0] = reinterpret_cast<const char*>(p.x);
                rowmask[0] = colmask[0] = 0;
                if (m < p.M) {
                    const int b = m / p.P, pp = m - b * p.P;
                    const int oh = pp / p.OW, ow = pp - oh * p.OW;
                    const int ih0 = oh * p.sh - p.ph;
                    for (int kh = 0; kh < p.KH; ++kh)
                        if (unsigned(ih0 + kh) < unsigned(p.H)) rowmask[0] |= 1u << kh;
                    colmask[0] = (ow > 0 ? 1u : 0u) | (ow + 2 < p.W ? 2u : 0u);  // value left / right of the two
                    x_pix[0] += ((long long)b * p.C * p.H * p.W + (long long)ih0 * p.W + ow) * 4;
                }
            } else if (CONV) {
#pragma unroll
                for (int q = 0; q < PIX; ++q) {
                    const int m = w.m0 + pt + q * WS_PROD;
                    x_pix[q] = reinterpret_cast<const char*>(p.x);
                    rowmask[q] = colmask[q] = 0;
                    if (m < p.M) {
                        const int b = m / p.P, pp = m - b * p.P;
                        const int oh = pp / p.OW, ow = pp - oh * p.OW;
                        const int ih0 = oh * p.sh - p.ph, iw0 = ow * p.sw - p.pw;
                        for (int kh = 0; kh < p.KH; ++kh)
                            if (unsigned(ih0 + kh) < unsigned(p.H)) rowmask[q] |= 1u << kh;
                        for (int kw = 0; kw < p.KW; ++kw)
                            if (unsigned(iw0 + kw) < unsigned(p.W)) colmask[q] |= 1u << kw;
                        // address of (b, 0, ih0, iw0): may lie outside the tensor, only valid taps are read
                        x_pix[q] += ((long long)b * p.C * p.H * p.W + (long long)ih0 * p.W + iw0) * 4;
                    }
                }
            } else {
                // x is [M,K]: this thread's row
                const int m = w.m0 + pt;
                x_pix[0] = reinterpret_cast<const char*>(p.x);
                rowmask[0] = colmask[0] = 0;
                if (m < p.M) {
                    rowmask[0] = 1u;
                    x_pix[0] += (long long)m * p.K * 4;
                }
            }
        };

        auto fill_table = [&](int tile) {
            if (!CONV || pt >= WS_BKT) return;
            KEntry e;
            e.pad = 0;
            e.off = 0;
            e.kh = 31;
            e.kw = 0;
            if (ROW) {
                const int row = tile * p.rows_per_tile + pt;  // global (ic,kh) row index
                if (pt < p.rows_per_tile && row < p.C * p.KH) {
                    const int ic = magic_div(row, p.magic_kh);
                    e.kh = row - ic * p.KH;
                    e.off = (ic * p.H * p.W + e.kh * p.W) * 4;
                }
            } else {
                const int k = tile * p.bk + pt;
                if (pt < p.bk && k < p.K) {
                    const int ic = magic_div(k, p.magic_khw);
                    const int tap = k - ic * (p.KH * p.KW);
                    e.kh = magic_div(tap, p.magic_kw);
                    e.kw = tap - e.kh * p.KW;
                    e.off = (ic * p.H * p.W + e.kh * p.W + e.kw) * 4;
                }
            }
            s.ktab[tile & 1][pt] = e;
        };

        // Issues the global loads of one k-tile into registers.  Positions outside the image or
        // the matrix get `padv` (0, or the marker that stands for an unquantised 0 for fp32 kinds).
        auto issue_loads = [&](int tile, int m0) {
            const int padv = p.pad_raw;
            if (!PRE) {
                const int w0 = tile * p.kt_words;
#pragma unroll
                for (int e = 0; e < EW; ++e) {
                    const int jw = (pt + e * WS_PROD) / BN;
                    uint32_t w = 0;
                    if (wrow && jw < p.kt_words && w0 + jw < p.dec.row_len && DS_W_OK(p, wrow + w0 + jw, 4)) w = uint32_t(__ldg(wrow + w0 + jw));
                    w_reg[e] = w;
                }
            }
            const int tb = tile & 1;
            if (QUAD) {
                // thread = (four pixels, row group): rows rg, rg + 4 of the k-tile
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int2 e = *reinterpret_cast<const int2*>(&s.ktab[tb][(pt >> 6) + 4 * j]);
                    const int* rowp = reinterpret_cast<const int*>(x_pix[0] + e.x);
                    int4 c = make_int4(padv, padv, padv, padv);
                    int l = padv, r = padv;
                    if ((rowmask[0] >> e.y) & 1u) {  // rows past the tile: kh = 31
                        if (DS_X_OK(p, rowp, 16)) c = __ldg(reinterpret_cast<const int4*>(rowp));
                        if ((colmask[0] & 1u) && DS_X_OK(p, rowp - 1, 4)) l = __ldg(rowp - 1);
                        if ((colmask[0] & 2u) && DS_X_OK(p, rowp + 4, 4)) r = __ldg(rowp + 4);
                    }
                    xr[6 * j + 0] = l;
                    xr[6 * j + 1] = c.x;
                    xr[6 * j + 2] = c.y;
                    xr[6 * j + 3] = c.z;
                    xr[6 * j + 4] = c.w;
                    xr[6 * j + 5] = r;
                }
            } else if (S2K7) {
                // thread = (four output pixels, row pt / 64 of the k-tile)
                const int2 e = *reinterpret_cast<const int2*>(&s.ktab[tb][pt >> 6]);
                const int4* rowp = reinterpret_cast<const int4*>(x_pix[0] + e.x);
                const bool rv = (rowmask[0] >> e.y) & 1u;  // rows past the tile: kh = 31
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    int4 c = make_int4(padv, padv, padv, padv);
                    if (rv && ((colmask[0] >> v) & 1u) && DS_X_OK(p, rowp + v, 16)) c = __ldg(rowp + v);
                    xr[4 * v + 0] = c.x;
                    xr[4 * v + 1] = c.y;
                    xr[4 * v + 2] = c.z;
                    xr[4 * v + 3] = c.w;
                }
            } else if (PAIR) {
                // thread = (two pixels, row group): rows rg, rg + 2, rg + 4, rg + 6 of the k-tile
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int2 e = *reinterpret_cast<const int2*>(&s.ktab[tb][(pt >> 7) + 2 * j]);
                    const int* rowp = reinterpret_cast<const int*>(x_pix[0] + e.x);
                    int2 c = make_int2(padv, padv);
                    int l = padv, r = padv;
                    if ((rowmask[0] >> e.y) & 1u) {  // rows past the tile: kh = 31
                        if (DS_X_OK(p, rowp, 8)) c = __ldg(reinterpret_cast<const int2*>(rowp));
                        if ((colmask[0] & 1u) && DS_X_OK(p, rowp - 1, 4)) l = __ldg(rowp - 1);
                        if ((colmask[0] & 2u) && DS_X_OK(p, rowp + 2, 4)) r = __ldg(rowp + 2);
                    }
                    xr[4 * j + 0] = l;
                    xr[4 * j + 1] = c.x;
                    xr[4 * j + 2] = c.y;
                    xr[4 * j + 3] = r;
                }
            } else if (ROW) {
#pragma unroll
                for (int u = 0; u < RMAX; ++u) {
                    const int2 e = *reinterpret_cast<const int2*>(&s.ktab[tb][u]);  // rows past the tile: kh = 31
#pragma unroll
                    for (int q = 0; q < PIX; ++q) {
                        const bool rv = (rowmask[q] >> e.y) & 1u;
                        const int* rowp = reinterpret_cast<const int*>(x_pix[q] + e.x);
#pragma unroll
                        for (int kw = 0; kw < KW; ++kw) {
                            int val = padv;
                            if (rv && (colmask[q] & (1u << kw)) && DS_X_OK(p, rowp + kw, 4)) val = __ldg(rowp + kw);
                            xr[(q * RMAX + u) * KW + kw] = val;
                        }
                    }
                }
            } else if (CONV) {
#pragma unroll
                for (int u = 0; u < WS_BKT; ++u) {
                    const int4 e = *reinterpret_cast<const int4*>(&s.ktab[tb][u]);
#pragma unroll
                    for (int q = 0; q < PIX; ++q) {
                        int val = padv;
                        if (((rowmask[q] >> e.y) & (colmask[q] >> e.z) & 1u) != 0u && DS_X_OK(p, x_pix[q] + e.x, 4))
                            val = __ldg(reinterpret_cast<const int*>(x_pix[q] + e.x));
                        xr[q * WS_BKT + u] = val;
                    }
                }
            } else {
                // x is [M,K] with K a multiple of 4 and 16-byte aligned rows (checked by the host):
                // whole 16-byte groups of this thread's row, each inside K or beyond it
                const int k0 = tile * p.bk;
                const int4* rp = reinterpret_cast<const int4*>(x_pix[0] + (long long)k0 * 4);
#pragma unroll
                for (int v = 0; v < WS_BKT / 4; ++v) {
                    int4 c = make_int4(padv, padv, padv, padv);
                    if (rowmask[0] && 4 * v < p.bk && k0 + 4 * v < p.K && DS_X_OK(p, rp + v, 16)) c = __ldg(rp + v);
                    xr[4 * v + 0] = c.x;
                    xr[4 * v + 1] = c.y;
                    xr[4 * v + 2] = c.z;
                    xr[4 * v + 3] = c.w;
                }
            }
        };

        // Converts the registers of one k-tile and stores them into stage `st`.  INK: input kind;
        // LAST: the tile may reach past K, where x is stored as 0 (see the weight tail below).
        auto store_x = [&](auto ink_tag, auto last_tag, int st, int k0) {
            constexpr int INK = decltype(ink_tag)::value;
            constexpr bool LAST = decltype(last_tag)::value;
            if (QUAD) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int u = (pt >> 6) + 4 * j;
                    if (u < p.rows_per_tile) {
                        float f[6];
#pragma unroll
                        for (int i = 0; i < 6; ++i) f[i] = operand_of<true, INK>(p, xr[6 * j + i]);
#pragma unroll
                        for (int kw = 0; kw < 3; ++kw) {
                            float4 v = make_float4(f[kw], f[kw + 1], f[kw + 2], f[kw + 3]);
                            if (LAST && k0 + u * 3 + kw >= p.K) v = make_float4(0.f, 0.f, 0.f, 0.f);
                            *reinterpret_cast<float4*>(&s.a[st][u * 3 + kw][4 * (pt & 63)]) = v;
                        }
                    }
                }
            } else if (S2K7) {
                const int u = pt >> 6;
                if (u < p.rows_per_tile) {
                    float f[16];
#pragma unroll
                    for (int i = 1; i < 14; ++i) f[i] = operand_of<true, INK>(p, xr[i]);
#pragma unroll
                    for (int kw = 0; kw < 7; ++kw) {
                        // pixel i of the four reads input 2*i + kw - 3, i.e. slot 2*i + kw + 1 of the sixteen
                        float4 v = make_float4(f[kw + 1], f[kw + 3], f[kw + 5], f[kw + 7]);
                        if (LAST && k0 + u * 7 + kw >= p.K) v = make_float4(0.f, 0.f, 0.f, 0.f);
                        *reinterpret_cast<float4*>(&s.a[st][u * 7 + kw][4 * (pt & 63)]) = v;
                    }
                }
            } else if (PAIR) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int u = (pt >> 7) + 2 * j;
                    if (u < p.rows_per_tile) {
                        float f[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) f[i] = operand_of<true, INK>(p, xr[4 * j + i]);
#pragma unroll
                        for (int kw = 0; kw < 3; ++kw) {
                            float2 v = make_float2(f[kw], f[kw + 1]);
                            if (LAST && k0 + u * 3 + kw >= p.K) v = make_float2(0.f, 0.f);
                            *reinterpret_cast<float2*>(&s.a[st][u * 3 + kw][2 * (pt & 127)]) = v;
                        }
                    }
                }
            } else if (ROW) {
#pragma unroll
                for (int u = 0; u < RMAX; ++u) {
                    if (u < p.rows_per_tile) {
#pragma unroll
                        for (int q = 0; q < PIX; ++q)
#pragma unroll
                            for (int kw = 0; kw < KW; ++kw) {
                                float o = operand_of<true, INK>(p, xr[(q * RMAX + u) * KW + kw]);
                                if (LAST && k0 + u * KW + kw >= p.K) o = 0.f;
                                s.a[st][u * KW + kw][pt + q * WS_PROD] = o;
                            }
                    }
                }
            } else if (CONV) {
#pragma unroll
                for (int u = 0; u < WS_BKT; ++u) {
                    if (u < p.bk) {
#pragma unroll
                        for (int q = 0; q < PIX; ++q) {
                            float o = operand_of<true, INK>(p, xr[q * WS_BKT + u]);
                            if (LAST && k0 + u >= p.K) o = 0.f;
                            s.a[st][u][pt + q * WS_PROD] = o;
                        }
                    }
                }
            } else {
                // consecutive threads hold consecutive rows: conflict-free stores
#pragma unroll
                for (int u = 0; u < WS_BKT; ++u) {
                    if (u < p.bk) {
                        float o = operand_of<true, INK>(p, xr[u]);
                        if (LAST && k0 + u >= p.K) o = 0.f;
                        s.a[st][u][pt] = o;
                    }
                }
            }
        };

        // Decodes this thread's weight words through the table into stage `st`.  Slots k >= K of
        // the last words decode like any field (a zero field is -2^0); the x values stored there
        // are 0, so they add nothing, and the epilogue takes their share (tail_neg) out of the
        // negative-weight count `negc` of the item.
        auto store_w = [&](auto num_tag, int st, int* negc) {
            constexpr int NUM = decltype(num_tag)::value;
            int negs = 0;
#pragma unroll
            for (int e = 0; e < EW; ++e) {
                const int jw = (pt + e * WS_PROD) / BN;
                if (jw < p.kt_words) {
                    uint32_t w = w_reg[e];
                    float* dst = &s.b[st][jw * NUM][wn];
#pragma unroll
                    for (int i = 0; i < NUM; ++i) {
                        const int v0 = s.lut0[w & fmask];
                        w >>= p.dec.fw;
                        dst[i * BN] = __int_as_float(v0);
                        negs += int(uint32_t(v0) >> 31);
                    }
                }
            }
            if (negs) atomicAdd(&negc[wn], negs);
        };

        // Expanded weights: rows k0 .. k0+bk-1, BN floats each, straight from global into the stage
        // (asynchronous 16-byte copies; the x conversion below runs while they are in flight).
        auto copy_w_async = [&](int tile, int st, int n0) {
            constexpr int C4 = BN / 4;
            const float* src = p.wd + (long long)tile * p.bk * p.npad + n0;
            for (int e = pt; e < p.bk * C4; e += WS_PROD) {
                const int r = e / C4, c = e - r * C4;
                cp_async_16(&s.b[st][r][4 * c], src + (long long)r * p.npad + 4 * c);
            }
        };

        // The CTA walks its items; within an item the k-tiles.  Loads run one k-tile ahead of the
        // stores -- also across item boundaries: while the consumers finish an output tile and run
        // its epilogue, the first k-tiles of the next item are already being staged.
        int item = blockIdx.x, seq = 0, git = 0;
        WS_T(long long tw = 0, ts = 0, tt = 0, tl = 0, t0 = 0, t1 = 0; const long long tstart = clock64();)
        if (item < total_items) {
            WsItem cur = ws_item(p, item, BM, BN);
            int tile = cur.t_begin;
            setup_item(cur);
            fill_table(tile);
            if (CONV) producer_bar();
            issue_loads(tile, cur.m0);
            while (true) {
                const int st = git % S::STAGES;
                WS_T(t0 = clock64();)
                if (git >= S::STAGES) mbar_wait(&s.empty[st], unsigned(git / S::STAGES - 1) & 1u, &s.err);
                WS_T(t1 = clock64(); tw += t1 - t0;)
                const int k0 = tile * p.bk;
                // Expanded weights are 0 beyond K, so the x values stored there need no care.
                const bool last = !PRE && tile + 1 >= p.ntiles;
                if (PRE) {
                    copy_w_async(tile, st, cur.n0);
                    cp_async_arrive_on(&s.full[st]);  // nobody waits here for the copies
                }
                with_input_kind(p, [&](auto ink_tag) {
                    if (last) store_x(ink_tag, std::true_type(), st, k0);
                    else store_x(ink_tag, std::false_type(), st, k0);
                });
                if (!PRE) {
                    int* negc = s.negc[seq & (S::NEGSETS - 1)];
                    switch (p.dec.num) {
                        case 4: store_w(std::integral_constant<int, 4>(), st, negc); break;
                        case 5: store_w(std::integral_constant<int, 5>(), st, negc); break;
                        case 6: store_w(std::integral_constant<int, 6>(), st, negc); break;
                        case 8: store_w(std::integral_constant<int, 8>(), st, negc); break;
                        case 10: store_w(std::integral_constant<int, 10>(), st, negc); break;
                        default: store_w(std::integral_constant<int, 16>(), st, negc); break;
                    }
                }
                warp_arrive(&s.full[st]);
                WS_T(ts += clock64() - t1;)
                ++git;
                // next (item, k-tile)
                if (++tile >= cur.t_end) {
                    item += gridDim.x;
                    if (item >= total_items) break;
                    ++seq;
                    cur = ws_item(p, item, BM, BN);
                    tile = cur.t_begin;
                    setup_item(cur);
                }
                WS_T(t0 = clock64();)
                fill_table(tile);
                if (CONV) producer_bar();
                WS_T(t1 = clock64(); tt += t1 - t0;)
                issue_loads(tile, cur.m0);
                WS_T(tl += clock64() - t1;)
            }
        }
        WS_T(if (blockIdx.x == 1 && (t & 31) == 0)
                 printf("ws_timing producer warp %d: cycles %lld wait_empty %lld convert_store %lld table %lld issue_loads %lld k_tiles %d\n",
                        t >> 5, clock64() - tstart, tw, ts, tt, tl, git);)
        if (s.err) *p.err_flag = 1;
        return;
    }

    // =============================== consumers ====================================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(WsRegs<AM>::CONS));
    // A warp covers 8 x 4 thread tiles, 8 along the direction in which the output is contiguous.
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
    float accf[kTM][TN];
    int git = 0, seq = 0;
    WS_T(long long tw = 0, te = 0, t0 = 0; const long long tstart = clock64();)
    for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++seq) {
        const WsItem cur = ws_item(p, item, BM, BN);
        const int my_tiles = cur.t_end - cur.t_begin;
#pragma unroll
        for (int i = 0; i < kTM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) accf[i][j] = kMagic;
        int ndrains = 0, since = 0;
        for (int it = 0; it < my_tiles; ++it, ++git) {
            const int st = git % S::STAGES;
            WS_T(t0 = clock64();)
            mbar_wait(&s.full[st], unsigned(git / S::STAGES) & 1u, &s.err);
            WS_T(tw += clock64() - t0;)
            // The k-tile sizes of 3x3, 1x1 / 7x7 and 5x5 windows get fully unrolled loops.
            auto k_loop = [&](auto bk_tag) {
                constexpr int CBK = decltype(bk_tag)::value;
                const int nk = CBK ? CBK : p.bk;
                constexpr int UNR = CBK ? CBK : 8;
#pragma unroll(UNR)
                for (int k = 0; k < nk; ++k) {
                    float a[kTM], b[TN];
                    *reinterpret_cast<float4*>(&a[0]) = *reinterpret_cast<const float4*>(&s.a[st][k][4 * tm]);
                    *reinterpret_cast<float4*>(&a[4]) = *reinterpret_cast<const float4*>(&s.a[st][k][BM / 2 + 4 * tm]);
                    *reinterpret_cast<float4*>(&b[0]) = *reinterpret_cast<const float4*>(&s.b[st][k][4 * tn]);
                    if (TN == 8)
                        *reinterpret_cast<float4*>(&b[TN - 4]) =
                            *reinterpret_cast<const float4*>(&s.b[st][k][BN / 2 + 4 * tn]);
#pragma unroll
                    for (int i = 0; i < kTM; ++i)
#pragma unroll
                        for (int j = 0; j < TN; ++j) accf[i][j] = __fmaf_rd(a[i], b[j], accf[i][j]);
                }
            };
            if (p.bk == 24) k_loop(std::integral_constant<int, 24>());
            else if (p.bk == 28) k_loop(std::integral_constant<int, 28>());
            else if (KW == 7 && p.bk == 21) k_loop(std::integral_constant<int, (KW == 7 ? 21 : 0)>());
            else if (KW == 1 && p.bk == 16) k_loop(std::integral_constant<int, (KW == 1 ? 16 : 0)>());
            else k_loop(std::integral_constant<int, 0>());
            warp_arrive(&s.empty[st]);
            if (++since == p.flush_tiles || it + 1 == my_tiles) {
                // Move the float accumulators (raw bits, kMagicBits + A) into this thread's int32
                // slots and restart them; the epilogue removes ndrains * kMagicBits.  The first
                // drain of an item overwrites what the previous item left in the slots.
                if (ndrains == 0) {
#pragma unroll
                    for (int i = 0; i < kTM; ++i)
#pragma unroll
                        for (int j = 0; j < TN; ++j) {
                            s.accs[(i * TN + j) * WS_CONS + t] = __float_as_int(accf[i][j]);
                            accf[i][j] = kMagic;
                        }
                } else {
#pragma unroll
                    for (int i = 0; i < kTM; ++i)
#pragma unroll
                        for (int j = 0; j < TN; ++j) {
                            red_shared_add(&s.accs[(i * TN + j) * WS_CONS + t], __float_as_int(accf[i][j]));
                            accf[i][j] = kMagic;
                        }
                }
                ++ndrains;
                since = 0;
            }
        }

        // ---- epilogue of the item ----------------------------------------------------------------
        // Negative weights of a column inside this unit's K range: counted by the producers while
        // they decode (tail_neg, the slots past K, belongs to the split that holds the last k-tile),
        // or read from the prefix counts that come with expanded weights.
        WS_T(t0 = clock64();)
        const int* negc = s.negc[seq & (S::NEGSETS - 1)];
        const int tailc = (cur.t_end == p.ntiles) ? p.tail_neg : 0;
        auto colcorr = [&](int col) -> int {
            if (PRE) {
                const int* np = p.negpre + cur.n0 + col;
                return __ldg(np + (long long)cur.t_end * p.npad) - __ldg(np + (long long)cur.t_begin * p.npad);
            }
            return negc[col] - tailc;
        };
        auto part = [&](int i, int j, long long) -> int {
            return s.accs[(i * TN + j) * WS_CONS + t] - ndrains * kMagicBits;
        };
        if (cur.tail_idx >= 0) {
            // Tail split: every CTA of the tile leaves its partial sums (negative-weight correction
            // included) in the workspace; the one that arrives last at the tile's counter adds them
            // up -- in a fixed order, each thread its own 8 x TN outputs -- and applies the epilogue.
            constexpr int SLOT = kTM * TN * WS_CONS;
            int* base = p.partials + (long long)cur.tail_idx * p.tail_splits * SLOT;
            int* mine = base + cur.sp * SLOT;
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                const int col = (TN == 8 && j >= 4) ? (BN / 2 + 4 * tn + j - 4) : (4 * tn + j);
                const int corr = colcorr(col);
#pragma unroll
                for (int i = 0; i < kTM; ++i) __stcg(mine + (i * TN + j) * WS_CONS + t, part(i, j, 0) + corr);
            }
            __threadfence();
            consumer_bar();
            if (t == 0) {
                int* cnt = p.counters + cur.tail_idx;
                const int prev = atomicAdd(cnt, 1);
                const int lastone = (prev == p.tail_splits - 1);
                if (lastone) *cnt = 0;  // ready for the next launch
                s.last_flag = lastone;
            }
            consumer_bar();
            if (s.last_flag) {
                __threadfence();
                store_tile<TN, CONV>(
                    p, cur.m0, cur.n0, tm, tn, BM, BN,
                    [&](int i, int j, long long) -> int {
                        int v = 0;
                        for (int q = 0; q < p.tail_splits; ++q) v += __ldcg(base + q * SLOT + (i * TN + j) * WS_CONS + t);
                        return v;
                    },
                    [&](int) -> int { return 0; });
            }
        } else if (p.splits == 1) {
            store_tile<TN, CONV>(p, cur.m0, cur.n0, tm, tn, BM, BN, part, colcorr);
        } else {
            // split-K: add the partial sums into the zeroed output; the CTA that arrives last at
            // this tile's counter reads the totals back and applies the epilogue in place.
            reduce_tile<TN, CONV>(p, cur.m0, cur.n0, tm, tn, BM, BN, part, colcorr);
            __threadfence();
            consumer_bar();
            if (t == 0) {
                int* cnt = p.counters + cur.tile_id;
                const int prev = atomicAdd(cnt, 1);
                const int lastone = (prev == p.splits - 1);
                if (lastone) *cnt = 0;  // ready for the next launch
                s.last_flag = lastone;
            }
            consumer_bar();
            if (s.last_flag) {
                __threadfence();
                const int* tot = static_cast<const int*>(p.out);
                store_tile<TN, CONV>(
                    p, cur.m0, cur.n0, tm, tn, BM, BN, [&](int, int, long long o) -> int { return __ldcg(tot + o); },
                    [&](int) -> int { return 0; });
            }
        }
        // All consumers have read this item's negative-weight counts before they are cleared for
        // a later item (the producers are filling other sets meanwhile).
        if (!PRE) {
            consumer_bar();
            for (int i = t; i < BN; i += WS_CONS) s.negc[seq & (S::NEGSETS - 1)][i] = 0;
        }
        WS_T(te += clock64() - t0;)
    }
    WS_T(if (blockIdx.x == 1 && lane == 0)
             printf("ws_timing consumer warp %d: cycles %lld wait_full %lld epilogue %lld k_tiles %d\n", warp,
                    clock64() - tstart, tw, te, git);)
    if (s.err) *p.err_flag = 1;
}

// Expands the packed weights of one launch into floats laid out as the k-tiles want them:
// wd[t * bk + j][n] = +-2^-r, 0 for a zero weight and for every slot beyond K or N, and counts the
// negative ones per (k-tile, column).  One thread per (column, k-tile), columns fastest.  bk need
// not be a multiple of the weights per packed word.
__global__ void __launch_bounds__(256) expand_weights_kernel(const GemmParams p, float* wd, int* negcnt)
{
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)p.npad * p.ntiles) return;
    const int t = int(idx / p.npad), n = int(idx - (long long)t * p.npad);
    const uint32_t fmask = (1u << p.dec.fw) - 1u;
    float* dst = wd + (long long)t * p.bk * p.npad + n;
    const int32_t* row = p.packed + (long long)n * p.dec.row_len;
    int negs = 0, have_word = -1;
    uint32_t w = 0;
    for (int j = 0; j < p.bk; ++j) {
        const int k = t * p.bk + j;
        const bool live = n < p.N && k < p.K;
        float v = 0.0f;
        if (live) {
            const int word = k / p.dec.num, slot = k - word * p.dec.num;
            if (word != have_word) {
                w = uint32_t(__ldg(row + word));
                have_word = word;
            }
            int neg;
            v = decode_f32((w >> (slot * p.dec.fw)) & fmask, p.dec, true, neg);
            negs += neg;
        }
        dst[(long long)j * p.npad] = v;
    }
    negcnt[idx] = negs;
}

// Exclusive prefix sums of the per-tile counts along the k-tiles: row t of `negpre` becomes the
// number of negative weights of the column in tiles 0 .. t-1, row ntiles the total.  A block
// takes 32 columns; its 32 warps each sum one segment of the tiles, exchange the segment sums
// through shared memory and then write the prefixes of their segment.
__global__ void __launch_bounds__(1024) negative_prefix_kernel(const int* __restrict__ negcnt, int* __restrict__ negpre,
                                                               int ntiles, int npad)
{
    __shared__ int seg[32][33];
    const int lane = threadIdx.x, sg = threadIdx.y;
    const int n = blockIdx.x * 32 + lane;
    const bool live = n < npad;
    const int per = (ntiles + 31) / 32;
    const int t0 = min(ntiles, sg * per), t1 = min(ntiles, t0 + per);
    int sum = 0;
    if (live)
        for (int t = t0; t < t1; ++t) sum += negcnt[(long long)t * npad + n];
    seg[sg][lane] = sum;
    __syncthreads();
    int run = 0;
    for (int q = 0; q < sg; ++q) run += seg[q][lane];
    if (!live) return;
    for (int t = t0; t < t1; ++t) {
        negpre[(long long)t * npad + n] = run;
        run += negcnt[(long long)t * npad + n];
    }
    if (sg == 31) negpre[(long long)ntiles * npad + n] = run;
}

// Chooses the k-tile, at most WS_BKT.  With packed weights decoded by the producers it is a
// multiple of num (whole packed words) and of the staging granularity (row mode: UR whole rows;
// table mode: 4 columns).  With expanded weights (`pre`) the row modes take any whole number of
// rows: the one that pads K least (7x7 windows on 3 channels: 7 tiles of 21 instead of 6 of 28).
template <int AM>
bool ws_choose_tile(GemmParams& p, bool pre)
{
    constexpr int KW = (AM == AM_QUAD3 || AM == AM_PAIR3) ? 3 : (AM == AM_S2K7 ? 7 : (AM >= 1 ? AM : 1));
    constexpr bool LIN = AM == AM_LINEAR;  // staged in 16-byte groups of four k
    constexpr int GRAN = AM >= 1 ? KW * ((KW == 1 || KW == 3) ? 4 : 2) : 4;
    constexpr int RMAX = (KW == 1) ? 28 : (KW == 3 ? 8 : 4);  // rows the producers have registers for
    int best = 0;
    if (pre && (AM >= 1 || LIN)) {
        long long best_padded = 0;
        for (int rows = RMAX; rows >= 1; --rows) {
            const int bk = rows * KW;
            if (LIN && bk % 4 != 0) continue;
            if (bk > WS_BKT || (bk < 12 && best)) continue;
            long long padded = ((long long)p.K + bk - 1) / bk * bk;
            // Linear layers have long K: there the fixed cost of a k-tile (hand-shake, loop set-up;
            // measured at about four k-steps) decides between tiles that pad K about equally.
            if (LIN) padded = padded / bk * (bk + 4);
            if (!best || padded < best_padded) {
                best = bk;
                best_padded = padded;
            }
        }
        if (!best) return false;
        p.bk = best;
        p.kt_words = 0;  // not used: the producers copy expanded weights
        p.rows_per_tile = best / KW;
        p.ntiles = (p.K + best - 1) / best;
        p.tail_neg = 0;  // expanded weights are 0 beyond K
    } else {
        for (int bk = WS_BKT; bk >= 2 && !best; --bk)
            if (bk % p.dec.num == 0 && bk % GRAN == 0) best = bk;
        if (!best) return false;
        p.bk = best;
        p.kt_words = best / p.dec.num;
        p.rows_per_tile = best / KW;
        p.ntiles = (p.dec.row_len + p.kt_words - 1) / p.kt_words;
        // Every slot from K to the end of the last tile decodes from a zero field, i.e. as -2^0.
        p.tail_neg = p.ntiles * p.bk - p.K;
    }
    p.flush_tiles /= p.bk;  // the caller left the number of terms that cannot overflow
    if (p.flush_tiles > 4096) p.flush_tiles = 4096;
    return p.flush_tiles >= 1;
}

inline int num_sms()
{
    static int sms[kMaxDevices];  // per device
    const int dev = device_slot();
    if (dev < 0) return 148;
    if (!sms[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        sms[dev] = n;
    }
    return sms[dev];
}

// Sets the shared-memory attribute of one kernel instantiation once and checks that it can be used.
template <int TN, int AM, bool PRE>
int ws_kernel_ready()
{
    static int states[kMaxDevices];  // per instantiation and device: 0 unknown, 1 usable, -1 not usable
    const int dev = device_slot();
    if (dev < 0) return DS_ERR_CUDA;
    int& attr_state = states[dev];
    if (attr_state == 0) {
        auto kern = ws_kernel<TN, AM, PRE>;
        cudaFuncAttributes fa;
        if (cudaFuncGetAttributes(&fa, kern) != cudaSuccess ||
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(WsSmem<TN>))) !=
                cudaSuccess) {
            cudaGetLastError();
            return DS_ERR_CUDA;
        }
        // The register hand-over in the kernel is sized for this launch allocation; with any
        // other one the consumers could wait for registers for ever, so the kernel is not used.
        attr_state = (fa.numRegs == WS_LAUNCH_REGS) ? 1 : -1;
    }
    return attr_state < 0 ? DS_ERR_UNSUPPORTED : DS_OK;
}

template <int TN, int AM>
int ws_launch_cfg(GemmParams p, cudaStream_t st)
{
    using S = WsSmem<TN>;
    const size_t smem = sizeof(S);
    const long long gx = ((long long)p.M + WS_BM - 1) / WS_BM, gy = (p.N + S::BN - 1) / S::BN;
    if (gx * gy > 500000000LL) return DS_ERR_RANGE;
    const long long tiles = gx * gy;
    const int sms = num_sms();
    constexpr long long SLOT_BYTES = (long long)kTM * TN * WS_CONS * 4;
    // Expanded weights: when many row tiles would each decode the same packed words again, decode
    // them once per launch into the front of the workspace (two small kernels ahead of this one).
    const GemmParams p_in = p;
    bool pre = false;
    if ((p.partials || p.prepared || p.prepare_only) && gx >= 8 && ws_kernel_ready<TN, AM, true>() == DS_OK &&
        ws_choose_tile<AM>(p, true)) {
        p.npad = int(gy) * S::BN;
        const long long wd_floats = (long long)p.ntiles * p.bk * p.npad;
        const long long neg_ints = (long long)(p.ntiles + 1) * p.npad, cnt_ints = (long long)p.ntiles * p.npad;
        const long long need = ((wd_floats + neg_ints + cnt_ints) * 4 + 255) / 256 * 256;
        auto expand_into = [&](int* base) {
            float* wd = reinterpret_cast<float*>(base);
            int* negpre = base + wd_floats;
            int* negcnt = negpre + neg_ints;
            p.wd = wd;
            p.negpre = negpre;
            const long long threads = (long long)p.npad * p.ntiles;
            expand_weights_kernel<<<unsigned((threads + 255) / 256), 256, 0, st>>>(p, wd, negcnt);
            negative_prefix_kernel<<<(p.npad + 31) / 32, dim3(32, 32), 0, st>>>(negcnt, negpre, p.ntiles, p.npad);
            note_launch(2);
            return cudaGetLastError() == cudaSuccess;
        };
        if (p.prepare_only) {
            // ds_conv2d_prepare: report the size; fill the caller's buffer if there is one
            *p.needed_out = need;
            if (!p.prepared) return DS_OK;
            if (need > p.prepared_bytes) return DS_ERR_SCRATCH;
            return expand_into(static_cast<int*>(const_cast<void*>(p.prepared))) ? DS_OK : DS_ERR_CUDA;
        }
        if (p.prepared && need <= p.prepared_bytes) {
            // expanded ahead of time for this geometry: same layout as expand_into writes
            p.wd = static_cast<const float*>(p.prepared);
            p.negpre = static_cast<const int*>(p.prepared) + wd_floats;
            pre = true;
        } else if (p.partials && need <= p.partial_bytes) {
            int* base = p.partials;
            p.partials += need / 4;
            p.partial_bytes -= need;
            if (!expand_into(base)) return DS_ERR_CUDA;
            pre = true;
        }
    }
    if (p.prepare_only) return DS_OK;  // this geometry does not use expanded weights
    if (!pre) {
        p = p_in;
        if (!ws_choose_tile<AM>(p, false)) return DS_ERR_UNSUPPORTED;
        if (int rc = ws_kernel_ready<TN, AM, false>()) return rc;
        p.npad = int(gy) * S::BN;
    }
    p.splits = 1;
    p.tiles_per_split = p.ntiles;
    p.tail_items = 0;
    p.tail_splits = 1;
    if (p.counters && p.partials && p.ntiles >= 12 && tiles % sms != 0) {
        // Tail split: the tiles beyond the last full wave are cut along K so that the CTAs which
        // would idle during that wave share its work.  cost = length of the tail in tile times.
        const long long full = tiles / sms * sms;
        const int tail = int(tiles - full);
        double best = 1.0;
        for (int sp = 2; sp <= 4; ++sp) {
            if (p.ntiles / sp < 4) break;
            if ((long long)tail * sp * SLOT_BYTES > p.partial_bytes || tail > p.counter_slots) break;
            const long long rounds = ((long long)tail * sp + sms - 1) / sms;
            const double cost = double(rounds) / sp + 0.04;  // + writing and re-reading the partial sums
            if (cost < best - 0.05) {
                best = cost;
                p.tail_splits = sp;
            }
        }
        if (p.tail_splits > 1) {
            p.tail_items = tail;
            p.tail_first = int(full);
            p.tail_tps = (p.ntiles + p.tail_splits - 1) / p.tail_splits;
            p.tail_splits = (p.ntiles + p.tail_tps - 1) / p.tail_tps;
        }
    } else if (p.counters && !p.partials && tiles <= p.counter_slots && p.ntiles >= 16 && !p.gate &&
               static_cast<const void*>(p.residual) != p.out) {
        // (not for a gated launch either: zeroing the output would undo the other path's result)
        // (an in-place residual add, residual == out, would be wiped by the zeroing below)
        // Split-K of every tile through integer atomics on the zeroed output, for callers whose
        // workspace holds counters only: used when the tiles alone fill the SMs badly.
        auto eff = [&](int sp) {
            const long long ctas = tiles * sp, waves = (ctas + sms - 1) / sms;
            return double(ctas) / double(waves * sms);
        };
        double best = eff(1);
        for (int sp = 2; sp <= 4; ++sp) {
            if (p.ntiles / sp < 8) break;
            const double e = eff(sp) * 0.92;  // measured cost of zeroing, atomics and the second pass
            if (e > best * 1.05) {
                best = e;
                p.splits = sp;
            }
        }
        if (p.splits > 1) {
            p.tiles_per_split = (p.ntiles + p.splits - 1) / p.splits;
            p.splits = (p.ntiles + p.tiles_per_split - 1) / p.tiles_per_split;
            if (cudaMemsetAsync(p.out, 0, size_t(p.M) * size_t(p.N) * 4, st) != cudaSuccess) return DS_ERR_CUDA;
        }
    }
    p.grid_m = int(gx);
    p.grid_n = int(gy);
    p.full_units = p.tail_items ? p.tail_first : int(tiles * p.splits);
    const long long items = (long long)p.full_units + (long long)p.tail_items * p.tail_splits;
    const dim3 grid((unsigned)(items < sms ? items : sms));
    if (pre) ws_kernel<TN, AM, true><<<grid, WS_NT, smem, st>>>(p);
    else ws_kernel<TN, AM, false><<<grid, WS_NT, smem, st>>>(p);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
}

template <int AM>
int ws_launch_am(const GemmParams& p, cudaStream_t st)
{
    if (p.N > 64) return ws_launch_cfg<8, AM>(p, st);  // 256 x 128
    return ws_launch_cfg<4, AM>(p, st);                // 256 x 64
}

}  // namespace
}  // namespace ds
