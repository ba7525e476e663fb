// Shift convolution on staged activations for sm_100a: TMA-fed, warp-specialised, persistent.
//
// Arithmetic: the FP32-pipe path of ds_gemm.cu (one FFMA with round-toward-minus-infinity per
// term into magic-offset accumulators, drained into int32 slots in shared memory).  What differs
// is how the operands reach shared memory:
//
//   * x: the staged tensor (fp32 NHWC with a physical halo of 0.5, see ds_staged.cuh) is read by
//     the tensor memory accelerator in im2col mode.  One `cp.async.bulk.tensor.4d ... im2col`
//     brings, for 256 consecutive output positions (b, oh, ow) and one filter tap (kh, kw), four
//     channels (16 bytes) per position -- the hardware walks the positions across row and image
//     boundaries with the convolution's stride.  No thread computes an address, tests a border or
//     converts a value: the im2col matrix exists neither in HBM nor in anybody's registers.
//   * w: expanded once per layer (ds_staged_prepare) into +-2^-r floats, in exactly the order a
//     k-tile wants them in shared memory, so a k-tile of weights is ONE bulk copy.
//   * k runs over (kh, kw, c) with c fastest (integer sums do not depend on the order of their
//     terms, so the result is still bit-identical to the reference's (c, kh, kw) order).
//
// Shared-memory layout of a stage: A[kq][row][4] (kq = group of four consecutive k, as TMA delivers
// it: four channels of a pixel are 16 contiguous bytes) and B[k][column] floats.  A consumer
// thread holds four rows x four k of A (four float4) and, per k, eight columns of B (two float4):
// 24 fragment loads per 256 FFMAs, every load a conflict-free 128-byte or broadcast 64-byte access.
//
// Roles: 16 consumer warps (8 x 8 outputs per thread: 256 x 128 tile, or 512 x 64 for layers with
// at most 64 output channels) and one producer warp whose lane 0 issues the copies.  STAGES-deep
// ring, full[s] (transaction bytes) / empty[s] (one arrival per consumer warp) mbarriers.  Every
// wait is bounded; a wait that gives up sets a flag (ds_last_kernel_error) and the kernel ends.
#include <cuda.h>

#include "ds_staged.cuh"

namespace ds {
namespace {

constexpr int ST_CONS = 512;
constexpr int ST_PROD = 128;  // one warp group, so that it can hand its registers over; only lane 0 of its first warp works
constexpr int ST_NT = ST_CONS + ST_PROD;
// Registers: the CTA starts with 640 * 96; the producer group keeps 24 each, which frees
// 128 * 72 = 9216, and the consumers take 512 * 16 = 8192 of them for 112 each (the 8 x 8 float
// accumulators, eight float4 weight fragments and a float4 of x).
constexpr int ST_LAUNCH_REGS = 96, ST_PROD_REGS = 24, ST_CONS_REGS = 112;
static_assert(ST_CONS * (ST_CONS_REGS - ST_LAUNCH_REGS) <= ST_PROD * (ST_LAUNCH_REGS - ST_PROD_REGS), "register pool");
constexpr int ST_WAIT_LIMIT = 1 << 12;
constexpr unsigned ST_WAIT_NS = 1000000;

template <int BN>
struct StCfg {
    static constexpr int TN = 8;
    static constexpr int TNG = BN / TN;        // threads along n
    static constexpr int TMG = ST_CONS / TNG;  // threads along m
    static constexpr int BM = TMG * kTM;       // 256 (BN = 128) or 512 (BN = 64)
    static constexpr int KQ = (BN == 128) ? 4 : 2;      // groups of four k per stage
    static constexpr int STAGES = (BN == 128) ? 4 : 5;
    static constexpr int A_BYTES = KQ * BM * 16;
    static constexpr int B_BYTES = KQ * BN * 16;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int ACC_BYTES = kTM * TN * ST_CONS * 4;
    static constexpr int OFF_ACC = STAGES * STAGE_BYTES;
    static constexpr int OFF_BAR = OFF_ACC + ACC_BYTES;
    static constexpr int SMEM_BYTES = OFF_BAR + 2 * STAGES * 8 + 16 + 1024;  // + slack to align the base
    static_assert(STAGE_BYTES % 1024 == 0, "stage alignment");
    static_assert(SMEM_BYTES <= 232448, "shared memory");
};

__device__ __forceinline__ unsigned st_smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void st_mbar_init(unsigned bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void st_mbar_arrive(unsigned bar)
{
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void st_mbar_expect_tx(unsigned bar, unsigned bytes)
{
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes)
                 : "memory");
}

// Bounded wait, see mbar_wait in ds_gemm_ws.cuh.
__device__ __forceinline__ bool st_mbar_wait(unsigned bar, unsigned parity, bool gave_up)
{
    const int limit = gave_up ? 1 : ST_WAIT_LIMIT;
    for (int i = 0; i < limit; ++i) {
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity), "r"(ST_WAIT_NS)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// 256 output positions starting at (q, p, n) x four channels starting at c, filter tap (kw, kh):
// box [256][4] floats = 4 KiB into `dst`, transaction bytes on `bar`.
__device__ __forceinline__ void st_tma_im2col(unsigned dst, const CUtensorMap* map, unsigned bar, int c, int w, int h,
                                              int n, unsigned short kw, unsigned short kh)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
        :
        : "r"(dst), "l"(reinterpret_cast<unsigned long long>(map)), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(kw),
          "h"(kh)
        : "memory");
}

// Plain bulk copy global -> shared (both 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void st_bulk_copy(unsigned dst, const void* src, unsigned bytes, unsigned bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void st_consumer_bar() { asm volatile("bar.sync 2, %0;" ::"n"(ST_CONS) : "memory"); }

struct StItem {
    int m0, n0, nt, t_begin, t_end, tile_id, tail_idx, sp;
};

__device__ __forceinline__ StItem st_item(const StagedConvParams& p, int unit, int BM, int BN)
{
    StItem w;
    int tile, tps;
    if (unit < p.full_units) {
        w.sp = 0;
        tile = unit;
        tps = p.ntiles;
        w.tail_idx = -1;
    } else {
        const int v = unit - p.full_units;
        w.sp = v / p.tail_items;
        w.tail_idx = v - w.sp * p.tail_items;
        tile = p.tail_first + w.tail_idx;
        tps = p.tail_tps;
    }
    w.nt = tile / p.grid_m;
    const int mt = tile - w.nt * p.grid_m;
    w.m0 = mt * BM;
    w.n0 = w.nt * BN;
    w.t_begin = w.sp * tps;
    w.t_end = min(p.ntiles, w.t_begin + tps);
    w.tile_id = tile;
    return w;
}

template <int BN>
__global__ void __launch_bounds__(ST_NT, 1) staged_conv_kernel(const __grid_constant__ CUtensorMap xmap,
                                                                const StagedConvParams p)
{
    using C = StCfg<BN>;
    constexpr int BM = C::BM, KQ = C::KQ, STAGES = C::STAGES, TN = C::TN, TMG = C::TMG, TNG = C::TNG;
    extern __shared__ unsigned char st_smem_raw[];
    // TMA destinations want 128-byte alignment; the base is rounded up to 1024.
    const unsigned base = (st_smem_u32(st_smem_raw) + 1023u) & ~1023u;
    unsigned char* gbase = st_smem_raw + (base - st_smem_u32(st_smem_raw));
    const unsigned bar_full = base + C::OFF_BAR, bar_empty = bar_full + STAGES * 8;
    int* accs = reinterpret_cast<int*>(gbase + C::OFF_ACC);
    int* flags = reinterpret_cast<int*>(gbase + C::OFF_BAR + 2 * STAGES * 8);  // [0] last_flag

    const int t = threadIdx.x;
    const int total_items = p.full_units + p.tail_items * p.tail_splits;
    if (t == 0) {
        for (int i = 0; i < STAGES; ++i) {
            st_mbar_init(bar_full + 8 * i, 1);
            st_mbar_init(bar_empty + 8 * i, ST_CONS / 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (t >= ST_CONS) {
        // ================================ producer ===============================================
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(ST_PROD_REGS));
        if (t != ST_CONS) return;
        bool bad = false;
        int git = 0;
        for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
            const StItem cur = st_item(p, item, BM, BN);
            // first output position of each 256-row half of the tile, as TMA coordinates
            int cw[BM / 256], ch[BM / 256], cn[BM / 256];
#pragma unroll
            for (int hlf = 0; hlf < BM / 256; ++hlf) {
                const int m = cur.m0 + 256 * hlf;
                const int n = m / p.P, pp = m - n * p.P;
                const int oh = pp / p.OW, ow = pp - oh * p.OW;
                cw[hlf] = ow * p.sw;
                ch[hlf] = oh * p.sh;
                cn[hlf] = n;
            }
            const char* wsrc = reinterpret_cast<const char*>(p.wt) + (size_t)cur.nt * p.ntiles * C::B_BYTES;
            for (int tile = cur.t_begin; tile < cur.t_end; ++tile, ++git) {
                const int s = git % STAGES;
                if (git >= STAGES && !st_mbar_wait(bar_empty + 8 * s, unsigned(git / STAGES - 1) & 1u, bad)) bad = true;
                const int kq0 = tile * KQ;
                const int nq = min(KQ, p.nkq - kq0);
                const unsigned full = bar_full + 8 * s;
                st_mbar_expect_tx(full, unsigned(nq * BM * 16 + C::B_BYTES));
                const unsigned sa = base + s * C::STAGE_BYTES;
                st_bulk_copy(sa + C::A_BYTES, wsrc + (size_t)tile * C::B_BYTES, C::B_BYTES, full);
                int tap = kq0 / p.cq_per_tap, cq = kq0 - tap * p.cq_per_tap;
                for (int q = 0; q < nq; ++q) {
                    const int kh = tap / p.KW, kw = tap - kh * p.KW;
#pragma unroll
                    for (int hlf = 0; hlf < BM / 256; ++hlf)
                        st_tma_im2col(sa + (q * BM + 256 * hlf) * 16, &xmap, full, 4 * cq, cw[hlf], ch[hlf], cn[hlf],
                                      (unsigned short)kw, (unsigned short)kh);
                    if (++cq == p.cq_per_tap) {
                        cq = 0;
                        ++tap;
                    }
                }
            }
        }
        if (bad) *p.err_flag = 1;
        return;
    }

    // ================================== consumers =================================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(ST_CONS_REGS));
    const int lane = t & 31, warp = t >> 5;
    constexpr int WMG = TMG / 8;  // warps along m
    const int tm = (warp % WMG) * 8 + (lane & 7);
    const int tn = (warp / WMG) * 4 + (lane >> 3);
    float accf[kTM][TN];
    bool bad = false;
    int git = 0;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
        const StItem cur = st_item(p, item, BM, BN);
        const int my_tiles = cur.t_end - cur.t_begin;
#pragma unroll
        for (int i = 0; i < kTM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) accf[i][j] = kMagic;
        int ndrains = 0, since = 0;
        for (int it = 0; it < my_tiles; ++it, ++git) {
            const int s = git % STAGES;
            if (!st_mbar_wait(bar_full + 8 * s, unsigned(git / STAGES) & 1u, bad)) bad = true;
            const float4* sa = reinterpret_cast<const float4*>(gbase + s * C::STAGE_BYTES) + tm;
            const float* sb = reinterpret_cast<const float*>(gbase + s * C::STAGE_BYTES + C::A_BYTES) + 4 * tn;
            const int nq = min(KQ, p.nkq - (cur.t_begin + it) * KQ);  // groups of this tile that hold data
#pragma unroll
            for (int kq = 0; kq < KQ; ++kq) {
                if (kq < nq) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        float4 a[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) a[i] = sa[kq * BM + (4 * h + i) * TMG];
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            float b[TN];
                            *reinterpret_cast<float4*>(&b[0]) = *reinterpret_cast<const float4*>(sb + (kq * 4 + kk) * BN);
                            *reinterpret_cast<float4*>(&b[4]) =
                                *reinterpret_cast<const float4*>(sb + (kq * 4 + kk) * BN + BN / 2);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float av = kk == 0 ? a[i].x : (kk == 1 ? a[i].y : (kk == 2 ? a[i].z : a[i].w));
#pragma unroll
                                for (int j = 0; j < TN; ++j) accf[4 * h + i][j] = __fmaf_rd(av, b[j], accf[4 * h + i][j]);
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) st_mbar_arrive(bar_empty + 8 * s);
            if (++since == p.flush_tiles || it + 1 == my_tiles) {
                if (ndrains == 0) {
#pragma unroll
                    for (int i = 0; i < kTM; ++i)
#pragma unroll
                        for (int j = 0; j < TN; ++j) {
                            accs[(i * TN + j) * ST_CONS + t] = __float_as_int(accf[i][j]);
                            accf[i][j] = kMagic;
                        }
                } else {
#pragma unroll
                    for (int i = 0; i < kTM; ++i)
#pragma unroll
                        for (int j = 0; j < TN; ++j) {
                            red_shared_add(&accs[(i * TN + j) * ST_CONS + t], __float_as_int(accf[i][j]));
                            accf[i][j] = kMagic;
                        }
                }
                ++ndrains;
                since = 0;
            }
        }

        // ---- epilogue --------------------------------------------------------------------------
        // thread (tm, tn): rows m0 + i*TMG + tm, columns n0 + (j/4)*(BN/2) + 4*tn + (j%4)
        int addc[TN];  // per column: negative-weight correction of this K range, and (below) the bias
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int* np = p.negpre + cur.n0 + (j >> 2) * (BN / 2) + 4 * tn + (j & 3);
            addc[j] = __ldg(np + (size_t)cur.t_end * p.npad) - __ldg(np + (size_t)cur.t_begin * p.npad) -
                      ndrains * kMagicBits;
        }
        bool finish_tile = true;
        if (cur.tail_idx >= 0) {
            // Tail split: every CTA of the tile leaves its partial sums in the workspace; the one that
            // arrives last at the tile's counter adds them up, each thread its own outputs, and goes on.
            constexpr int SLOT = kTM * TN * ST_CONS;
            int* basep = p.partials + (size_t)cur.tail_idx * p.tail_splits * SLOT;
            int* mine = basep + (size_t)cur.sp * SLOT;
#pragma unroll
            for (int i = 0; i < kTM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j)
                    __stcg(mine + (i * TN + j) * ST_CONS + t, accs[(i * TN + j) * ST_CONS + t] + addc[j]);
            __threadfence();
            st_consumer_bar();
            if (t == 0) {
                int* cnt = p.counters + cur.tail_idx;
                const int prev = atomicAdd(cnt, 1);
                const int lastone = (prev == p.tail_splits - 1);
                if (lastone) *cnt = 0;  // ready for the next launch
                flags[0] = lastone;
            }
            st_consumer_bar();
            finish_tile = flags[0] != 0;
            st_consumer_bar();  // flags[0] is rewritten by the next tail item
            if (finish_tile) {
                __threadfence();
                // totals back into this thread's slots, so that the code below serves both cases
#pragma unroll
                for (int i = 0; i < kTM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j) {
                        int a = 0;
                        for (int q = 0; q < p.tail_splits; ++q)
                            a += __ldcg(basep + (size_t)q * SLOT + (i * TN + j) * ST_CONS + t);
                        accs[(i * TN + j) * ST_CONS + t] = a;
                    }
#pragma unroll
                for (int j = 0; j < TN; ++j) addc[j] = 0;
            }
        }
        if (finish_tile) {
            if (p.bias) {
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    const int n = cur.n0 + (j >> 2) * (BN / 2) + 4 * tn + (j & 3);
                    if (n < p.N) addc[j] += __ldg(p.bias + n);
                }
            }
            const bool vec = (p.N & 3) == 0;  // then a group of four columns is inside N or outside it
            const bool need_pix = p.out_staged || p.out_nchw;
#pragma unroll 1
            for (int i = 0; i < kTM; ++i) {
                const int m = cur.m0 + i * TMG + tm;
                if (m >= p.M) break;
                int b = 0, pp = 0, oh = 0, ow = 0;
                if (need_pix) {
                    // m = (b, oh, ow); floor(2^32/d) multipliers are at most one short of the quotient
                    b = int(__umulhi(unsigned(m), p.inv_P));
                    pp = m - b * p.P;
                    if (pp >= p.P) { pp -= p.P; ++b; }
                    oh = int(__umulhi(unsigned(pp), p.inv_OW));
                    ow = pp - oh * p.OW;
                    if (ow >= p.OW) { ow -= p.OW; ++oh; }
                }
                const size_t orow = (size_t)m * p.N;
                const size_t srow = need_pix && p.out_staged
                    ? (((size_t)b * p.os_H2 + oh + p.os_halo) * p.os_W2 + ow + p.os_halo) * p.os_Cs : 0;
#pragma unroll
                for (int h = 0; h < TN / 4; ++h) {
                    const int n = cur.n0 + h * (BN / 2) + 4 * tn;
                    if (n >= p.N) continue;
                    int v[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) v[e] = accs[(i * TN + 4 * h + e) * ST_CONS + t] + addc[4 * h + e];
                    if (p.residual) {
                        int r4[4] = {0, 0, 0, 0};
                        if (vec) {
                            const int4 r = __ldg(reinterpret_cast<const int4*>(p.residual + orow + n));
                            r4[0] = r.x; r4[1] = r.y; r4[2] = r.z; r4[3] = r.w;
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                if (n + e < p.N) r4[e] = __ldg(p.residual + orow + n + e);
                        }
                        // fp32 add of the two values as the reference's `out += identity` does it
#pragma unroll
                        for (int e = 0; e < 4; ++e) v[e] = __float2int_rn(__int2float_rn(v[e]) + __int2float_rn(r4[e]));
                    }
                    if (p.relu) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) v[e] = max(v[e], 0);
                    }
                    if (p.round_f32) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) v[e] = __float2int_rn(__int2float_rn(v[e]));
                    }
                    if (p.out_codes) {
                        if (vec) {
                            *reinterpret_cast<int4*>(p.out_codes + orow + n) = make_int4(v[0], v[1], v[2], v[3]);
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                if (n + e < p.N) p.out_codes[orow + n + e] = v[e];
                        }
                    }
                    if (p.out_f32) {
                        if (vec) {
                            *reinterpret_cast<float4*>(p.out_f32 + orow + n) =
                                make_float4(__int2float_rn(v[0]) * p.inv_scale, __int2float_rn(v[1]) * p.inv_scale,
                                            __int2float_rn(v[2]) * p.inv_scale, __int2float_rn(v[3]) * p.inv_scale);
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                if (n + e < p.N) p.out_f32[orow + n + e] = __int2float_rn(v[e]) * p.inv_scale;
                        }
                    }
                    if (p.out_nchw) {
                        const size_t on = ((size_t)b * p.N + n) * p.P + pp;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            if (n + e >= p.N) continue;
                            if (p.out_nchw_f32)
                                static_cast<float*>(p.out_nchw)[on + (size_t)e * p.P] = __int2float_rn(v[e]) * p.inv_scale;
                            else
                                static_cast<int*>(p.out_nchw)[on + (size_t)e * p.P] = v[e];
                        }
                    }
                    if (p.out_staged) {
                        // channels n .. n+3 of one pixel: 16 bytes (os_Cs is a multiple of 4 >= N)
                        float f[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            int c = min(max(v[e], p.rq_lo), p.rq_hi);
                            if (p.rq_mul != 1) c = c * p.rq_mul + p.rq_add;
                            f[e] = (n + e < p.N) ? (__int2float_rn(c) + 0.5f) : 0.5f;
                        }
                        *reinterpret_cast<float4*>(p.out_staged + srow + n) = make_float4(f[0], f[1], f[2], f[3]);
                    }
                }
            }
        }
    }
    if (bad) *p.err_flag = 1;
}

// Expands packed weights into the layout the kernel copies per k-tile:
//   wt[nt][t][kl][nl] = weight(n = nt*BN + nl, k' = t*4*KQ + kl),  k' = tap * Cs + c  (tap = kh*KW + kw),
// the reference's k being c*KH*KW + tap; 0 for c >= C, tap >= KH*KW, n >= N and zero weights.
// negcnt[t][n] counts the negative ones.  One thread per (k-tile, column).
template <int BN>
__global__ void __launch_bounds__(256) staged_expand_kernel(const int32_t* __restrict__ packed, Decode dec, int C, int Cs,
                                                            int taps, int N, int ntiles, int npad,
                                                            float* __restrict__ wt, int* __restrict__ negcnt)
{
    constexpr int KT = 4 * StCfg<BN>::KQ;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // (tile, n)
    if (idx >= (long long)ntiles * npad) return;
    const int tl = int(idx / npad), n = int(idx - (long long)tl * npad);
    const int nt = n / BN, nl = n - nt * BN;
    const uint32_t fmask = (1u << dec.fw) - 1u;
    float* dst = wt + ((size_t)nt * ntiles + tl) * (KT * BN) + nl;
    int negs = 0;
    for (int kl = 0; kl < KT; ++kl) {
        const int kp = tl * KT + kl;
        const int tap = kp / Cs, c = kp - tap * Cs;
        float v = 0.f;
        if (n < N && tap < taps && c < C) {
            const int k = c * taps + tap;
            const int word = k / dec.num, sl = k - word * dec.num;
            const uint32_t w = uint32_t(__ldg(packed + (size_t)n * dec.row_len + word));
            int neg;
            v = decode_f32((w >> (sl * dec.fw)) & fmask, dec, true, neg);
            negs += neg;
        }
        dst[(size_t)kl * BN] = v;
    }
    negcnt[idx] = negs;
}

// Exclusive prefix sums along the k-tiles (one thread per column; ntiles is at most a few hundred).
__global__ void staged_prefix_kernel(const int* __restrict__ negcnt, int* __restrict__ negpre, int ntiles, int npad)
{
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= npad) return;
    int run = 0;
    for (int t = 0; t < ntiles; ++t) {
        negpre[(size_t)t * npad + n] = run;
        run += negcnt[(size_t)t * npad + n];
    }
    negpre[(size_t)ntiles * npad + n] = run;
}

// ---- host side -----------------------------------------------------------------------------------
using EncodeIm2colFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const int*, const int*, cuuint32_t, cuuint32_t, const cuuint32_t*,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

EncodeIm2colFn encode_im2col_fn()
{
    static EncodeIm2colFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeIm2colFn>(ptr);
        else
            cudaGetLastError();
    }
    return fn;
}

struct StGeom {
    int BN, KQ, nkq, ntiles, grid_n, npad;
    long long wt_floats, neg_ints, cnt_ints, bytes;
};

StGeom st_geometry(int Cs, int taps, int N)
{
    StGeom g;
    g.BN = (N > 64) ? 128 : 64;
    g.KQ = (N > 64) ? StCfg<128>::KQ : StCfg<64>::KQ;
    g.nkq = taps * (Cs / 4);
    g.ntiles = (g.nkq + g.KQ - 1) / g.KQ;
    g.grid_n = (N + g.BN - 1) / g.BN;
    g.npad = g.grid_n * g.BN;
    g.wt_floats = (long long)g.grid_n * g.ntiles * g.KQ * g.BN * 4;
    g.neg_ints = (long long)(g.ntiles + 1) * g.npad;
    g.cnt_ints = (long long)g.ntiles * g.npad;
    g.bytes = ((g.wt_floats + g.neg_ints + g.cnt_ints) * 4 + 255) / 256 * 256;
    return g;
}

template <int BN>
int st_kernel_ready()
{
    static int states[kMaxDevices];
    const int dev = device_slot();
    if (dev < 0) return DS_ERR_CUDA;
    if (states[dev] == 0) {
        cudaFuncAttributes fa;
        if (cudaFuncGetAttributes(&fa, staged_conv_kernel<BN>) != cudaSuccess ||
            cudaFuncSetAttribute(staged_conv_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 StCfg<BN>::SMEM_BYTES) != cudaSuccess) {
            cudaGetLastError();
            states[dev] = -1;
        } else {
            // The register hand-over is sized for this launch allocation; with any other one the
            // consumers could wait for registers for ever, so the kernel is not used.
            states[dev] = (fa.numRegs == ST_LAUNCH_REGS) ? 1 : -1;
        }
    }
    return states[dev] > 0 ? DS_OK : DS_ERR_UNSUPPORTED;
}

inline int st_num_sms()
{
    static int sms[kMaxDevices];
    const int dev = device_slot();
    if (dev < 0) return 148;
    if (!sms[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        sms[dev] = n;
    }
    return sms[dev];
}

template <int BN>
int st_launch(const CUtensorMap& map, StagedConvParams p, void* workspace, long long workspace_bytes, cudaStream_t st)
{
    using C = StCfg<BN>;
    if (int rc = st_kernel_ready<BN>()) return rc;
    const long long gx = ((long long)p.M + C::BM - 1) / C::BM;
    const long long tiles = gx * p.grid_n;
    if (tiles > 500000000LL) return DS_ERR_RANGE;
    const int sms = st_num_sms();
    p.grid_m = int(gx);
    p.full_units = int(tiles);
    p.tail_first = p.tail_items = 0;
    p.tail_splits = 1;
    p.tail_tps = p.ntiles;
    p.counters = nullptr;
    p.partials = nullptr;
    constexpr long long SLOT_BYTES = (long long)kTM * C::TN * ST_CONS * 4;
    if (workspace && workspace_bytes > (long long)kWorkspaceCounters * 4 && p.ntiles >= 12 && tiles % sms != 0) {
        // Tail split (see ws_launch_cfg in ds_gemm_ws.cuh): the tiles after the last full wave are
        // cut along K so that the SMs which would idle during that wave share them.
        const long long partial_bytes = workspace_bytes - (long long)kWorkspaceCounters * 4;
        const long long full = tiles / sms * sms;
        const int tail = int(tiles - full);
        double best = 1.0;
        int splits = 1;
        for (int sp = 2; sp <= 4; ++sp) {
            if (p.ntiles / sp < 4) break;
            if ((long long)tail * sp * SLOT_BYTES > partial_bytes || tail > kWorkspaceGateSlot) break;
            const long long rounds = ((long long)tail * sp + sms - 1) / sms;
            const double cost = double(rounds) / sp + 0.04;
            if (cost < best - 0.05) {
                best = cost;
                splits = sp;
            }
        }
        if (splits > 1) {
            p.tail_items = tail;
            p.tail_first = int(full);
            p.tail_tps = (p.ntiles + splits - 1) / splits;
            p.tail_splits = (p.ntiles + p.tail_tps - 1) / p.tail_tps;
            p.full_units = int(full);
            p.counters = static_cast<int*>(workspace);
            p.partials = p.counters + kWorkspaceCounters;
        }
    }
    const long long items = (long long)p.full_units + (long long)p.tail_items * p.tail_splits;
    const unsigned grid = unsigned(items < sms ? items : sms);
    staged_conv_kernel<BN><<<grid, ST_NT, C::SMEM_BYTES, st>>>(map, p);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
}

}  // namespace
}  // namespace ds

using namespace ds;

extern "C" long long ds_staged_bytes(int B, int H, int W, int C, int halo)
{
    if (B < 0 || H <= 0 || W <= 0 || C <= 0 || halo < 0) return -1;
    return (long long)B * (H + 2 * halo) * (W + 2 * halo) * ((C + 3) / 4 * 4) * 4;
}

extern "C" int ds_staged_prepare(const int32_t* packed, int C, int OC, int KH, int KW, int bits, int base,
                                 void* prepared, long long prepared_bytes, long long* bytes_needed, void* stream)
{
    if (!packed || !bytes_needed || C <= 0 || OC <= 0 || KH <= 0 || KW <= 0) return DS_ERR_BAD_ARG;
    if (bits < 1 || bits > 7 || base != 0 || KH > 31 || KW > 31) return DS_ERR_UNSUPPORTED;
    const int Cs = (C + 3) / 4 * 4, taps = KH * KW;
    const long long K = (long long)C * taps;
    if (K > 2147483647LL || (long long)Cs * taps > 2147483647LL) return DS_ERR_RANGE;
    const StGeom g = st_geometry(Cs, taps, OC);
    *bytes_needed = g.bytes;
    if (!prepared) return DS_OK;
    if (prepared_bytes < g.bytes) return DS_ERR_SCRATCH;
    if (reinterpret_cast<uintptr_t>(prepared) & 15u) return DS_ERR_ALIGN;
    Decode dec;
    dec.bits = bits;
    dec.fw = bits + 1;
    dec.num = 32 / (bits + 1);
    dec.base = base;
    dec.row_len = int((K + dec.num - 1) / dec.num);
    float* wt = static_cast<float*>(prepared);
    int* negpre = reinterpret_cast<int*>(wt + g.wt_floats);
    int* negcnt = negpre + g.neg_ints;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long threads = (long long)g.ntiles * g.npad;
    const unsigned blocks = unsigned((threads + 255) / 256);
    if (g.BN == 128)
        staged_expand_kernel<128><<<blocks, 256, 0, st>>>(packed, dec, C, Cs, taps, OC, g.ntiles, g.npad, wt, negcnt);
    else
        staged_expand_kernel<64><<<blocks, 256, 0, st>>>(packed, dec, C, Cs, taps, OC, g.ntiles, g.npad, wt, negcnt);
    staged_prefix_kernel<<<(g.npad + 127) / 128, 128, 0, st>>>(negcnt, negpre, g.ntiles, g.npad);
    note_launch(2);
    return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
}

extern "C" int ds_staged_conv2d(const ds_staged_t* x, const void* prepared, long long prepared_bytes,
                                const int32_t* bias, int OC, int KH, int KW, int sh, int sw, int ph, int pw,
                                const ds_staged_out_t* out, void* workspace, long long workspace_bytes, void* stream)
{
    if (!x || !x->data || !prepared || !out || OC <= 0 || KH <= 0 || KW <= 0 || sh <= 0 || sw <= 0 || ph < 0 || pw < 0)
        return DS_ERR_BAD_ARG;
    if (x->B < 0 || x->H <= 0 || x->W <= 0 || x->C <= 0 || x->halo < ph || x->halo < pw) return DS_ERR_BAD_ARG;
    if (KH > 31 || KW > 31 || sh > 8 || sw > 8) return DS_ERR_UNSUPPORTED;
    if (x->H + 2 * ph < KH || x->W + 2 * pw < KW) return DS_ERR_BAD_ARG;
    if (x->B == 0) return DS_OK;
    const int I = out->act_integer_bits, F = out->act_fraction_bits;
    if (F < 0 || F > 16) return DS_ERR_BAD_ARG;
    if (!out->codes && !out->f32 && !out->nchw && !(out->staged && out->staged->data)) return DS_ERR_BAD_ARG;
    const int Cs = (x->C + 3) / 4 * 4, taps = KH * KW;
    const int Hs = x->H + 2 * x->halo, Ws = x->W + 2 * x->halo;
    const int Hv = x->H + 2 * ph, Wv = x->W + 2 * pw;
    const int OH = (Hv - KH) / sh + 1, OW = (Wv - KW) / sw + 1;
    const long long M = (long long)x->B * OH * OW;
    if (M > 2147483647LL - 1024 || (long long)Cs * taps > 2147483647LL) return DS_ERR_RANGE;
    const StGeom g = st_geometry(Cs, taps, OC);
    if (prepared_bytes < g.bytes) return DS_ERR_SCRATCH;
    if ((reinterpret_cast<uintptr_t>(prepared) | reinterpret_cast<uintptr_t>(x->data)) & 15u) return DS_ERR_ALIGN;

    StagedConvParams p = {};
    p.wt = static_cast<const float*>(prepared);
    p.negpre = reinterpret_cast<const int*>(p.wt + g.wt_floats);
    p.bias = bias;
    p.residual = out->residual;
    p.out_codes = out->codes;
    p.out_f32 = out->f32;
    p.out_nchw = out->nchw;
    p.out_nchw_f32 = out->nchw_is_f32;
    p.M = int(M); p.N = OC; p.P = OH * OW; p.OH = OH; p.OW = OW;
    p.sh = sh; p.sw = sw; p.KW = KW;
    p.cq_per_tap = Cs / 4;
    p.nkq = g.nkq;
    p.ntiles = g.ntiles;
    p.npad = g.npad;
    p.grid_n = g.grid_n;
    p.relu = out->relu;
    p.round_f32 = out->round_f32;
    p.inv_scale = 1.0f / float(1ll << F);
    p.inv_P = p.P == 1 ? 0xFFFFFFFFu : unsigned((1ull << 32) / unsigned(p.P));
    p.inv_OW = OW == 1 ? 0xFFFFFFFFu : unsigned((1ull << 32) / unsigned(OW));
    // Terms between drains: every staged value is code + 0.5 with |code| <= 2^(ab-1).
    const int ab = out->in_act_bits;
    if (ab < 1 || ab > 18) return DS_ERR_UNSUPPORTED;
    const long long per_term = (1ll << (ab - 1)) + 1;
    const long long terms = ((1ll << 22) - 1) / per_term;
    p.flush_tiles = int(terms / (4 * g.KQ) > 4096 ? 4096 : terms / (4 * g.KQ));
    if (p.flush_tiles < 1) return DS_ERR_UNSUPPORTED;
    p.rq_lo = p.rq_hi = p.rq_add = 0;
    p.rq_mul = 1;
    if (out->staged && out->staged->data) {
        const ds_staged_t* o = out->staged;
        if (o->B != x->B || o->H != OH || o->W != OW || o->C != OC || o->halo < 0) return DS_ERR_BAD_ARG;
        if (I < 1 || I + F > 18) return DS_ERR_BAD_ARG;
        if (reinterpret_cast<uintptr_t>(o->data) & 15u) return DS_ERR_ALIGN;
        p.out_staged = static_cast<float*>(o->data);
        p.os_H2 = OH + 2 * o->halo;
        p.os_W2 = OW + 2 * o->halo;
        p.os_Cs = (OC + 3) / 4 * 4;
        p.os_halo = o->halo;
        if (I == 1) {
            p.rq_lo = -1; p.rq_hi = 1; p.rq_mul = 1 << F; p.rq_add = -(1 << F);
        } else {
            p.rq_lo = -(1 << (I - 1 + F));
            p.rq_hi = ((1 << (I - 1)) - 1) * (1 << F);
        }
    }
    p.err_flag = kernel_error_flag();
    if (!p.err_flag) return DS_ERR_CUDA;

    EncodeIm2colFn enc = encode_im2col_fn();
    if (!enc) return DS_ERR_UNSUPPORTED;
    // The view the convolution reads: the image with exactly its own padding, inside the halo.
    char* view = static_cast<char*>(x->data) + (((size_t)(x->halo - ph) * Ws) + (x->halo - pw)) * Cs * 4;
    const cuuint64_t dims[4] = {cuuint64_t(Cs), cuuint64_t(Wv), cuuint64_t(Hv), cuuint64_t(x->B)};
    const cuuint64_t strides[3] = {cuuint64_t(Cs) * 4, cuuint64_t(Ws) * Cs * 4, cuuint64_t(Hs) * Ws * Cs * 4};
    const int lower[2] = {0, 0};
    const int upper[2] = {-(KW - 1), -(KH - 1)};
    const cuuint32_t estr[4] = {1, cuuint32_t(sw), cuuint32_t(sh), 1};
    CUtensorMap map;
    const CUresult er = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, view, dims, strides, lower, upper, 4, 256, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (er != CUDA_SUCCESS) return DS_ERR_UNSUPPORTED;
    {
        // Drivers up to CUDA 13.1 encode im2col maps of tensors below 128 KiB with a flag the
        // hardware mishandles; CUTLASS (cute/atom/copy_traits_sm90_im2col.hpp) clears it, and so
        // does this.
        static int driver_version = -1;
        if (driver_version < 0 && cudaDriverGetVersion(&driver_version) != cudaSuccess) driver_version = 0;
        const unsigned long long span =
            ((unsigned long long)(x->B - 1) * Hs * Ws + (unsigned long long)(Hv - 1) * Ws + Wv) * Cs * 4ull;
        if (driver_version <= 13010 && span < 131072ull) reinterpret_cast<unsigned long long*>(&map)[1] &= ~(1ull << 21);
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (g.BN == 128) return st_launch<128>(map, p, workspace, workspace_bytes, st);
    return st_launch<64>(map, p, workspace, workspace_bytes, st);
}
