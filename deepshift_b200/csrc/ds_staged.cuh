// Declarations of the staged-activation path: convolutions whose input tiles are brought into
// shared memory by the tensor memory accelerator (TMA, im2col mode) instead of by producer warps.
//
// "Staged" activations are what the FP32-pipe arithmetic wants to read, laid out as TMA wants to
// fetch them: fp32 NHWC with a physical halo, value = code + 0.5 where code is the int32
// fixed-point activation after the quantiser clamp of the layer that will read it.  The halo and
// the channels beyond C (C is rounded up to a multiple of 4 so that a pixel's channel group is
// 16 bytes) hold 0.5, the image of the code 0: a zero-padded tap then needs no predicate and no
// fill value, TMA's im2col traversal reads it like any other pixel.
#pragma once
#include "ds_gemm_common.cuh"

namespace ds {

// Geometry of one staged tensor: [B][H + 2*halo][W + 2*halo][Cs] floats.
struct StagedDesc {
    float* data;
    int B, H, W, C;  // logical extent
    int Cs;          // channels stored per pixel, a multiple of 4, >= C
    int halo;        // pixels of 0.5 around every image
};

struct StagedConvParams {
    const float* wt;      // prepared weights, [grid_n][ntiles][4*KQ][BN] floats (see the expand kernel)
    const int* negpre;    // [ntiles + 1][npad]: negative weights of a column in the k-tiles before t
    const int32_t* bias;  // [N] or null
    const int32_t* residual;  // [M][N] int32 codes (NHWC) or null
    // outputs, any subset:
    int32_t* out_codes;   // [M][N] int32 (NHWC): the finished value v
    float* out_f32;       // [M][N] fp32: v / 2^F
    void* out_nchw;       // [B][N][OH][OW] int32 (v) or fp32 (v / 2^F) per out_nchw_f32
    float* out_staged;    // staged operand of the next layer: clamp(v) + 0.5 into the interior
    int out_nchw_f32;
    int os_H2, os_W2, os_Cs, os_halo;  // out_staged: rows and columns with halo, channels per pixel, halo
    int M, N, P, OH, OW;  // M = B * OH * OW output positions, P = OH * OW
    unsigned inv_P, inv_OW;  // floor(2^32 / d): __umulhi(x, inv) is x / d or one less
    int sh, sw, KW;
    int cq_per_tap;       // channel groups of four per filter tap = Cs / 4
    int nkq;              // groups of four k in total = KH * KW * cq_per_tap
    int ntiles;           // k-tiles = ceil(nkq / KQ)
    int npad;             // grid_n * BN
    int flush_tiles;      // k-tiles between drains of the float accumulators
    int relu, round_f32;
    int rq_lo, rq_hi, rq_mul, rq_add;  // quantiser of the layer that reads out_staged (see GemmParams)
    float inv_scale;
    // work units: see WsItem in ds_gemm_ws.cuh; same scheme
    int grid_m, grid_n;
    int full_units, tail_first, tail_items, tail_splits, tail_tps;
    int* counters;
    int* partials;
    int* err_flag;
};

int* kernel_error_flag();  // device address of the flag bounded waits set (ds_gemm_ws.cu), null on failure

}  // namespace ds
