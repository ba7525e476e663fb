/*
 * deepshift_b200 -- C ABI of the B200 (sm_100a) shift-inference kernels.
 *
 * Drop-in boundary for DeepShift's `use_kernel=True` inference path.  Each entry point
 * replaces one function of the reference's pybind module `deepshift_cuda`
 * (pytorch/deepshift/kernels/cuda/shift_cuda.cpp:64-68) and is called by the Python shim
 * deepshift_b200/kernels.py, which keeps the reference's `deepshift.kernels` signatures
 * (pytorch/deepshift/kernels/kernels.py:10,28,69).
 *
 * Conventions
 *   - Plain device pointers and sizes; the caller owns and allocates every buffer.  The
 *     library allocates nothing on these paths and keeps no state between calls.
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).  Work is
 *     enqueued on it and the call returns without synchronising.  The current CUDA device
 *     must be the one that owns the pointers.
 *   - Every function returns a ds_status (0 = success).  No device-side assert or trap.
 *   - int32 tensors are two's-complement; sums wrap modulo 2^32 exactly as the reference.
 *
 * Packed weights ("ConcWeight", pytorch/deepshift/utils.py:54-88, shift.cu:27-55)
 *   num = 32 / (bits + 1) weights per int32 word, row_len = ceil(K / num) words per output
 *   row; weight i of a word sits in bits [i*(bits+1), i*(bits+1)+bits) as `field` and bit
 *   i*(bits+1)+bits as `positive`.  Decoded right shift r = field + base, sign = positive ?
 *   +1 : -1.  r in [0,31]: term = sign*(x >> r) (arithmetic shift, negate AFTER the shift);
 *   r < 0: term = sign*(x << -r); r >= 32: term = 0 (the zero-weight encoding).
 */
#ifndef DEEPSHIFT_B200_H
#define DEEPSHIFT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    DS_OK = 0,
    DS_ERR_BAD_ARG = 1,      /* null pointer, non-positive size, inconsistent shape      */
    DS_ERR_UNSUPPORTED = 2,  /* bits outside 1..7, base > 0, kernel window > 31, ...     */
    DS_ERR_CUDA = 3,         /* the CUDA runtime reported an error at launch              */
    DS_ERR_RANGE = 4,        /* a size exceeds what 32-bit indexing of this build allows  */
    DS_ERR_ALIGN = 5,        /* a pointer is not 16-byte aligned                          */
    DS_ERR_SCRATCH = 6       /* ds_conv2d_noalloc: more output tiles than its fixed scratch holds */
} ds_status;

/* ds_fuse_t.act_bits: no promise about the range of int32 inputs, but let the library find out.  A
 * one-pass kernel looks for an |x| beyond 2^15; the FP32-pipe launch and the integer-path launch are
 * both enqueued, each gated on what it found (one of them returns at once).  About twice as fast as
 * act_bits = 0 for activations that a 16-bit quantiser produced, exact for all others.  Needs
 * fuse->workspace (its last counter word holds the result); without one, with base < 0 or for other
 * input kinds it means the same as 0. */
#define DS_ACT_BITS_AUTO (-1)

/* Input element kinds of the *_ex entry points. */
enum {
    DS_IN_I32 = 0,       /* int32 fixed point (what the reference kernels receive)                         */
    DS_IN_F32_CONV = 1,  /* fp32, quantised in the kernel as Conv2dShift does: clamp(floor(x*2^F)) -- utils.py:7-21, modules.py:153,317 */
    DS_IN_F32_LINEAR = 2,/* fp32, quantised as LinearShift does: trunc(x*2^F), no clamp -- modules.py:25 */
    DS_IN_I32_CLAMP = 3  /* int32 fixed point, clamped on read to [-2^(I-1+F), (2^(I-1)-1)*2^F]: what
                            Conv2dShift's round_to_fixed does to a value already on the 2^-F grid.
                            Lets one unclamped tensor feed both a convolution and a residual add.
                            With I == 1 round_to_fixed is sign(x) - 1 (utils.py:12-13), so a code
                            c < 0, c == 0, c > 0 is read as -2^(F+1), -2^F, 0: apply it to codes that
                            have NOT been through round_to_fixed yet (it is not idempotent there). */
};

/* Output element kinds of the *_ex entry points. */
enum {
    DS_OUT_I32 = 0, /* int32 accumulator + bias (what the reference kernels write)     */
    DS_OUT_F32 = 1  /* float(acc) / 2^F, the conversion of modules.py:30-31,161-162      */
};

/*
 * Optional fused prologue/epilogue of ds_linear_ex / ds_conv2d_ex.  Zero-initialise for the
 * plain int32-in / int32-out behaviour.  Order of the epilogue on v = acc + bias:
 *   residual add -> ReLU -> requantise clamp -> fp32 rounding -> store.
 */
typedef struct {
    int in_kind;            /* DS_IN_*                                                     */
    int out_kind;           /* DS_OUT_*                                                    */
    int act_integer_bits;   /* I of round_to_fixed; used by DS_IN_F32_CONV and `requant`   */
    int act_fraction_bits;  /* F; used by every fp32 conversion                            */
    int relu;               /* v = max(v, 0)                                               */
    int requant;            /* v = clamp(v, -2^(I-1+F), (2^(I-1)-1)*2^F): what the next
                               Conv2dShift's round_to_fixed would do to v/2^F (I == 1: the
                               sign rule described at DS_IN_I32_CLAMP)                     */
    const int32_t *residual;/* same shape/layout as the output, added before ReLU; may be NULL.  May be
                               the int32 output buffer itself (in-place add); any other overlap with
                               the output is not allowed                                   */
    int act_bits;           /* caller's guarantee on int32 inputs: every x satisfies
                               -2^(act_bits-1) <= x <= 2^(act_bits-1).  0 = no guarantee
                               (exact integer path).  1..20 enables the FP32-pipe path.
                               Implied by DS_IN_F32_CONV and DS_IN_I32_CLAMP (I+F, or F+2
                               when I == 1).                                               */
    int round_f32;          /* v = int(float(v)): the rounding the reference's `out.float()` applies
                               to sums beyond 2^24, so that an int32 tensor handed to the next layer
                               holds exactly the value the reference's fp32 tensor would        */
    int reserved[3];
    void *workspace;        /* optional scratch for sharing an output tile (256 rows x 128 or 64
                               columns) between CTAs along K.  The first 16384 int32 are arrival
                               counters: zero them once; every launch leaves them zero (the last of
                               them is the range flag of DS_ACT_BITS_AUTO, rewritten by each such call).  Bytes beyond
                               those 64 KiB (any contents) hold, per launch, the layer's weights
                               expanded to fp32 (4 bytes per weight, when the launch has at least 8
                               row tiles) and partial sums, 128 KiB per shared tile and split; about
                               90 MB serve every ResNet-18 layer on a 148-SM GPU, less is used as far
                               as it goes.
                               With counters and partial-sum space, the tiles left over after the last
                               full wave of CTAs are cut along K into 2-4 ranges so that the SMs
                               which would idle share them; the CTA that arrives last at a tile's
                               counter adds the partial sums in a fixed order and applies the
                               epilogue.  With counters only (<= 64 KiB), layers whose tiles fill the
                               SMs badly are split along K through integer atomics on the zeroed
                               output instead.  Results are bit-identical either way.  NULL = never
                               split.  Launches that share a workspace must not overlap on the GPU. */
    long long workspace_bytes;
    const void *prepared;   /* optional, convolutions only: this layer's weights expanded ahead of time
                               by ds_conv2d_prepare for exactly this geometry (B, C, H, W, OC, window,
                               stride, padding, bits, base).  With it the launch skips its own
                               weight expansion (two small kernels).  NULL = expand per launch (with
                               a workspace) or decode in the kernel (without).                     */
    long long prepared_bytes;
} ds_fuse_t;

/*
 * Shift "GEMM": out[m,n] = bias[n] + sum_k term(x[m,k], weight[n,k]).
 * Replaces DEEP_SHIFT_LINEAR (shift_cuda.cpp:26-39 -> shift.cu:174-387, kernel :57-120).
 *   x [M,K] int32 row-major, packed [N, ceil(K/num)] int32, bias [N] int32 or NULL,
 *   out [M,N] int32 row-major (need not be zero-initialised).
 * act_bits: see ds_fuse_t.act_bits.
 */
int ds_linear_i32(const int32_t *x, const int32_t *packed, const int32_t *bias, int32_t *out,
                  int M, int K, int N, int bits, int base, int act_bits, void *stream);

/*
 * Shift convolution on the UNPADDED NCHW input (zero padding is implicit).
 * Replaces F.pad + DEEP_SHIFT_CONV (kernels.py:32-53, shift_cuda.cpp:41-53 ->
 * shift.cu:399-669: IM2COL :122-153, GEMM :57-120, COL2IM :155-172) without the im2col and
 * col2im buffers.  K = C*KH*KW flattened in (ic,kh,kw) order; OH = (H+2ph-KH)/sh+1.
 *   x [B,C,H,W] int32, packed [OC, ceil(K/num)], bias [OC] or NULL, out [B,OC,OH,OW] int32.
 * No dilation, no groups (the reference ignores both, kernels.py:28).
 */
int ds_conv2d_i32(const int32_t *x, const int32_t *packed, const int32_t *bias, int32_t *out,
                  int B, int C, int H, int W, int OC, int KH, int KW, int sh, int sw, int ph,
                  int pw, int bits, int base, int act_bits, void *stream);

/* As above with a fused prologue/epilogue.  x is int32 or fp32 per fuse->in_kind, out is
 * int32 or fp32 per fuse->out_kind.  fuse->workspace serves ds_linear_ex (M > 64, FP32-pipe path,
 * K a multiple of 4, x 16-byte aligned, N > 32) exactly as it serves convolutions; fuse->prepared
 * is ignored by ds_linear_ex. */
int ds_linear_ex(const void *x, const int32_t *packed, const int32_t *bias, void *out, int M,
                 int K, int N, int bits, int base, const ds_fuse_t *fuse, void *stream);
int ds_conv2d_ex(const void *x, const int32_t *packed, const int32_t *bias, void *out, int B,
                 int C, int H, int W, int OC, int KH, int KW, int sh, int sw, int ph, int pw,
                 int bits, int base, const ds_fuse_t *fuse, void *stream);

/*
 * ds_conv2d_ex for callers that must not allocate device memory (no counterpart in the reference).
 *
 * Who needs it: a host that has already handed all of the GPU's memory to its own pool or to other
 * tenants, so that a cudaMalloc for the split-K counters could fail; or a latency-critical loop in
 * which an allocation (and the device-wide synchronisation it can imply) is not acceptable and no
 * pre-allocated workspace was threaded through to this call.
 *
 * Same arguments, result and bit-exactness as ds_conv2d_ex, except that fuse->workspace is ignored:
 * the split-K arrival counters live in a fixed array inside the library (64 KiB on every GPU that
 * loads the library, until the process exits).  The call itself and everything under it make no
 * cudaMalloc / cudaFree and call no allocating library routine.
 *   - Limit: at most 16384 output tiles per call, a tile being 256 output positions (b,oh,ow) by
 *     128 output channels (64 when OC <= 64).  Larger problems return DS_ERR_SCRATCH and run nothing;
 *     use ds_conv2d_ex with a workspace, or without one, for those.  The limit is applied by tile
 *     count alone, also to calls whose launch would not have used a counter (integer path, few
 *     output channels).
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current).  Make that first call before starting any stream capture.
 *   - All calls on a device share the array.  Every call clears the counters it will use on
 *     `stream` before its kernel, but two calls whose kernels overlap on the GPU (different streams,
 *     no ordering between them) race on it: order such calls yourself.
 */
int ds_conv2d_noalloc(const void *x, const int32_t *packed, const int32_t *bias, void *out, int B,
                      int C, int H, int W, int OC, int KH, int KW, int sh, int sw, int ph, int pw,
                      int bits, int base, const ds_fuse_t *fuse, void *stream);

/*
 * Packs (shift', sign) into words.  Replaces COMPRESS_SIGN_SHIFT (shift_cuda.cpp:55-61 ->
 * shift.cu:388-397, one launch per output channel there; one launch in total here).
 *   shiftp, sign [OC,K] int32; packed [OC, ceil(K/num)] int32; field = shiftp - base.
 */
int ds_compress(const int32_t *shiftp, const int32_t *sign, int32_t *packed, int OC, int K,
                int bits, int base, void *stream);

/*
 * round_to_fixed(x, I, F) * 2^F as int32 (utils.py:7-21 + modules.py:153), one pass.
 * kind = DS_IN_F32_CONV (floor + clamp) or DS_IN_F32_LINEAR (trunc, no clamp, modules.py:25).
 */
int ds_quantize_f32(const float *x, int32_t *out, long long n, int kind, int act_integer_bits,
                    int act_fraction_bits, void *stream);

/*
 * Inter-layer glue of the integer pipeline (no counterpart in the reference's native code, which
 * leaves these steps to torch ops on fp32: F.max_pool2d / adaptive_avg_pool2d in the model
 * definitions, e.g. torchvision ResNet).  Both are exact restatements on the int32 codes.
 *   ds_maxpool2d_i32   : square window k, stride, symmetric pad; out [B,C,OH,OW].
 *   ds_avgpool_fix_i32 : global average over H*W, then the LinearShift entry conversion
 *                        trunc(mean * 2^F) (modules.py:25); out [B,C] int32.  mean is
 *                        float(exact integer sum) / 2^F / (H*W) in fp32.
 */
int ds_maxpool2d_i32(const int32_t *x, int32_t *out, int B, int C, int H, int W, int k, int stride,
                     int pad, void *stream);
int ds_avgpool_fix_i32(const int32_t *x, int32_t *out, int B, int C, int H, int W, int F, void *stream);

/*
 * Glue of the fp32 module path: y[i] = y[i] + r[i], then max(., 0) when relu != 0, in place and in
 * one pass -- what a residual block's `out += identity; out = relu(out)` (two torch kernels, five
 * passes over the tensor) computes, bit for bit (IEEE fp32 addition; a NaN stays a NaN).
 * r may be NULL (ReLU only).  y and r must not overlap unless they are the same buffer.
 */
int ds_add_relu_f32(float *y, const float *r, long long n, int relu, void *stream);

/*
 * Glue of the fp32 module path: F.max_pool2d on fp32 NCHW (square window, symmetric padding, no
 * dilation, floor mode; a NaN in the window is the result, as in torch).  Same kernels as
 * ds_maxpool2d_i32; the 3x3 / stride 2 / padding 1 pool of a ResNet stem takes a quarter of the time of
 * torch's kernel.
 */
int ds_maxpool2d_f32(const float *x, float *out, int B, int C, int H, int W, int k, int stride, int pad,
                     void *stream);

/*
 * Register-only issue-rate probe used for the roofline denominator.
 *   mode 0: shift + add (both on the integer ALU pipe)
 *   mode 1: shift + integer multiply-add (ALU pipe + FMA pipe)
 *   mode 2: FP32 fused multiply-add with round-down (FMA pipe)
 * Runs on `stream`, synchronises, and writes the sustained rate in shift-accumulate
 * operations per second (one op = one shift plus one signed accumulate) to *ops_per_s.
 */
int ds_pipe_peak(int mode, int iters, double *ops_per_s, void *stream);

/*
 * Expands the packed weights of one convolution layer once, for callers whose weights do not
 * change between calls (inference): the result goes into fuse->prepared (device memory of the
 * caller, fuse->prepared_bytes long) and is handed to later ds_conv2d_ex calls of the SAME
 * geometry through the same two fields.  *bytes_needed receives the size this geometry wants:
 * 0 when its launches would not use expanded weights (few rows, integer path, few channels), in
 * which case nothing is written and `prepared` may stay NULL.  Call with fuse->prepared = NULL
 * to ask for the size only.  DS_ERR_SCRATCH if the buffer is too small.  The other fields of
 * `fuse` must be the ones the later calls will use (they select the arithmetic path).  No
 * counterpart in the reference, which decodes the packed words inside every kernel launch.
 */
int ds_conv2d_prepare(const int32_t *packed, int B, int C, int H, int W, int OC, int KH, int KW,
                      int sh, int sw, int ph, int pw, int bits, int base, const ds_fuse_t *fuse,
                      long long *bytes_needed, void *stream);

/*
 * ---- Staged activations: the TMA-fed convolution path (no counterpart in the reference) ----------
 *
 * For a chain of shift layers (a whole network) the activations can stay in the form the FP32-pipe
 * arithmetic reads and the tensor memory accelerator fetches: fp32 NHWC, value = code + 0.5, where
 * code is the int32 fixed-point activation AFTER the quantiser clamp of the layer that will read it
 * (round_to_fixed, utils.py:7-21, applied to a value already on the 2^-F grid), with `halo` pixels
 * of 0.5 (the code 0) around every image and C rounded up to a multiple of 4 channels per pixel
 * (the extra channels hold 0.5 too).  ds_staged_conv2d replaces F.pad + DEEP_SHIFT_CONV
 * (kernels.py:32-53, shift.cu:399-669) on such a tensor: its input tiles come into shared memory
 * through `cp.async.bulk.tensor` in im2col mode, so the im2col matrix exists neither in HBM nor in
 * registers, and zero padding is the halo.  Results are bit-identical to ds_conv2d_ex.
 *
 * The caller owns every buffer.  A staged tensor must be filled with 0.5 once (ds_staged_fill)
 * before its first use; the kernels only ever write its interior.
 */
typedef struct {
    void *data;      /* fp32 [B][H + 2*halo][W + 2*halo][Cs], Cs = C rounded up to a multiple of 4; 16-byte aligned */
    int B, H, W, C;  /* logical extent */
    int halo;        /* >= the padding of every convolution that reads the tensor */
} ds_staged_t;

/* What ds_staged_conv2d writes; any subset of the four outputs.  v = acc + bias, then residual add
 * (fp32 add of the two codes, as `out += identity` does), ReLU, fp32 rounding (round_f32). */
typedef struct {
    int32_t *codes;            /* [B][OH][OW][OC] int32 (NHWC): v                                   */
    float *f32;                /* [B][OH][OW][OC] fp32: v / 2^F (modules.py:161-162)               */
    void *nchw;                /* [B][OC][OH][OW]: v as int32, or v / 2^F as fp32 when nchw_is_f32 */
    int nchw_is_f32;
    const ds_staged_t *staged; /* operand of the next layer: clamp(v) + 0.5 with the clamp of I, F below
                                  (geometry must be B, OH, OW, OC; any halo); may be NULL          */
    const int32_t *residual;   /* [B][OH][OW][OC] int32 (NHWC) or NULL                             */
    int relu, round_f32;
    int act_integer_bits;      /* I and F of the quantiser of the layer that reads `staged`        */
    int act_fraction_bits;     /* F: also the scale of f32 / nchw fp32 outputs                     */
    int in_act_bits;           /* bound on the input: every staged value is code + 0.5 with
                                  |code| <= 2^(in_act_bits-1); 1..18 (16 for 4.12 activations)     */
    int reserved[3];
} ds_staged_out_t;

/* Bytes of a staged tensor of this geometry; -1 for bad arguments. */
long long ds_staged_bytes(int B, int H, int W, int C, int halo);

/* Writes 0.5 into every element (halo, padding channels and interior). */
int ds_staged_fill(const ds_staged_t *t, void *stream);

/* Quantises an NCHW tensor into the interior of a staged one.  in_kind: DS_IN_F32_CONV (fp32,
 * round_to_fixed(x, I, F), utils.py:7-21 + modules.py:153), DS_IN_I32_CLAMP (int32 codes, the same
 * quantiser applied to code / 2^F) or DS_IN_I32 (int32 codes taken as they are; |code| <= 2^17). */
int ds_stage_nchw(const void *x, int in_kind, int act_integer_bits, int act_fraction_bits,
                  const ds_staged_t *dst, void *stream);

/* Expands the packed weights of one layer for ds_staged_conv2d (once per layer; depends on the
 * weights, C, OC and the window only).  Call with prepared = NULL to get the size.  base must be 0. */
int ds_staged_prepare(const int32_t *packed, int C, int OC, int KH, int KW, int bits, int base,
                      void *prepared, long long prepared_bytes, long long *bytes_needed, void *stream);

/* The convolution.  x->halo >= ph, pw.  `workspace` as ds_fuse_t.workspace (optional: lets the tiles
 * after the last full wave of CTAs be shared along K); launches sharing one must not overlap. */
int ds_staged_conv2d(const ds_staged_t *x, const void *prepared, long long prepared_bytes,
                     const int32_t *bias, int OC, int KH, int KW, int sh, int sw, int ph, int pw,
                     const ds_staged_out_t *out, void *workspace, long long workspace_bytes, void *stream);

/* Max pooling of int32 NHWC codes [B][H][W][C] (square window k, stride, symmetric pad, as
 * F.max_pool2d); writes int32 NHWC codes (may be NULL) and/or the staged operand of the next layer
 * (clamp of I, F; may be NULL). */
int ds_maxpool_nhwc(const int32_t *x, int B, int H, int W, int C, int k, int stride, int pad,
                    int32_t *out_codes, const ds_staged_t *out_staged, int act_integer_bits,
                    int act_fraction_bits, void *stream);

/* Global average of int32 NHWC codes followed by the LinearShift entry conversion, as
 * ds_avgpool_fix_i32; out [B][C] int32. */
int ds_avgpool_fix_nhwc(const int32_t *x, int32_t *out, int B, int H, int W, int C, int F, void *stream);

/*
 * The reference's "unoptimized" fp32 baseline (pytorch/unoptimized/kernels/cuda/unoptimized.cu:63-103
 * GEMM, :10-61 IM2COL / COL2IM; entry points unoptimized_cuda.cpp:24-56): ordinary multiply-accumulate
 * layers at the same (deliberately low) level of tuning as its shift kernels, for the latency
 * comparison of its README.  weight is [N][K] / [OC][C][KH][KW] fp32, bias may be NULL, out is
 * [M][N] / NCHW fp32; the convolution reads the unpadded input.
 */
int ds_unopt_linear_f32(const float *x, const float *weight, const float *bias, float *out, int M, int K,
                        int N, void *stream);
int ds_unopt_conv2d_f32(const float *x, const float *weight, const float *bias, float *out, int B, int C,
                        int H, int W, int OC, int KH, int KW, int sh, int sw, int ph, int pw, void *stream);

/*
 * Reads and clears the device-side flag that a kernel of this library sets when one of its
 * bounded waits ran out (its output is then undefined; it never happens in a correct run).
 * Synchronises the current device.  *flag = 0 means no error.
 */
int ds_last_kernel_error(int *flag);

/*
 * Checked build.  The library compiled with -DDS_BOUNDS_CHECK (deepshift_b200/_build.py, flavour
 * "checked": libdeepshift_b200_checked.so) tests the address of every global load of activations,
 * packed weights and residual and of every global store in the linear / convolution kernels against
 * the extents implied by the call's arguments.  An access outside is skipped, never performed, and
 * the first one leaves its kind in a status word: 1 activations, 2 packed weights, 3 output /
 * residual.  Nothing traps.  (The TMA-fed staged kernel is not instrumented: the
 * tensor map bounds its loads in hardware.)
 *   ds_bounds_status        reads and clears the status word (synchronises the device); *checked
 *                           says whether this library was built with the checks.
 *   ds_bounds_debug_shrink_x  checked build only: declares x `bytes` shorter than it is, so that the
 *                           checks can be seen to fire without anything leaving a real buffer.
 */
int ds_bounds_status(int *status, int *checked);
int ds_bounds_debug_shrink_x(long long bytes);

/*
 * Timing build.  The library compiled with -DDS_WS_TIMING (flavour "timing":
 * libdeepshift_b200_timing.so) has the warp-specialised convolution / linear kernel print, for every
 * warp of its CTA 1, the cycles spent waiting at the producer / consumer hand-shake, staging and in
 * the epilogue ("ws_timing ..." lines on stdout, one set per launch).  Same entry points, same results;
 * a diagnostic, slower by the printing.
 */

/*
 * Number of kernels this library has launched in this process so far (a host-side counter;
 * diagnostics, no counterpart in the reference).  The difference across one forward pass is the
 * pass's kernel count, whatever path the launch heuristics took.
 */
long long ds_launch_count(void);

const char *ds_strerror(int status);
int ds_version(void);

#ifdef __cplusplus
}
#endif
#endif /* DEEPSHIFT_B200_H */
