/*
 * CPU oracle for the DeepShift use_kernel inference path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the reference
 * algorithm, used by tests/, by __graft_entry__.smoke() and by the cpu_baseline /
 * reference legs of bench.py as the checker.  The product (deepshift_b200/) never
 * imports, links or executes it.
 *
 * Parity pin: every function here is checked bit-for-bit against the reference's own
 * compiled CPU kernel (pytorch/deepshift/kernels/cpu/shift_cpu.cpp, built unmodified by
 * oracle/build_ref.py into oracle/_ref/) and against the golden vectors under
 * tests/golden/, which were produced by running that compiled reference.
 *
 * All arithmetic is two's-complement int32.  Left shifts are done on uint32_t so that
 * the wrap-around is defined; `>>` on a negative int32_t is the arithmetic (floor)
 * shift on every compiler this project builds with.
 *
 * Domain: shift amounts in [-31, 31].  The reference's `x >> 32` is undefined behaviour
 * in C++ (and differs between its CPU and CUDA builds), so a weight that must contribute
 * nothing is expressed as sign == 0 in the unpacked form and as "decoded right shift
 * >= 32" in the packed form.
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define DSO_EXPORT __attribute__((visibility("default")))

static inline int32_t shl32(int32_t x, int s) { return (int32_t)((uint32_t)x << s); }

/* One (activation, weight) term exactly as the four-way if/else chain of
 * shift_cpu.cpp:190-201 (linear) computes it: sign<0 subtracts, sign>0 adds, s>=0 shifts
 * left, s<0 shifts right by -s, sign==0 adds nothing. */
static inline int32_t term_linear(int32_t x, int s, int32_t sign)
{
    if (sign < 0 && s >= 0) return -shl32(x, s);
    if (sign > 0 && s >= 0) return shl32(x, s);
    if (sign < 0 && s < 0) return -(x >> (-s));
    if (sign > 0 && s < 0) return x >> (-s);
    return 0;
}

/* shift_cpu.cpp:109-229 (live loop 176-221): out[m][n] = bias[n] + sum_k term. */
DSO_EXPORT void dso_linear(const int32_t *x, const int32_t *shift, const int32_t *sign,
                           const int32_t *bias, int32_t *out, int M, int K, int N)
{
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        for (int n = 0; n < N; ++n) {
            uint32_t y = 0;
            const int32_t *xs = x + (size_t)m * K;
            const int32_t *sh = shift + (size_t)n * K;
            const int32_t *sg = sign + (size_t)n * K;
            for (int k = 0; k < K; ++k)
                y += (uint32_t)term_linear(xs[k], sh[k], sg[k]);
            y += (uint32_t)(bias ? bias[n] : 0);
            out[(size_t)m * N + n] = (int32_t)y;
        }
    }
}

/*
 * shift_cpu.cpp:295-374: direct convolution over an ALREADY zero-padded NCHW input
 * (the reference's Python wrapper pads before the call, kernels.py:32-36).
 *   OH = (Hp - KH) / sh + 1, OW = (Wp - KW) / sw + 1               (shift_cpu.cpp:318-320)
 *   out[b][oc][oh][ow] = bias[oc] + sum_{kh,kw,ic} term             (shift_cpu.cpp:327-366)
 *
 * zero_sign_as_plus != 0 reproduces the reference conv kernel's trailing `else`
 * (shift_cpu.cpp:351-353): any weight that is not matched by the first three branches,
 * sign == 0 included, is added as `x >> (-s)`; that branch is only defined for s <= 0.
 * zero_sign_as_plus == 0 is the canonical rule shared with the linear kernel (sign 0
 * contributes nothing).
 */
DSO_EXPORT void dso_conv2d_prepadded(const int32_t *x, const int32_t *shift,
                                     const int32_t *sign, const int32_t *bias, int32_t *out,
                                     int B, int C, int Hp, int Wp, int OC, int KH, int KW,
                                     int sh, int sw, int zero_sign_as_plus)
{
    const int OH = (Hp - KH) / sh + 1;
    const int OW = (Wp - KW) / sw + 1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b) {
        for (int oc = 0; oc < OC; ++oc) {
            for (int oh = 0; oh < OH; ++oh) {
                for (int ow = 0; ow < OW; ++ow) {
                    uint32_t y = 0;
                    for (int kh = 0; kh < KH; ++kh)
                        for (int kw = 0; kw < KW; ++kw)
                            for (int ic = 0; ic < C; ++ic) {
                                size_t wi = (((size_t)oc * C + ic) * KH + kh) * KW + kw;
                                int s = shift[wi];
                                int32_t g = sign[wi];
                                int32_t xv = x[(((size_t)b * C + ic) * Hp + (oh * sh + kh)) * Wp +
                                               (ow * sw + kw)];
                                if (g == 0 && zero_sign_as_plus)
                                    y += (uint32_t)(xv >> (-s));
                                else
                                    y += (uint32_t)term_linear(xv, s, g);
                            }
                    y += (uint32_t)(bias ? bias[oc] : 0);
                    out[(((size_t)b * OC + oc) * OH + oh) * OW + ow] = (int32_t)y;
                }
            }
        }
    }
}

/*
 * Zero padding (kernels.py:32-36 with the H/W order of torch.nn.functional.conv2d:
 * ph rows above and below, pw columns left and right).
 */
DSO_EXPORT void dso_pad_nchw(const int32_t *x, int32_t *xp, int B, int C, int H, int W,
                             int ph, int pw)
{
    const int Hp = H + 2 * ph, Wp = W + 2 * pw;
    memset(xp, 0, (size_t)B * C * Hp * Wp * sizeof(int32_t));
    for (size_t bc = 0; bc < (size_t)B * C; ++bc)
        for (int h = 0; h < H; ++h)
            memcpy(xp + (bc * Hp + h + ph) * Wp + pw, x + (bc * H + h) * W,
                   (size_t)W * sizeof(int32_t));
}

/*
 * Packing of (shift', sign) into int32 words, the COMPRESS helper and its per-row kernel
 * (shift.cu:27-55): word w of row oc holds `num` weights, weight i in bits
 * [i*(bits+1), i*(bits+1)+bits) = shift'[k] - base, and bit i*(bits+1)+bits = (sign > 0).
 * K is the row length IC*KH*KW; row_len = ceil(K / num) (utils.py:82-84).
 */
DSO_EXPORT void dso_compress(const int32_t *shiftp, const int32_t *sign, int32_t *packed,
                             int OC, int K, int bits, int base)
{
    const int num = 32 / (bits + 1);
    const int row_len = (K + num - 1) / num;
    for (int oc = 0; oc < OC; ++oc)
        for (int w = 0; w < row_len; ++w) {
            uint32_t value = 0;
            int s = 0;
            int len = K - w * num < num ? K - w * num : num;
            for (int i = 0; i < len; ++i) {
                size_t k = (size_t)oc * K + (size_t)w * num + i;
                value |= (uint32_t)(shiftp[k] - base) << s;
                s += bits;
                value |= (uint32_t)(sign[k] > 0 ? 1 : 0) << s;
                s += 1;
            }
            packed[(size_t)oc * row_len + w] = (int32_t)value;
        }
}

/*
 * Shift "GEMM" on packed weights, following the decode of the reference CUDA kernel
 * (shift.cu:92-111): field = word & mask, sign bit clear -> -1, set -> +1, then
 * `word >>= bits + 1`.  The decoded net right shift is r = field + base.
 *   r in [0, 31]  : term = sgn * (x >> r)
 *   r < 0         : term = sgn * (x << -r)      (CPU semantics of a positive shift)
 *   r >= 32       : term = 0                     (the zero-weight encoding of utils.py:67-70)
 */
DSO_EXPORT void dso_linear_packed(const int32_t *x, const int32_t *packed, const int32_t *bias,
                                  int32_t *out, int M, int K, int N, int bits, int base)
{
    const int num = 32 / (bits + 1);
    const int row_len = (K + num - 1) / num;
    const uint32_t mask = (1u << bits) - 1u;
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        for (int n = 0; n < N; ++n) {
            uint32_t y = 0;
            for (int k = 0; k < K; ++k) {
                uint32_t word = (uint32_t)packed[(size_t)n * row_len + k / num];
                uint32_t f = word >> ((k % num) * (bits + 1));
                int r = (int)(f & mask) + base;
                int32_t sgn = ((f >> bits) & 1u) ? 1 : -1;
                int32_t xv = x[(size_t)m * K + k];
                int32_t t;
                if (r >= 32) t = 0;
                else if (r >= 0) t = xv >> r;
                else t = shl32(xv, -r);
                y += (uint32_t)(sgn * t);
            }
            y += (uint32_t)(bias ? bias[n] : 0);
            out[(size_t)m * N + n] = (int32_t)y;
        }
    }
}

/* Gather of the reference IM2COL kernel (shift.cu:122-153) on a pre-padded input:
 * col[(b,oh,ow)][(ic,kh,kw)] = xp[b][ic][oh*sh+kh][ow*sw+kw]. */
DSO_EXPORT void dso_im2col(const int32_t *xp, int32_t *col, int B, int C, int Hp, int Wp,
                           int KH, int KW, int sh, int sw)
{
    const int OH = (Hp - KH) / sh + 1;
    const int OW = (Wp - KW) / sw + 1;
    const int K = C * KH * KW;
#pragma omp parallel for schedule(static)
    for (int b = 0; b < B; ++b)
        for (int oh = 0; oh < OH; ++oh)
            for (int ow = 0; ow < OW; ++ow) {
                int32_t *row = col + (((size_t)b * OH + oh) * OW + ow) * K;
                for (int ic = 0; ic < C; ++ic)
                    for (int kh = 0; kh < KH; ++kh)
                        for (int kw = 0; kw < KW; ++kw)
                            row[(ic * KH + kh) * KW + kw] =
                                xp[(((size_t)b * C + ic) * Hp + oh * sh + kh) * Wp + ow * sw + kw];
            }
}

/* Transpose of the reference COL2IM kernel (shift.cu:155-172):
 * [B*OH*OW, OC] -> NCHW [B, OC, OH, OW]. */
DSO_EXPORT void dso_col2im(const int32_t *col, int32_t *im, int B, int OC, int OH, int OW)
{
    for (int b = 0; b < B; ++b)
        for (int p = 0; p < OH * OW; ++p)
            for (int oc = 0; oc < OC; ++oc)
                im[((size_t)b * OC + oc) * OH * OW + p] = col[((size_t)b * OH * OW + p) * OC + oc];
}

DSO_EXPORT int dso_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
