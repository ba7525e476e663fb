// The "unoptimized" fp32 baseline of the reference (pytorch/unoptimized/kernels/cuda/unoptimized.cu):
// ordinary multiply-accumulate layers written as simply as its shift kernels, which its README uses
// to show what replacing multiplies by shifts buys at equal (lack of) tuning.  One kernel serves the
// linear layer and the convolution: a 16 x 16 tile of outputs per block, operands staged through
// shared memory 16 values of k at a time, the im2col gather done on the fly (the reference
// materialises the matrix, unoptimized.cu:10-41, and scatters the result back, :43-61).
// fp32 throughout; sums run over k in increasing order within a thread, so results agree with
// torch's to rounding, not bit for bit.
#include "ds_common.cuh"

namespace ds {
namespace {

constexpr int UT = 16;

struct UnoptParams {
    const float* x;
    const float* w;     // [N][K]
    const float* bias;  // [N] or null
    float* out;
    int M, K, N;
    int conv;           // 0: x is [M][K]; 1: x is NCHW and row m = (b, oh, ow), column k = (c, kh, kw)
    int C, H, W, KH, KW, sh, sw, ph, pw, OH, OW;
};

__global__ void __launch_bounds__(UT * UT) unopt_kernel(const UnoptParams p)
{
    __shared__ float As[UT][UT + 1], Bs[UT][UT + 1];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int m = blockIdx.y * UT + ty, n = blockIdx.x * UT + tx;
    // the row this thread stages (same m as it computes) and, for convolutions, where its window starts
    int b = 0, ih0 = 0, iw0 = 0;
    if (p.conv && m < p.M) {
        const int P = p.OH * p.OW;
        b = m / P;
        const int pp = m - b * P;
        ih0 = (pp / p.OW) * p.sh - p.ph;
        iw0 = (pp % p.OW) * p.sw - p.pw;
    }
    float acc = 0.f;
    for (int k0 = 0; k0 < p.K; k0 += UT) {
        const int ka = k0 + tx;  // k of the x value this thread stages
        float a = 0.f;
        if (m < p.M && ka < p.K) {
            if (p.conv) {
                const int c = ka / (p.KH * p.KW), r = ka - c * (p.KH * p.KW);
                const int ih = ih0 + r / p.KW, iw = iw0 + r % p.KW;
                if (unsigned(ih) < unsigned(p.H) && unsigned(iw) < unsigned(p.W))
                    a = p.x[(((size_t)b * p.C + c) * p.H + ih) * p.W + iw];
            } else {
                a = p.x[(size_t)m * p.K + ka];
            }
        }
        As[ty][tx] = a;
        const int nb = blockIdx.x * UT + ty;  // weight row this thread stages
        Bs[ty][tx] = (nb < p.N && ka < p.K) ? p.w[(size_t)nb * p.K + ka] : 0.f;
        __syncthreads();
#pragma unroll
        for (int j = 0; j < UT; ++j) acc += As[ty][j] * Bs[tx][j];
        __syncthreads();
    }
    if (m >= p.M || n >= p.N) return;
    if (p.bias) acc += p.bias[n];
    if (p.conv) {
        const int P = p.OH * p.OW;
        p.out[((size_t)b * p.N + n) * P + (m - b * P)] = acc;
    } else {
        p.out[(size_t)m * p.N + n] = acc;
    }
}

int launch_unopt(const UnoptParams& p, void* stream)
{
    const long long gx = (p.N + UT - 1) / UT, gy = ((long long)p.M + UT - 1) / UT;
    if (gy > 65535LL * 1024) return DS_ERR_RANGE;
    if (gy > 65535) return DS_ERR_RANGE;
    unopt_kernel<<<dim3(unsigned(gx), unsigned(gy)), dim3(UT, UT), 0, static_cast<cudaStream_t>(stream)>>>(p);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
}

}  // namespace
}  // namespace ds

using namespace ds;

extern "C" int ds_unopt_linear_f32(const float* x, const float* weight, const float* bias, float* out, int M, int K,
                                   int N, void* stream)
{
    if (!x || !weight || !out || M < 0 || K <= 0 || N <= 0) return DS_ERR_BAD_ARG;
    if (M == 0) return DS_OK;
    UnoptParams p = {};
    p.x = x; p.w = weight; p.bias = bias; p.out = out;
    p.M = M; p.K = K; p.N = N;
    return launch_unopt(p, stream);
}

extern "C" int ds_unopt_conv2d_f32(const float* x, const float* weight, const float* bias, float* out, int B, int C,
                                   int H, int W, int OC, int KH, int KW, int sh, int sw, int ph, int pw, void* stream)
{
    if (!x || !weight || !out || B < 0 || C <= 0 || H <= 0 || W <= 0 || OC <= 0 || KH <= 0 || KW <= 0 || sh <= 0 ||
        sw <= 0 || ph < 0 || pw < 0 || H + 2 * ph < KH || W + 2 * pw < KW)
        return DS_ERR_BAD_ARG;
    if (B == 0) return DS_OK;
    UnoptParams p = {};
    p.x = x; p.w = weight; p.bias = bias; p.out = out;
    p.conv = 1;
    p.C = C; p.H = H; p.W = W; p.KH = KH; p.KW = KW; p.sh = sh; p.sw = sw; p.ph = ph; p.pw = pw;
    p.OH = (H + 2 * ph - KH) / sh + 1;
    p.OW = (W + 2 * pw - KW) / sw + 1;
    const long long M = (long long)B * p.OH * p.OW, K = (long long)C * KH * KW;
    if (M > 2147483647LL || K > 2147483647LL) return DS_ERR_RANGE;
    p.M = int(M); p.K = int(K); p.N = OC;
    return launch_unopt(p, stream);
}
