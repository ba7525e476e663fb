// One-pass kernels around the staged convolution: filling a staged tensor, quantising an NCHW
// tensor into one, max pooling and global average pooling of int32 NHWC codes.  All are bound by
// HBM bandwidth (8-12 bytes per element moved once).
#include <climits>

#include "ds_staged.cuh"

namespace ds {
namespace {

__global__ void __launch_bounds__(256) staged_fill_kernel(float4* __restrict__ dst, long long n4)
{
    const float4 h = make_float4(0.5f, 0.5f, 0.5f, 0.5f);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x)
        dst[i] = h;
}

// The quantiser of round_to_fixed on an int32 code (see GemmParams::rq_*), then + 0.5.
struct CodeQuant {
    int lo, hi, mul, add;
};

__device__ __forceinline__ float staged_of_code(int v, const CodeQuant& q)
{
    return __int2float_rn(min(max(v, q.lo), q.hi) * q.mul + q.add) + 0.5f;
}

// NCHW (fp32 or int32) -> staged.  A block transposes 32 channels x 64 pixels through shared
// memory: reads run along the pixels of one channel plane, writes along the channels of one pixel.
template <int KIND>  // DS_IN_F32_CONV, DS_IN_I32_CLAMP or DS_IN_I32
__global__ void __launch_bounds__(256) stage_nchw_kernel(const void* __restrict__ x, float* __restrict__ dst, int B, int C,
                                                         int H, int W, int Cs, int halo, Quant qf, CodeQuant qc)
{
    __shared__ float tile[32][65];
    const long long npix = (long long)B * H * W;
    const long long p0 = (long long)blockIdx.x * 64;
    const int c0 = blockIdx.y * 32;
    const int HW = H * W;
    // load: thread (px = t % 64, cg = t / 64) reads channels c0 + cg, cg + 4, ...
    {
        const int px = threadIdx.x & 63, cg = threadIdx.x >> 6;
        const long long p = p0 + px;
        if (p < npix) {
            const long long b = p / HW;
            const int hw = int(p - b * HW);
            for (int cl = cg; cl < 32; cl += 4) {
                const int c = c0 + cl;
                float v = 0.5f;  // padding channel: the code 0
                if (c < C) {
                    const long long src = (b * C + c) * HW + hw;
                    if (KIND == DS_IN_F32_CONV) {
                        v = quant_conv_f(__ldg(static_cast<const float*>(x) + src), qf) + 0.5f;
                    } else {
                        const int raw = __ldg(static_cast<const int*>(x) + src);
                        v = (KIND == DS_IN_I32_CLAMP) ? staged_of_code(raw, qc) : (__int2float_rn(raw) + 0.5f);
                    }
                }
                tile[cl][px] = v;
            }
        }
    }
    __syncthreads();
    // store: thread (c4 = t % 8, px = t / 8) writes four channels of pixels px, px + 32
    {
        const int c4 = threadIdx.x & 7;
        if (c0 + 4 * c4 < Cs) {
            for (int px = threadIdx.x >> 3; px < 64; px += 32) {
                const long long p = p0 + px;
                if (p >= npix) break;
                const long long b = p / HW;
                const int hw = int(p - b * HW);
                const int h = hw / W, w = hw - h * W;
                const long long o = ((b * (H + 2 * halo) + h + halo) * (W + 2 * halo) + w + halo) * Cs + c0 + 4 * c4;
                *reinterpret_cast<float4*>(dst + o) =
                    make_float4(tile[4 * c4][px], tile[4 * c4 + 1][px], tile[4 * c4 + 2][px], tile[4 * c4 + 3][px]);
            }
        }
    }
}

// Max pooling of int32 NHWC codes; a thread owns four channels of one output pixel.  Positions
// outside the image do not take part (F.max_pool2d's implicit -inf padding).  C % 4 == 0.
__global__ void __launch_bounds__(256) maxpool_nhwc_kernel(const int32_t* __restrict__ x, long long total, int H, int W,
                                                           int C, int OH, int OW, int k, int st, int pad,
                                                           int32_t* __restrict__ out_codes, float* __restrict__ out_staged,
                                                           int os_halo, CodeQuant q)
{
    const int C4 = C / 4;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c4 = int(i % C4);
        long long r = i / C4;
        const int ow = int(r % OW);
        r /= OW;
        const int oh = int(r % OH);
        const long long b = r / OH;
        int4 best = make_int4(INT_MIN, INT_MIN, INT_MIN, INT_MIN);
        for (int kh = 0; kh < k; ++kh) {
            const int ih = oh * st - pad + kh;
            if (unsigned(ih) >= unsigned(H)) continue;
            for (int kw = 0; kw < k; ++kw) {
                const int iw = ow * st - pad + kw;
                if (unsigned(iw) >= unsigned(W)) continue;
                const int4 v = __ldg(reinterpret_cast<const int4*>(x + ((b * H + ih) * W + iw) * C) + c4);
                best.x = max(best.x, v.x);
                best.y = max(best.y, v.y);
                best.z = max(best.z, v.z);
                best.w = max(best.w, v.w);
            }
        }
        if (out_codes) *reinterpret_cast<int4*>(out_codes + ((b * OH + oh) * OW + ow) * C + 4 * c4) = best;
        if (out_staged) {
            const long long o = ((b * (OH + 2 * os_halo) + oh + os_halo) * (OW + 2 * os_halo) + ow + os_halo) * C + 4 * c4;
            *reinterpret_cast<float4*>(out_staged + o) = make_float4(staged_of_code(best.x, q), staged_of_code(best.y, q),
                                                                     staged_of_code(best.z, q), staged_of_code(best.w, q));
        }
    }
}

// Global average of int32 NHWC codes and the LinearShift entry conversion: the exact integer sum,
// one rounding to fp32, / 2^F, / (H*W), trunc(. * 2^F)  (same rule as avgpool_fix_kernel in ds_misc.cu).
// A thread owns one (b, c); neighbouring threads read neighbouring channels.
__global__ void __launch_bounds__(256) avgpool_nhwc_kernel(const int32_t* __restrict__ x, int32_t* __restrict__ out,
                                                           long long total, int HW, int C, float inv_scale, float scale)
{
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long b = i / C;
    const int c = int(i - b * C);
    const int32_t* src = x + b * HW * C + c;
    long long sum = 0;
    for (int p = 0; p < HW; ++p) sum += __ldg(src + (long long)p * C);
    const float mean = __fdiv_rn(__ll2float_rn(sum) * inv_scale, float(HW));
    out[i] = __float2int_rz(mean * scale);
}

bool code_quant(int I, int F, CodeQuant& q)
{
    if (I < 1 || F < 0 || I + F > 18) return false;
    if (I == 1) {
        q.lo = -1; q.hi = 1; q.mul = 1 << F; q.add = -(1 << F);
    } else {
        q.lo = -(1 << (I - 1 + F));
        q.hi = ((1 << (I - 1)) - 1) * (1 << F);
        q.mul = 1;
        q.add = 0;
    }
    return true;
}

bool staged_ok(const ds_staged_t* t)
{
    return t && t->data && t->B >= 0 && t->H > 0 && t->W > 0 && t->C > 0 && t->halo >= 0 &&
           (reinterpret_cast<uintptr_t>(t->data) & 15u) == 0;
}

}  // namespace
}  // namespace ds

using namespace ds;

extern "C" int ds_staged_fill(const ds_staged_t* t, void* stream)
{
    if (!staged_ok(t)) return DS_ERR_BAD_ARG;
    const long long n4 = ds_staged_bytes(t->B, t->H, t->W, t->C, t->halo) / 16;
    if (n4 == 0) return DS_OK;
    const long long want = (n4 + 255) / 256;
    const int blocks = int(want > 148 * 32 ? 148 * 32 : want);
    staged_fill_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<float4*>(t->data), n4);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
}

extern "C" int ds_stage_nchw(const void* x, int in_kind, int I, int F, const ds_staged_t* dst, void* stream)
{
    if (!x || !staged_ok(dst)) return DS_ERR_BAD_ARG;
    if (in_kind != DS_IN_F32_CONV && in_kind != DS_IN_I32_CLAMP && in_kind != DS_IN_I32) return DS_ERR_BAD_ARG;
    if (dst->B == 0) return DS_OK;
    Quant qf = {};
    CodeQuant qc = {0, 0, 1, 0};
    if (in_kind != DS_IN_I32) {
        if (!code_quant(I, F, qc)) return DS_ERR_BAD_ARG;
        qf.scale = float(1ll << F);
        qf.sign_mode = (I == 1);
        qf.lo = -float(1ll << (I - 1 + F));
        qf.hi = float(((1ll << (I - 1)) - 1) * (1ll << F));
    }
    const int Cs = (dst->C + 3) / 4 * 4;
    const long long npix = (long long)dst->B * dst->H * dst->W;
    const long long gx = (npix + 63) / 64;
    if (gx > 2147483647LL) return DS_ERR_RANGE;
    const dim3 grid(unsigned(gx), unsigned((Cs + 31) / 32));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float* d = static_cast<float*>(dst->data);
    if (in_kind == DS_IN_F32_CONV)
        stage_nchw_kernel<DS_IN_F32_CONV><<<grid, 256, 0, st>>>(x, d, dst->B, dst->C, dst->H, dst->W, Cs, dst->halo, qf, qc);
    else if (in_kind == DS_IN_I32_CLAMP)
        stage_nchw_kernel<DS_IN_I32_CLAMP><<<grid, 256, 0, st>>>(x, d, dst->B, dst->C, dst->H, dst->W, Cs, dst->halo, qf, qc);
    else
        stage_nchw_kernel<DS_IN_I32><<<grid, 256, 0, st>>>(x, d, dst->B, dst->C, dst->H, dst->W, Cs, dst->halo, qf, qc);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
}

extern "C" int ds_maxpool_nhwc(const int32_t* x, int B, int H, int W, int C, int k, int stride, int pad,
                               int32_t* out_codes, const ds_staged_t* out_staged, int I, int F, void* stream)
{
    if (!x || B < 0 || C <= 0 || H <= 0 || W <= 0 || k <= 0 || stride <= 0 || pad < 0 || 2 * pad > k)
        return DS_ERR_BAD_ARG;
    if (H + 2 * pad < k || W + 2 * pad < k || (!out_codes && !out_staged)) return DS_ERR_BAD_ARG;
    if (C % 4 != 0) return DS_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out_codes)) & 15u) return DS_ERR_ALIGN;
    const int OH = (H + 2 * pad - k) / stride + 1, OW = (W + 2 * pad - k) / stride + 1;
    CodeQuant q = {0, 0, 1, 0};
    float* os = nullptr;
    int os_halo = 0;
    if (out_staged) {
        if (!staged_ok(out_staged) || out_staged->B != B || out_staged->H != OH || out_staged->W != OW ||
            out_staged->C != C || !code_quant(I, F, q))
            return DS_ERR_BAD_ARG;
        os = static_cast<float*>(out_staged->data);
        os_halo = out_staged->halo;
    }
    const long long total = (long long)B * OH * OW * (C / 4);
    if (total == 0) return DS_OK;
    const long long want = (total + 255) / 256;
    const int blocks = int(want > 148 * 64 ? 148 * 64 : want);
    maxpool_nhwc_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, total, H, W, C, OH, OW, k, stride, pad,
                                                                             out_codes, os, os_halo, q);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
}

extern "C" int ds_avgpool_fix_nhwc(const int32_t* x, int32_t* out, int B, int H, int W, int C, int F, void* stream)
{
    if (!x || !out || B < 0 || C <= 0 || H <= 0 || W <= 0 || F < 0 || F > 30) return DS_ERR_BAD_ARG;
    const long long total = (long long)B * C;
    if (total == 0) return DS_OK;
    const float scale = float(1ll << F);
    avgpool_nhwc_kernel<<<unsigned((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        x, out, total, H * W, C, 1.0f / scale, scale);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
}
