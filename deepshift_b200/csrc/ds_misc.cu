// Weight packing, the standalone quantiser, the issue-rate probe and the status strings.
#include <climits>

#include "ds_common.cuh"

#include <atomic>

namespace ds {
namespace {

// One thread per output word: OR together up to `num` (field, sign) pairs of one row.
// Layout of the reference's COMPRESS helper (shift.cu:27-38): field in the low `bits`
// bits of the slot, (sign > 0) in the bit above it.
__global__ void compress_kernel(const int32_t* __restrict__ shiftp, const int32_t* __restrict__ sign,
                                int32_t* __restrict__ packed, int OC, int K, int bits, int base, int num,
                                int row_len)
{
    const long long total = (long long)OC * row_len;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int oc = int(i / row_len), w = int(i - (long long)oc * row_len);
        const int k0 = w * num;
        const int len = min(num, K - k0);
        const int32_t* sp = shiftp + (long long)oc * K + k0;
        const int32_t* gp = sign + (long long)oc * K + k0;
        uint32_t value = 0;
        int s = 0;
        for (int j = 0; j < len; ++j) {
            value |= uint32_t(__ldg(sp + j) - base) << s;
            s += bits;
            value |= uint32_t(__ldg(gp + j) > 0 ? 1 : 0) << s;
            s += 1;
        }
        packed[i] = int32_t(value);
    }
}

__global__ void quantize_kernel(const float* __restrict__ x, int32_t* __restrict__ out, long long n, int kind,
                                Quant q)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        const float v = __ldg(x + i);
        out[i] = (kind == DS_IN_F32_CONV) ? __float2int_rz(quant_conv_f(v, q)) : __float2int_rz(v * q.scale);
    }
}

// Element types of the max pools: int32 codes, or fp32 values with torch's rule that a NaN in the
// window is the result.
template <typename T>
struct Pool;
template <>
struct Pool<int32_t> {
    using V4 = int4;
    static __device__ __forceinline__ int32_t lowest() { return INT_MIN; }
    static __device__ __forceinline__ int32_t mx(int32_t a, int32_t b) { return max(a, b); }
};
template <>
struct Pool<float> {
    using V4 = float4;
    static __device__ __forceinline__ float lowest() { return __int_as_float(0xff800000); }  // -inf
    static __device__ __forceinline__ float mx(float a, float b) { return (b > a || b != b) ? b : a; }
};

// Max pooling on NCHW; positions outside the image do not take part (as with
// torch.nn.functional.max_pool2d's implicit -inf padding).  On int32 codes: monotone, hence identical
// to pooling the fp32 values int / 2^F and converting back.
template <typename T>
__global__ void maxpool_kernel(const T* __restrict__ x, T* __restrict__ out, long long total, int H,
                               int W, int OH, int OW, int k, int st, int pad)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int ow = int(i % OW);
        const long long r = i / OW;
        const int oh = int(r % OH);
        const long long bc = r / OH;
        const T* src = x + bc * H * W;
        T best = Pool<T>::lowest();
        for (int kh = 0; kh < k; ++kh) {
            const int ih = oh * st - pad + kh;
            if (unsigned(ih) >= unsigned(H)) continue;
            for (int kw = 0; kw < k; ++kw) {
                const int iw = ow * st - pad + kw;
                if (unsigned(iw) < unsigned(W)) best = Pool<T>::mx(best, __ldg(src + ih * W + iw));
            }
        }
        out[i] = best;
    }
}

// The 3x3 / stride 2 / padding 1 pool of the ResNet stem when W is a multiple of 8 and both
// tensors are 16-byte aligned: a thread produces four neighbouring outputs from, per input row,
// two 16-byte loads and the one value to their left (9 loads instead of 36), one 16-byte store.
template <typename T>
__global__ void __launch_bounds__(256) maxpool3s2_quad_kernel(const T* __restrict__ x, T* __restrict__ out,
                                                              long long quads, int H, int W, int OH, int OW)
{
    using V4 = typename Pool<T>::V4;
    auto mx = [](T a, T b) { return Pool<T>::mx(a, b); };
    const int qw = OW / 4;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < quads;
         i += (long long)gridDim.x * blockDim.x) {
        const int q = int(i % qw);
        const long long r = i / qw;
        const int oh = int(r % OH);
        const long long bc = r / OH;
        const T* src = x + bc * H * W + 8 * q;
        const T lo = Pool<T>::lowest();
        V4 best;
        best.x = best.y = best.z = best.w = lo;
#pragma unroll
        for (int kh = 0; kh < 3; ++kh) {
            const int ih = 2 * oh - 1 + kh;
            if (unsigned(ih) >= unsigned(H)) continue;
            const T* row = src + (long long)ih * W;
            const V4 a = __ldg(reinterpret_cast<const V4*>(row));
            const V4 b = __ldg(reinterpret_cast<const V4*>(row) + 1);
            const T left = q > 0 ? __ldg(row - 1) : lo;
            best.x = mx(best.x, mx(left, mx(a.x, a.y)));
            best.y = mx(best.y, mx(a.y, mx(a.z, a.w)));
            best.z = mx(best.z, mx(a.w, mx(b.x, b.y)));
            best.w = mx(best.w, mx(b.y, mx(b.z, b.w)));
        }
        *reinterpret_cast<V4*>(out + (bc * OH + oh) * OW + 4 * q) = best;
    }
}

// Global average pooling of int32 fixed-point planes followed by the LinearShift entry
// conversion: one warp per (b, c) plane sums the codes exactly (int64), then
// mean = float(sum) * 2^-F / (H*W) in fp32 and out = trunc(mean * 2^F).
__global__ void avgpool_fix_kernel(const int32_t* __restrict__ x, int32_t* __restrict__ out, int planes, int hw,
                                   float inv_scale, float scale)
{
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= planes) return;
    const int32_t* src = x + (long long)warp * hw;
    long long sum = 0;
    for (int i = lane; i < hw; i += 32) sum += __ldg(src + i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) {
        const float mean = __fdiv_rn(__ll2float_rn(sum) * inv_scale, float(hw));
        out[warp] = __float2int_rz(mean * scale);
    }
}

// ---- issue-rate probe: 16 independent chains per thread, register operands only ----------------
constexpr int kChains = 16;

template <int MODE>
__global__ void __launch_bounds__(256) peak_kernel(int iters, int seed, int* sink)
{
    int s[4];
    int mu[4];
    float wf[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        s[j] = ((seed >> (3 * j)) & 7) + 1;  // shift amounts unknown to the compiler
        mu[j] = ((seed >> j) & 1) ? 1 : -1;
        wf[j] = __int_as_float(((127 - s[j]) << 23) | (((seed >> j) & 1) ? 0 : 0x80000000));
    }
    int a[kChains];
    float f[kChains];
#pragma unroll
    for (int c = 0; c < kChains; ++c) {
        a[c] = seed * (threadIdx.x + 1) + c * 977;
        f[c] = kMagic + float(c);
    }
    const float xf = float(threadIdx.x) + 0.5f;
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < kChains; ++c) {
                if (MODE == 0) a[c] = a[c] + (a[(c + 1) % kChains] >> s[r]);
                else if (MODE == 1) a[c] = (a[(c + 1) % kChains] >> s[r]) * mu[r] + a[c];
                else f[c] = __fmaf_rd(xf, wf[r], f[c]);
            }
    }
    int r = 0;
#pragma unroll
    for (int c = 0; c < kChains; ++c) r ^= (MODE == 2) ? __float_as_int(f[c]) : a[c];
    if (r == 0x7fffffff) *sink = r;  // practically never; keeps the work alive
}

}  // namespace

static std::atomic<long long> g_launches{0};

void note_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

const char* status_string(int s)
{
    switch (s) {
        case DS_OK: return "ok";
        case DS_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size or inconsistent shape)";
        case DS_ERR_UNSUPPORTED: return "unsupported configuration (bits outside 1..7, base > 0, window > 31)";
        case DS_ERR_CUDA: return "CUDA runtime error at launch";
        case DS_ERR_RANGE: return "size exceeds 32-bit indexing limits of this build";
        case DS_ERR_ALIGN: return "pointer not sufficiently aligned (outputs need 16 bytes)";
        case DS_ERR_SCRATCH:
            return "problem has more output tiles than the fixed scratch of the no-allocation entry point holds "
                   "(16384 tiles of 256 positions x 128 channels)";
        default: return "unknown status";
    }
}

}  // namespace ds

using namespace ds;

extern "C" int ds_compress(const int32_t* shiftp, const int32_t* sign, int32_t* packed, int OC, int K,
                           int bits, int base, void* stream)
{
    if (!shiftp || !sign || !packed || OC <= 0 || K <= 0) return DS_ERR_BAD_ARG;
    if (bits < 1 || bits > 7) return DS_ERR_UNSUPPORTED;
    const int num = 32 / (bits + 1);
    const int row_len = (K + num - 1) / num;
    const long long total = (long long)OC * row_len;
    const int threads = 256;
    const int blocks = int(total / threads + 1 > 148 * 16 ? 148 * 16 : total / threads + 1);
    compress_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(shiftp, sign, packed, OC, K, bits,
                                                                             base, num, row_len);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
}

extern "C" int ds_quantize_f32(const float* x, int32_t* out, long long n, int kind, int I, int F, void* stream)
{
    if (n < 0 || (n > 0 && (!x || !out))) return DS_ERR_BAD_ARG;
    if (kind != DS_IN_F32_CONV && kind != DS_IN_F32_LINEAR) return DS_ERR_BAD_ARG;
    if (F < 0 || F > 30 || (kind == DS_IN_F32_CONV && (I < 1 || I + F > 32))) return DS_ERR_BAD_ARG;
    if (n == 0) return DS_OK;
    Quant q;
    q.scale = float(1ll << F);
    q.sign_mode = (kind == DS_IN_F32_CONV && I == 1);
    q.lo = q.hi = 0.f;
    if (kind == DS_IN_F32_CONV) {
        q.lo = -float(1ll << (I - 1 + F));
        q.hi = float(((1ll << (I - 1)) - 1) * (1ll << F));
    }
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    const int blocks = int(want > 148 * 32 ? 148 * 32 : want);
    quantize_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(x, out, n, kind, q);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
}

template <typename T>
static int maxpool2d_run(const T* x, T* out, int B, int C, int H, int W, int k, int stride, int pad, void* stream)
{
    if (!x || !out || B < 0 || C <= 0 || H <= 0 || W <= 0 || k <= 0 || stride <= 0 || pad < 0 || 2 * pad > k)
        return DS_ERR_BAD_ARG;
    if (H + 2 * pad < k || W + 2 * pad < k) return DS_ERR_BAD_ARG;
    const int OH = (H + 2 * pad - k) / stride + 1, OW = (W + 2 * pad - k) / stride + 1;
    const long long total = (long long)B * C * OH * OW;
    if (total == 0) return DS_OK;
    const int threads = 256;
    if (k == 3 && stride == 2 && pad == 1 && W % 8 == 0 &&
        ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0) {
        const long long quads = total / 4;  // OW = W / 2 is a multiple of 4
        const long long wantq = (quads + threads - 1) / threads;
        const int blocksq = int(wantq > 148 * 64 ? 148 * 64 : wantq);
        maxpool3s2_quad_kernel<T><<<blocksq, threads, 0, static_cast<cudaStream_t>(stream)>>>(x, out, quads, H, W,
                                                                                             OH, OW);
        note_launch();
        return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
    }
    const long long want = (total + threads - 1) / threads;
    const int blocks = int(want > 148 * 32 ? 148 * 32 : want);
    maxpool_kernel<T><<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(x, out, total, H, W, OH, OW, k,
                                                                               stride, pad);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
}

extern "C" int ds_maxpool2d_i32(const int32_t* x, int32_t* out, int B, int C, int H, int W, int k, int stride,
                                int pad, void* stream)
{
    return maxpool2d_run<int32_t>(x, out, B, C, H, W, k, stride, pad, stream);
}

extern "C" int ds_maxpool2d_f32(const float* x, float* out, int B, int C, int H, int W, int k, int stride, int pad,
                                void* stream)
{
    return maxpool2d_run<float>(x, out, B, C, H, W, k, stride, pad, stream);
}

// y = relu?(y + r) in place, four elements per thread where the pointers allow.
__global__ void __launch_bounds__(256) add_relu_f32_kernel(float* __restrict__ y, const float* r, long long n,
                                                           int relu, int vec)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long first = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    auto fin = [&](float a, float b) {
        const float f = a + b;
        return (relu && f < 0.f) ? 0.f : f;
    };
    if (vec) {
        const long long n4 = n >> 2;
        float4* y4 = reinterpret_cast<float4*>(y);
        const float4* r4 = reinterpret_cast<const float4*>(r);
        for (long long i = first; i < n4; i += stride) {
            const float4 a = y4[i];
            const float4 b = r ? __ldg(r4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            y4[i] = make_float4(fin(a.x, b.x), fin(a.y, b.y), fin(a.z, b.z), fin(a.w, b.w));
        }
        for (long long i = (n4 << 2) + first; i < n; i += stride) y[i] = fin(y[i], r ? r[i] : 0.f);
    } else {
        for (long long i = first; i < n; i += stride) y[i] = fin(y[i], r ? r[i] : 0.f);
    }
}

extern "C" int ds_add_relu_f32(float* y, const float* r, long long n, int relu, void* stream)
{
    if (!y || n < 0) return DS_ERR_BAD_ARG;
    if (n == 0 || (!r && !relu)) return DS_OK;
    if ((reinterpret_cast<uintptr_t>(y) & 3u) || (reinterpret_cast<uintptr_t>(r) & 3u)) return DS_ERR_ALIGN;
    const int vec = ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(r)) & 15u) == 0;
    const int threads = 256;
    const long long want = ((vec ? (n + 3) / 4 : n) + threads - 1) / threads;
    const int blocks = int(want > 148 * 32 ? 148 * 32 : want);
    add_relu_f32_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(y, r, n, relu, vec);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
}

extern "C" int ds_avgpool_fix_i32(const int32_t* x, int32_t* out, int B, int C, int H, int W, int F, void* stream)
{
    if (!x || !out || B < 0 || C <= 0 || H <= 0 || W <= 0 || F < 0 || F > 30) return DS_ERR_BAD_ARG;
    const long long planes = (long long)B * C;
    if (planes == 0) return DS_OK;
    if (planes > 2147483647LL / 32) return DS_ERR_RANGE;
    const int threads = 256;
    const int blocks = int((planes * 32 + threads - 1) / threads);
    const float scale = float(1ll << F);
    avgpool_fix_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(x, out, int(planes), H * W,
                                                                                1.0f / scale, scale);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? DS_OK : DS_ERR_CUDA;
}

extern "C" int ds_pipe_peak(int mode, int iters, double* ops_per_s, void* stream)
{
    if (!ops_per_s || iters <= 0 || mode < 0 || mode > 2) return DS_ERR_BAD_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return DS_ERR_CUDA;
    int* sink = nullptr;
    if (cudaMalloc(&sink, sizeof(int)) != cudaSuccess) return DS_ERR_CUDA;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    const int blocks = sms * 8, threads = 256;
    auto run = [&](int n) {
        if (mode == 0) peak_kernel<0><<<blocks, threads, 0, st>>>(n, 0x2b5a9, sink);
        else if (mode == 1) peak_kernel<1><<<blocks, threads, 0, st>>>(n, 0x2b5a9, sink);
        else peak_kernel<2><<<blocks, threads, 0, st>>>(n, 0x2b5a9, sink);
        note_launch();
    };
    run(iters / 8 + 1);  // warm-up
    cudaEventRecord(e0, st);
    run(iters);
    cudaEventRecord(e1, st);
    int rc = DS_OK;
    if (cudaEventSynchronize(e1) != cudaSuccess || cudaGetLastError() != cudaSuccess) rc = DS_ERR_CUDA;
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(sink);
    if (rc == DS_OK && ms > 0.f)
        *ops_per_s = double(blocks) * threads * double(iters) * 4.0 * kChains / (double(ms) * 1e-3);
    return rc;
}

extern "C" const char* ds_strerror(int status) { return status_string(status); }
extern "C" int ds_version(void) { return 100; }

// Kernels launched by this library in this process so far (host-side counter).
extern "C" long long ds_launch_count(void) { return ds::launch_count(); }
