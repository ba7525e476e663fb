// Shared declarations of the deepshift_b200 CUDA sources (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/deepshift_b200.h"

namespace ds {

// Host-side count of the kernels this library has launched (ds_launch_count); every launch site
// calls note_launch right after its <<<>>>.
void note_launch(int n = 1);
long long launch_count();

// Index of the current CUDA device for the small per-device caches the launch code keeps
// (function attributes are set per device); -1 when it cannot be had or is out of range.
constexpr int kMaxDevices = 64;
inline int device_slot()
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
    return dev;
}

// 1.5 * 2^23: a float in [2^23, 2^24) has ulp 1, so MAGIC + a (|a| < 2^22) keeps a as a
// two's-complement integer in its low mantissa bits.
constexpr float kMagic = 12582912.0f;
constexpr int kMagicBits = 0x4B400000;
// 1.5 * 2^22: ulp 0.5, used to build x + 0.5 from an integer x with one integer and one float add.
constexpr float kHalfMagic = 6291456.0f;
constexpr int kHalfMagicBits = 0x4AC00000;

// Decode parameters of one packed weight tensor.
struct Decode {
    int bits;     // width of the shift field
    int fw;       // bits + 1: field + sign bit
    int num;      // weights per word = 32 / fw
    int base;     // added to the field to get the net right shift
    int row_len;  // words per output row
};

// One decoded weight for the integer path: term = (x >> sh) * mul.
//   right shift r in [0,31]: sh = r, mul = +-1;  left shift: sh = 0, mul = +-2^-r;
//   zero weight: sh = 0, mul = 0.
__device__ __forceinline__ void decode_int(uint32_t field, const Decode& d, bool live, int& sh,
                                           int& mul)
{
    const int r = int(field & ((1u << d.bits) - 1u)) + d.base;
    const int sgn = ((field >> d.bits) & 1u) ? 1 : -1;
    if (!live || r >= 32) { sh = 0; mul = 0; }
    else if (r >= 0) { sh = r; mul = sgn; }
    else { sh = 0; mul = (-r >= 32) ? 0 : int(uint32_t(sgn) << (-r)); }
}

// One decoded weight for the FP32-pipe path: +-2^-r as a float (exact), 0 for a zero weight.
// Only used with base == 0, so r >= 0.
__device__ __forceinline__ float decode_f32(uint32_t field, const Decode& d, bool live, int& neg)
{
    const int r = int(field & ((1u << d.bits) - 1u)) + d.base;
    const bool pos = (field >> d.bits) & 1u;
    const bool nz = live && r < 32;
    neg = (nz && !pos) ? 1 : 0;
    const uint32_t b = (uint32_t(127 - r) << 23) | (pos ? 0u : 0x80000000u);
    return nz ? __uint_as_float(b) : 0.0f;
}

// Fixed-point entry of the reference's Python layer, on one fp32 value.
//   DS_IN_F32_CONV  : int(clamp(floor(x / 2^-F) * 2^-F, -2^(I-1), 2^(I-1)-1) * 2^F)
//   DS_IN_F32_LINEAR: int(x * 2^F), truncation toward zero, no clamp
// Scaling by a power of two is exact, so the clamp can be applied to the scaled value.
struct Quant {
    float scale;  // 2^F
    float lo;     // -2^(I-1+F)
    float hi;     // (2^(I-1)-1) * 2^F
    int sign_mode;  // I == 1: round_to_fixed returns sign(x) - 1 (utils.py:12-13)
};

__device__ __forceinline__ float quant_conv_f(float x, const Quant& q)
{
    if (q.sign_mode) {
        const float s = (x > 0.f) ? 1.f : ((x < 0.f) ? -1.f : 0.f);
        return (s - 1.f) * q.scale;
    }
    return fminf(fmaxf(floorf(x * q.scale), q.lo), q.hi);
}

const char* status_string(int s);

}  // namespace ds
