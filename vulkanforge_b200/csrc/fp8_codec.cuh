// Device-side E4M3 / binary16 converters.  Bit-for-bit the same results as the
// reference's CPU codec (src/backend/vulkan/fp8_ext.rs:104-211): round to
// nearest even, |x| >= 448 (and +-Inf) saturate to 0x7E, NaN -> 0x7F with the
// sign dropped, signed zeros kept.
#pragma once

#include <cuda_fp16.h>
#include <cstdint>

namespace vfkv {

// Two floats -> two E4M3 codes, `lo` in bits 0-7 and `hi` in bits 8-15.
// cvt.rn.satfinite.e4m3x2.f32 rounds to nearest even and clamps finite
// overflow and infinities to +-448; a NaN input comes back as a NaN code whose
// sign is not specified, so NaNs are forced to 0x7F afterwards.
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float lo, float hi)
{
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    uint32_t v = r;
    if (lo != lo) v = (v & 0xFF00u) | 0x7Fu;
    if (hi != hi) v = (v & 0x00FFu) | 0x7F00u;
    return v;
}

__device__ __forceinline__ uint32_t f32x4_to_e4m3x4(float a, float b, float c, float d)
{
    return f32x2_to_e4m3x2(a, b) | (f32x2_to_e4m3x2(c, d) << 16);
}

// Two E4M3 codes (bits 0-15) -> half2; exact, every E4M3 value is a binary16 value.
__device__ __forceinline__ __half2 e4m3x2_to_half2(uint32_t v)
{
    uint32_t r;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"((uint16_t)v));
    return *reinterpret_cast<__half2 *>(&r);
}

__device__ __forceinline__ float2 e4m3x2_to_float2(uint32_t v)
{
    return __half22float2(e4m3x2_to_half2(v));
}

// packHalf2x16 of vk_shaders/kv_copy_fp16.comp:50 with round-to-nearest-even:
// first element in the low half.
__device__ __forceinline__ uint32_t f32x2_to_f16x2(float lo, float hi)
{
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

}  // namespace vfkv
