// Element codecs on the device. Bit-for-bit the CPU rules of the reference's
// crates/core/src/num.rs:86-201 (its device twins: crates/backend/kernels/fwd.hip:20-45,
// crates/backend/kernels/formats.hpp:42-106).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

// bf16 bits -> f32, exact.
__device__ __forceinline__ float rv_bf16_to_f32(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }

// f32 -> bf16 bits, round to nearest even; NaN stays NaN (quiet).
__device__ __forceinline__ uint16_t rv_f32_to_bf16(float x) {
    uint32_t b = __float_as_uint(x);
    if ((b & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((b >> 16) | 0x0040u);
    uint32_t r = ((b >> 16) & 1u) + 0x7fffu;
    return (uint16_t)((b + r) >> 16);
}

// Software path for |x| < 2^-6 (e4m3 subnormals and zero) and NaN: the reference rounds
// subnormals HALF AWAY from zero and promotes m == 8 to the smallest normal, which the
// hardware converter (round to nearest EVEN everywhere) does not reproduce on exact ties.
__device__ __forceinline__ uint8_t rv_e4m3_small(float x) {
    if (x != x) return 0x7f;
    uint8_t sign = (uint8_t)((__float_as_uint(x) >> 24) & 0x80u);
    float a = fabsf(x);
    if (a < 0.0009765625f) return sign;  // < 2^-10
    float s = a * 512.0f;                // exact
    float fl = floorf(s);
    int m = (int)fl + ((s - fl) >= 0.5f ? 1 : 0);
    return m >= 8 ? (uint8_t)(sign | 0x08) : (uint8_t)(sign | (uint8_t)m);
}

// Two f32 -> two e4m3 codes (lo byte = a, hi byte = b). Normals go through the sm_100
// converter (RNE over the dropped mantissa bits with carry, saturating to +-448 = 0x7e);
// values below 2^-6 in magnitude and NaN take the software path above.
__device__ __forceinline__ uint16_t rv_f32x2_to_e4m3x2(float a, float b) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(r) : "f"(a), "f"(b));
    if (!(fabsf(a) >= 0.015625f)) r = (uint16_t)((r & 0xff00u) | rv_e4m3_small(a));
    if (!(fabsf(b) >= 0.015625f)) r = (uint16_t)((r & 0x00ffu) | ((uint16_t)rv_e4m3_small(b) << 8));
    return r;
}

__device__ __forceinline__ uint8_t rv_f32_to_e4m3(float a) { return (uint8_t)(rv_f32x2_to_e4m3x2(a, 0.0f) & 0xff); }

// Two e4m3 codes (16 bits) -> two f32, exact (e4m3 -> f16 is exact; f16 -> f32 is exact).
__device__ __forceinline__ float2 rv_e4m3x2_to_f32x2(uint16_t c) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(c));
    __half2 h = *reinterpret_cast<__half2*>(&h2);
    return __half22float2(h);
}

__device__ __forceinline__ float rv_e4m3_to_f32(uint8_t c) { return rv_e4m3x2_to_f32x2((uint16_t)c).x; }

// Quantise with the reference's scale rule: scl = amax > 0 ? amax/448 : 1 (IEEE divide).
__device__ __forceinline__ float rv_scale_from_amax(float amax) {
    return amax > 0.0f ? __fdiv_rn(amax, 448.0f) : 1.0f;
}
