// Shared pieces of the V4 cousin path (block indexer, selection, sparse attention, KV compressor).
#pragma once

#include "codec.cuh"
#include "common.cuh"

__device__ __forceinline__ float v4_rbf16(float x) { return rv_bf16_to_f32(rv_f32_to_bf16(x)); }

// One element of an f32 or a bf16 array, widened exactly.
__device__ __forceinline__ float v4_load_f32(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float v4_load_f32(const uint16_t* p, size_t i) { return rv_bf16_to_f32(p[i]); }

constexpr int V4_ROT_MAX = 256;
constexpr float V4_FP4_MAX = 6.0f;

// e2m1 round trip of q (already clamped to [-6, 6]): nearest grid point, midpoints to the even code.
__device__ __forceinline__ float v4_e2m1_roundtrip(float q) {
    const float a = fabsf(q);
    int code = 0;
    code += a > 0.25f;
    code += a >= 0.75f;
    code += a > 1.25f;
    code += a >= 1.75f;
    code += a > 2.5f;
    code += a >= 3.5f;
    code += a > 5.0f;
    const float mag = code < 4 ? 0.5f * (float)code : (code == 4 ? 2.0f : (code == 5 ? 3.0f : (code == 6 ? 4.0f : 6.0f)));
    return signbit(q) ? -mag : mag;
}

// Smallest power of two >= amax / 6, from the exponent field of the product.
__device__ __forceinline__ float v4_round_scale(float amax) {
    const uint32_t b = __float_as_uint(__fmul_rn(amax, __fdiv_rn(1.0f, V4_FP4_MAX)));
    const int e = (int)((b >> 23) & 0xffu) - 127 + ((b & 0x7fffffu) ? 1 : 0);
    return __uint_as_float((uint32_t)(e + 127) << 23);
}

static inline int v4_check_geom(const V4Geom* g, int n_seqs) {
    if (!g || n_seqs <= 0) return 1001;
    if (g->n_heads <= 0 || g->head_dim <= 0 || g->window <= 0 || g->index_heads <= 0 || g->index_dim <= 0 ||
        g->index_topk <= 0 || g->ratio <= 1 || g->max_comp <= 0)
        return 1001;
    return 0;
}
