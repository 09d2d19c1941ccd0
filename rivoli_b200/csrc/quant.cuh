// Warp-cooperative fp8 e4m3 quantisation of token rows into the paged pools: shared by the
// append operator and by the fused decode-step prologue.
#pragma once

#include "codec.cuh"
#include "common.cuh"

// ------------------------------------------------------------------------------------------
// Paged layout. One warp per token row; 4 rows per CTA.
//   latent row (c_kv | k_rope, <= 1024 values, one scale): lane owns two 16-value chunks.
//   key (index_dim <= 512, one scale):                      lane owns one 16-value chunk.
// Every store is one 16-byte vector. A lane whose chunk lies past the vector's end
// contributes 0 to the absmax and stores nothing, so any multiple of 16 works.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void unpack8(const uint4& p, float* f) {
    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// A vector of `n` bf16 values (n % 16 == 0, n <= 512) spread over a warp, 16 values per lane, in
// two steps so a caller can have several vectors' loads in flight before it finishes any.
__device__ __forceinline__ bool load_vec16(const uint16_t* __restrict__ src, int n, int lane, float (&f)[16]) {
    const bool act = lane * 16 < n;
    if (act) {
        const uint4* p = reinterpret_cast<const uint4*>(src + lane * 16);
        unpack8(p[0], f);
        unpack8(p[1], f + 8);
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) f[i] = 0.0f;
    }
    return act;
}
__device__ __forceinline__ void store_codes16(const float (&f)[16], float scl, uint8_t* __restrict__ dst) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t lo = rv_f32x2_to_e4m3x2(__fdiv_rn(f[4 * i], scl), __fdiv_rn(f[4 * i + 1], scl));
        uint32_t hi = rv_f32x2_to_e4m3x2(__fdiv_rn(f[4 * i + 2], scl), __fdiv_rn(f[4 * i + 3], scl));
        w[i] = lo | (hi << 16);
    }
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ float absmax16(const float (&f)[16]) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
    return amax;
}

// Quantise a vector of `n` bf16 values (n % 16 == 0, n <= 512) cooperatively across a
// warp; returns the scale (all lanes) and stores 16 codes per active lane.
__device__ __forceinline__ float quant_vec16(const uint16_t* __restrict__ src, int n, uint8_t* __restrict__ dst,
                                             int lane) {
    float f[16];
    const bool act = load_vec16(src, n, lane, f);
    const float scl = rv_scale_from_amax(rv_warp_max(absmax16(f)));
    if (act) store_codes16(f, scl, dst + lane * 16);
    return scl;
}

// A row of up to 1024 bf16 values (n % 16 == 0) under ONE scale: lane owns the 16-value chunks
// lane and lane + 32, so each store is still a single 16-byte vector.
__device__ __forceinline__ float quant_row_wide(const uint16_t* __restrict__ src, int n, uint8_t* __restrict__ dst,
                                                int lane) {
    float f0[16], f1[16];
    const bool a0 = load_vec16(src, n, lane, f0), a1 = load_vec16(src, n, lane + 32, f1);
    const float scl = rv_scale_from_amax(rv_warp_max(fmaxf(absmax16(f0), absmax16(f1))));
    if (a0) store_codes16(f0, scl, dst + lane * 16);
    if (a1) store_codes16(f1, scl, dst + (lane + 32) * 16);
    return scl;
}

// One token row into the paged pools, by one warp. The row's latent and key loads are issued
// together with the page lookup, so the position -> page -> store chain costs two memory round
// trips (position, then everything else) instead of four.
__device__ __forceinline__ void append_row_paged(const DsaGeom& g, const uint16_t* __restrict__ latent,
                                                 const uint16_t* __restrict__ index_key, int row, int seq, int pos,
                                                 const int32_t* __restrict__ block_table,
                                                 uint8_t* __restrict__ latent_pool, float* __restrict__ latent_scale,
                                                 uint8_t* __restrict__ index_pool, float* __restrict__ index_scale,
                                                 int32_t* __restrict__ status, int lane) {
    const int w = g.kv_lora + g.rope_dim;
    const int lp = pos / g.page_tokens;
    int page = -1;
    if (pos >= 0 && lp < g.max_pages_per_seq) page = block_table[(size_t)seq * g.max_pages_per_seq + lp];
    float f0[16], f1[16], fk[16];
    const uint16_t* src = latent + (size_t)row * w;
    const bool a0 = load_vec16(src, w, lane, f0), a1 = load_vec16(src, w, lane + 32, f1);
    const bool ak = load_vec16(index_key + (size_t)row * g.index_dim, g.index_dim, lane, fk);
    const float s_l = rv_scale_from_amax(rv_warp_max(fmaxf(absmax16(f0), absmax16(f1))));   // c_kv and k_rope share one scale
    const float s_i = rv_scale_from_amax(rv_warp_max(absmax16(fk)));
    if (page < 0 || page >= g.n_pool_pages) {
        if (lane == 0 && status) atomicOr(status, 1);
        return;
    }
    const size_t r = (size_t)page * g.page_tokens + (pos & (g.page_tokens - 1));
    uint8_t* dl = latent_pool + r * w;
    if (a0) store_codes16(f0, s_l, dl + lane * 16);
    if (a1) store_codes16(f1, s_l, dl + (lane + 32) * 16);
    if (ak) store_codes16(fk, s_i, index_pool + r * g.index_dim + lane * 16);
    if (lane == 0) {
        latent_scale[r] = s_l;
        index_scale[r] = s_i;
    }
}
