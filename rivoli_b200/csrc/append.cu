// KV-cache append: quantise new tokens to fp8 e4m3 with absmax scales and store them.
//
//   rivoli_append_kv / rivoli_index_append / rivoli_gather_rope : the reference's
//       single-token, contiguous-slab operators (crates/backend/kernels/fwd.hip:47-84,
//       crates/backend/kernels/indexer.hip:52-58).
//   rivoli_kv_append_paged / rivoli_index_q_quant : the batched paged form.
//
// All of it is HBM-bound byte work: one warp per 128-wide (or per-vector) quantisation
// group, absmax by warp shuffle (max is order independent, so the result is bit exact),
// IEEE division by the scale, packed code stores (16 bytes per lane on the latent row).
#include "codec.cuh"
#include "common.cuh"
#include "quant.cuh"

// ------------------------------------------------------------------------------------------
// Reference layout: one token, f32 in, block of 128 per scale.
// One warp per 128-block (4 values per lane); the rope half rides warp 0.. as bf16.
// ------------------------------------------------------------------------------------------
__global__ void append_kv_slab_kernel(const float* __restrict__ latent, const float* __restrict__ rope,
                                      unsigned char* __restrict__ lc8, float* __restrict__ lscale,
                                      unsigned short* __restrict__ rc, int pos, int kvl, int ropn,
                                      int n_blocks) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blk = warp;  // kvl/128 warps
    const float* src = latent + blk * 128 + lane * 4;  // scalar loads: no alignment demand on the caller
    const float4 v = make_float4(src[0], src[1], src[2], src[3]);
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    amax = rv_warp_max(amax);
    const float scl = rv_scale_from_amax(amax);
    if (lane == 0) lscale[(size_t)pos * n_blocks + blk] = scl;
    const uint32_t lo = rv_f32x2_to_e4m3x2(__fdiv_rn(v.x, scl), __fdiv_rn(v.y, scl));
    const uint32_t hi = rv_f32x2_to_e4m3x2(__fdiv_rn(v.z, scl), __fdiv_rn(v.w, scl));
    reinterpret_cast<uint32_t*>(lc8 + (size_t)pos * kvl + blk * 128)[lane] = lo | (hi << 16);
    for (int i = threadIdx.x; i < ropn; i += blockDim.x) rc[(size_t)pos * ropn + i] = rv_f32_to_bf16(rope[i]);
}

RIVOLI_API int rivoli_append_kv(const float* latent, const float* rope, unsigned char* lc8,
                                float* lscale, unsigned short* rc, int pos, int kvl, int ropn,
                                int n_blocks) {
    if (pos < 0 || kvl <= 0 || ropn <= 0 || n_blocks <= 0) return 1001;
    if (kvl > 1024 || kvl < 128 || (kvl % 128) != 0 || ropn > kvl) return 1002;
    rv_drain_error();
    append_kv_slab_kernel<<<1, (kvl / 128) * 32>>>(latent, rope, lc8, lscale, rc, pos, kvl, ropn, n_blocks);
    return rv_launch_status();
}

__global__ void gather_rope_kernel(const float* __restrict__ q, float* __restrict__ qrope, int h, int qh,
                                   int nope, int ropn) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= h * ropn) return;
    qrope[idx] = q[(size_t)(idx / ropn) * qh + nope + idx % ropn];
}

RIVOLI_API int rivoli_gather_rope(const float* q, float* qrope, int h, int qh, int nope, int ropn) {
    if (h <= 0 || qh <= 0 || nope < 0 || ropn <= 0) return 1001;
    rv_drain_error();
    gather_rope_kernel<<<(h * ropn + 255) / 256, 256>>>(q, qrope, h, qh, nope, ropn);
    return rv_launch_status();
}

__global__ void index_append_slab_kernel(const float* __restrict__ k, unsigned short* __restrict__ kcache,
                                         int pos, int hd) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < hd) kcache[(size_t)pos * hd + i] = rv_f32_to_bf16(k[i]);
}

RIVOLI_API int rivoli_index_append(const float* k, unsigned short* kcache, int pos, int hd) {
    if (hd <= 0 || pos < 0) return 1001;
    rv_drain_error();
    index_append_slab_kernel<<<(hd + 255) / 256, 256>>>(k, kcache, pos, hd);
    return rv_launch_status();
}

__global__ void __launch_bounds__(128)
kv_append_paged_kernel(DsaGeom g, const uint16_t* __restrict__ latent, const uint16_t* __restrict__ index_key,
                       const int32_t* __restrict__ row_seq, const int32_t* __restrict__ row_pos, int n_rows,
                       const int32_t* __restrict__ block_table, uint8_t* __restrict__ latent_pool,
                       float* __restrict__ latent_scale, uint8_t* __restrict__ index_pool,
                       float* __restrict__ index_scale, int32_t* __restrict__ status) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    append_row_paged(g, latent, index_key, row, row_seq ? row_seq[row] : row, row_pos[row], block_table, latent_pool,
                     latent_scale, index_pool, index_scale, status, lane);
}

RIVOLI_API int rivoli_kv_append_paged(const DsaGeom* g, const uint16_t* latent, const uint16_t* index_key,
                                      const int32_t* row_seq, const int32_t* row_pos, int n_rows,
                                      const int32_t* block_table, uint8_t* latent_pool,
                                      float* latent_scale, uint8_t* index_pool, float* index_scale,
                                      int32_t* status, void* stream) {
    if (int e = rv_check_geom(g)) return e;
    if (n_rows <= 0 || !latent || !index_key || !row_pos || !block_table || !latent_pool ||
        !latent_scale || !index_pool || !index_scale)
        return 1001;
    if ((g->rope_dim % 4) != 0 || ((g->kv_lora + g->rope_dim) % 16) != 0) return 1004;
    // 16-byte vector loads/stores: rows are multiples of 16 bytes, so only the bases matter.
    if ((((uintptr_t)latent | (uintptr_t)index_key | (uintptr_t)latent_pool | (uintptr_t)index_pool) & 15) ||
        ((uintptr_t)latent_scale & 3))
        return 1005;
    rv_drain_error();
    kv_append_paged_kernel<<<(n_rows + 3) / 4, 128, 0, (cudaStream_t)stream>>>(
        *g, latent, index_key, row_seq, row_pos, n_rows, block_table, latent_pool, latent_scale,
        index_pool, index_scale, status);
    return rv_launch_status();
}

// Indexer query vectors: one warp per vector, same codec and scale rule.
__global__ void __launch_bounds__(128)
index_q_quant_kernel(const uint16_t* __restrict__ q, int n_vec, int hd, uint8_t* __restrict__ codes,
                     float* __restrict__ scales) {
    const int lane = threadIdx.x & 31;
    const int v = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (v >= n_vec) return;
    const float s = quant_vec16(q + (size_t)v * hd, hd, codes + (size_t)v * hd, lane);
    if (lane == 0) scales[v] = s;
}

RIVOLI_API int rivoli_index_q_quant(const uint16_t* q, int n_vec, int hd, uint8_t* codes, float* scales,
                                    void* stream) {
    if (n_vec <= 0 || hd <= 0 || !q || !codes || !scales) return 1001;
    if ((hd % 16) != 0 || hd > 512) return 1004;
    if (((uintptr_t)q | (uintptr_t)codes) & 15) return 1005;
    rv_drain_error();
    index_q_quant_kernel<<<(n_vec + 3) / 4, 128, 0, (cudaStream_t)stream>>>(q, n_vec, hd, codes, scales);
    return rv_launch_status();
}
