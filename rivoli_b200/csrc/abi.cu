// Entry points that only dispatch or do small elementwise work: the public paged attention
// (tensor-core kernel where its geometry applies, CUDA-core kernel otherwise), the
// cross-shard partial merge, device sync and the build tag.
#include "codec.cuh"
#include "common.cuh"

extern "C" size_t rivoli_attend_simt_scratch_bytes(const DsaGeom* g, int B);
extern "C" int rivoli_attend_simt_paged_bf16(const DsaGeom* g, const uint16_t* q, const uint8_t* latent_pool,
                                             const float* latent_scale, const int32_t* block_table,
                                             const uint32_t* rows, int row_stride, const int32_t* n_rows,
                                             int B, uint16_t* out, float* out_m, float* out_lse,
                                             void* scratch, void* stream);

RIVOLI_API size_t rivoli_mla_attend_paged_scratch_bytes(const DsaGeom* g, int B) {
    return rivoli_attend_simt_scratch_bytes(g, B);
}

RIVOLI_API int rivoli_mla_attend_paged_bf16(const DsaGeom* g, const uint16_t* q, const uint8_t* latent_pool,
                                            const float* latent_scale, const int32_t* block_table,
                                            const uint32_t* rows, int row_stride, const int32_t* n_rows,
                                            int B, uint16_t* out, float* out_m, float* out_lse,
                                            void* scratch, void* stream) {
    return rivoli_attend_simt_paged_bf16(g, q, latent_pool, latent_scale, block_table, rows, row_stride,
                                         n_rows, B, out, out_m, out_lse, scratch, stream);
}

// out[v] = sum_g w_g * part_out[g][v] / sum_g w_g,  w_g = exp(lse_g - max_g lse), ascending g.
// One warp per vector; lanes stride the columns.
__global__ void __launch_bounds__(256)
merge_partials_kernel(const uint16_t* __restrict__ part_out, const float* __restrict__ part_lse, int G,
                      int n_vec, int kvl, uint16_t* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int v = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (v >= n_vec) return;
    float m_g = -INFINITY;
    for (int s = 0; s < G; ++s) m_g = fmaxf(m_g, part_lse[(size_t)s * n_vec + v]);
    float wsum = 0.0f;
    for (int s = 0; s < G; ++s) wsum += isfinite(m_g) ? expf(part_lse[(size_t)s * n_vec + v] - m_g) : 0.0f;
    const float inv = wsum > 0.0f ? 1.0f / wsum : 0.0f;
    for (int i = lane; i < kvl; i += 32) {
        float sum = 0.0f;
        for (int s = 0; s < G; ++s) {
            const float w = isfinite(m_g) ? expf(part_lse[(size_t)s * n_vec + v] - m_g) : 0.0f;
            sum += rv_bf16_to_f32(part_out[((size_t)s * n_vec + v) * kvl + i]) * w;
        }
        out[(size_t)v * kvl + i] = rv_f32_to_bf16(sum * inv);
    }
}

RIVOLI_API int rivoli_attend_merge_partials(const uint16_t* part_out, const float* part_lse, int G,
                                            int n_vec, int kvl, uint16_t* out, void* stream) {
    if (G <= 0 || n_vec <= 0 || kvl <= 0 || !part_out || !part_lse || !out) return 1001;
    if (G > 64) return 1002;
    rv_drain_error();
    merge_partials_kernel<<<(n_vec + 7) / 8, 256, 0, (cudaStream_t)stream>>>(part_out, part_lse, G, n_vec, kvl, out);
    return rv_launch_status();
}

RIVOLI_API int rivoli_device_sync(void) {
    cudaError_t e = cudaDeviceSynchronize();
    return e == cudaSuccess ? 0 : -(int)e;
}

RIVOLI_API const char* rivoli_kernels_arch(void) { return "sm_100a"; }
