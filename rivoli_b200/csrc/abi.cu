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

extern "C" bool rivoli_attend_mma_supported(const DsaGeom* g);
extern "C" size_t rivoli_attend_mma_scratch_bytes(const DsaGeom* g, int B);
extern "C" int rivoli_attend_mma_paged_bf16(const DsaGeom* g, const uint16_t* q, const uint8_t* latent_pool,
                                            const float* latent_scale, const int32_t* block_table,
                                            const uint32_t* rows, int row_stride, const int32_t* n_rows, int B,
                                            uint16_t* out, float* out_m, float* out_lse, void* scratch,
                                            int q_early, int min_rows_hint, void* stream);
extern "C" int rivoli_attend_mma_status(void* scratch, void* stream);

RIVOLI_API size_t rivoli_mla_attend_paged_scratch_bytes(const DsaGeom* g, int B) {
    if (!g || B <= 0) return 0;
    const size_t a = rivoli_attend_simt_scratch_bytes(g, B);
    const size_t m = rivoli_attend_mma_supported(g) ? rivoli_attend_mma_scratch_bytes(g, B) : 0;
    return a > m ? a : m;
}

// 1 when rivoli_mla_attend_paged_bf16 runs on the tensor cores for this geometry (given scratch).
RIVOLI_API int rivoli_mla_attend_paged_uses_mma(const DsaGeom* g) {
    return (g && rv_check_geom(g) == 0 && rivoli_attend_mma_supported(g)) ? 1 : 0;
}

// Synchronises `stream`; 1008 if a bounded device-side wait of the last tensor-core attention
// call on this scratch gave up (its output is then undefined), else 0.
RIVOLI_API int rivoli_mla_attend_paged_status(const DsaGeom* g, void* scratch, void* stream) {
    if (!g || !scratch) return 1001;
    if (!rivoli_attend_mma_supported(g)) return 0;
    return rivoli_attend_mma_status(scratch, stream);
}

static cudaEvent_t g_timing_events[5];
static bool g_timing_on = false;
extern "C" cudaEvent_t* rivoli_step_timing_events() { return g_timing_on ? g_timing_events : nullptr; }

// events[0..5): CUDA events (cudaEvent_t) the following decode-step calls record around their kernels: 0 before the
// prologue (append + query preparation), 1 before the scorer, 2 before the selection, 3 before the attention, 4 after
// it. NULL switches the hook off. The records serialise the kernels (no programmatic overlap between them).
RIVOLI_API void rivoli_dsa_step_set_timing_events(void* const* events) {
    g_timing_on = events != nullptr;
    if (events)
        for (int i = 0; i < 5; ++i) g_timing_events[i] = (cudaEvent_t)events[i];
}

static int attend_paged_dispatch(const DsaGeom* g, const uint16_t* q, const uint8_t* latent_pool,
                                 const float* latent_scale, const int32_t* block_table, const uint32_t* rows,
                                 int row_stride, const int32_t* n_rows, int B, uint16_t* out, float* out_m,
                                 float* out_lse, void* scratch, int q_early, int min_rows_hint, void* stream) {
    if (int e = rv_check_geom(g)) return e;
    if (B <= 0 || !q || !latent_pool || !latent_scale || !block_table || !n_rows || !out) return 1001;
    if (rows && row_stride <= 0) return 1001;
    // Tensor-core kernel for the model geometry (64 heads, 512 + 64 dims), given scratch (error word and
    // split partials); inside that call, sequences of fewer than 128 rows go to the CUDA-core kernel.
    // Every other geometry runs on the CUDA-core kernel.
    if (scratch && rivoli_attend_mma_supported(g))
        return rivoli_attend_mma_paged_bf16(g, q, latent_pool, latent_scale, block_table, rows, row_stride, n_rows,
                                            B, out, out_m, out_lse, scratch, q_early, min_rows_hint, stream);
    return rivoli_attend_simt_paged_bf16(g, q, latent_pool, latent_scale, block_table, rows, row_stride,
                                         n_rows, B, out, out_m, out_lse, scratch, stream);
}

RIVOLI_API int rivoli_mla_attend_paged_bf16(const DsaGeom* g, const uint16_t* q, const uint8_t* latent_pool,
                                            const float* latent_scale, const int32_t* block_table,
                                            const uint32_t* rows, int row_stride, const int32_t* n_rows,
                                            int B, uint16_t* out, float* out_m, float* out_lse,
                                            void* scratch, void* stream) {
    // q may have been written by the kernel launched just before this call: the attention kernel reads it
    // only after its dependency wait.
    return attend_paged_dispatch(g, q, latent_pool, latent_scale, block_table, rows, row_stride, n_rows, B, out, out_m,
                                 out_lse, scratch, 0, 0, stream);
}

// One decode layer-step in one call: append the step's token of every sequence, select the attended rows,
// attend over them. q is an input of the CALL, so it is complete before the first kernel of the call starts
// and the attention kernel may convert it while the selection kernel is still running. min_rows_hint: a lower
// bound the caller's scheduler knows for min(top_k, seq_len[b]) over the batch (0 = unknown); from 128 on, the
// launch of the short-context attention arm is left out.
RIVOLI_API int rivoli_dsa_decode_step_paged(const DsaGeom* g, const uint16_t* latent, const uint16_t* index_key,
                                            const int32_t* row_pos, const int32_t* block_table, uint8_t* latent_pool,
                                            float* latent_scale, uint8_t* index_pool, float* index_scale,
                                            int32_t* status, const uint16_t* index_q, const float* w,
                                            const int32_t* seq_len, int B, int score_stride, uint32_t* rows,
                                            int32_t* n_sel, void* select_scratch, const uint16_t* q, uint16_t* out,
                                            float* out_m, float* out_lse, void* attend_scratch, int min_rows_hint,
                                            void* stream) {
    if (!q || !out || !rows || !n_sel || !g) return 1001;
    if (int e = rivoli_dsa_append_select_paged(g, latent, index_key, row_pos, block_table, latent_pool, latent_scale,
                                               index_pool, index_scale, status, index_q, w, seq_len, B, score_stride,
                                               rows, n_sel, select_scratch, stream))
        return e;
    rv_stage_event(3, (cudaStream_t)stream);
    const int e = attend_paged_dispatch(g, q, latent_pool, latent_scale, block_table, rows, g->top_k, n_sel, B, out, out_m,
                                        out_lse, attend_scratch, 1, min_rows_hint, stream);
    rv_stage_event(4, (cudaStream_t)stream);
    return e;
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

// Rows a layer serves under the one-step-stale selection (crates/engine/src/indexer.rs:14-63, batched): per sequence
// mode 0 = the rows stored at the previous token, verbatim; 1 = this token's fresh rows; 2 = dense over the whole
// prefix (first entry = the dense marker 0xFFFFFFFF, which the attention kernels read as "row j = token j").
__global__ void stale_compose_kernel(const uint32_t* __restrict__ prev_rows, const int32_t* __restrict__ prev_n,
                                     const uint32_t* __restrict__ cur_rows, const int32_t* __restrict__ cur_n,
                                     const int32_t* __restrict__ mode, const int32_t* __restrict__ seq_len, int k,
                                     uint32_t* __restrict__ out_rows, int32_t* __restrict__ out_n) {
    const int b = blockIdx.x, m = mode[b];
    const uint32_t* src = m == 0 ? prev_rows + (size_t)b * k : cur_rows + (size_t)b * k;
    const int n = m == 0 ? prev_n[b] : (m == 1 ? cur_n[b] : seq_len[b]);
    for (int j = threadIdx.x; j < k; j += blockDim.x) out_rows[(size_t)b * k + j] = (m == 2 && j == 0) ? 0xffffffffu : src[j];
    if (threadIdx.x == 0) out_n[b] = n;
}

RIVOLI_API int rivoli_stale_compose_rows(const uint32_t* prev_rows, const int32_t* prev_n, const uint32_t* cur_rows,
                                         const int32_t* cur_n, const int32_t* mode, const int32_t* seq_len, int B, int k,
                                         uint32_t* out_rows, int32_t* out_n, void* stream) {
    if (B <= 0 || k <= 0 || !prev_rows || !prev_n || !cur_rows || !cur_n || !mode || !seq_len || !out_rows || !out_n)
        return 1001;
    rv_drain_error();
    stale_compose_kernel<<<B, 256, 0, (cudaStream_t)stream>>>(prev_rows, prev_n, cur_rows, cur_n, mode, seq_len, k, out_rows, out_n);
    return rv_launch_status();
}

RIVOLI_API int rivoli_device_sync(void) {
    cudaError_t e = cudaDeviceSynchronize();
    return e == cudaSuccess ? 0 : -(int)e;
}

RIVOLI_API const char* rivoli_kernels_arch(void) { return "sm_100a"; }
