/*
 * C ABI of librivolikernels (CUDA, sm_100a): the decode-time MLA + DSA KV-cache operators.
 *
 * This is the FFI wall the reference's `crates/backend` binds: launch-only entry points
 * `extern "C" int rivoli_<op>(...)` over caller-owned DEVICE pointers. None of them
 * allocates, copies to the host or synchronises unless its comment says so.
 *
 * Return code convention (reference: crates/backend/kernels/mla.hip:7-8,
 * crates/backend/src/hip.rs:328-336):
 *      0           launched
 *      > 0         argument guard, decided on the host BEFORE anything is dereferenced
 *                  1001 argument <= 0 / out of range      1002 size bound
 *                  1003 grouping / power of two           1004 divisibility / unsupported width
 *                  1005 geometry                          1006 shared-memory / scalar range
 *                  1007 page pool exhausted               1008 library state (no device, ...)
 *      < 0         -(cudaError_t) of the launch
 *
 * Part 1 keeps the reference's signatures symbol for symbol (single sequence, f32
 * activations, contiguous slabs, null stream). Part 2 is the batched / paged / bf16
 * surface the reference does not have; every such entry point takes one `const DsaGeom*`
 * and a trailing `void* stream` (a cudaStream_t; NULL = the legacy default stream), the
 * convention of crates/backend/kernels/mla.hip:508-525.
 */
#ifndef RIVOLI_KERNELS_H
#define RIVOLI_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------------------------------
 * Part 1 - reference-compatible symbols
 * ------------------------------------------------------------------------------------- */

/* Replaces crates/backend/kernels/fwd.hip:224-235 (Rust: launch_append_kv,
 * crates/backend/src/hip_attn.rs:130-147). One token: per-128 block absmax scale + e4m3
 * codes into row `pos` of lc8/lscale, roped key as bf16 into row `pos` of rc.
 * Guards: 1001 pos<0 or any size <=0; 1002 kvl not a multiple of 128 in [128,1024] or ropn>kvl. */
int rivoli_append_kv(const float* latent, const float* rope, unsigned char* lc8, float* lscale,
                     unsigned short* rc, int pos, int kvl, int ropn, int n_blocks);

/* Replaces crates/backend/kernels/fwd.hip:237-245 (launch_gather_rope). */
int rivoli_gather_rope(const float* q, float* qrope, int h, int qh, int nope, int ropn);

/* Replaces crates/backend/kernels/indexer.hip:268-276 (launch_index_append,
 * crates/backend/src/hip_attn.rs:445-455): one bf16 indexer key row at `pos`. */
int rivoli_index_append(const float* k, unsigned short* kcache, int pos, int hd);

/* Replaces crates/backend/kernels/indexer.hip:278-295 (launch_index_score,
 * hip_attn.rs:457-476): scores[t] = sum over active heads of w[h]*wscale*ReLU((q_h.k_t)*dscale).
 * heads NULL = all nh heads. Guards: 1001 sizes / nact>nh; 1002 nact>1024 or staging > 64 KiB. */
int rivoli_index_score(const float* q, const float* w, const unsigned short* kcache,
                       const unsigned int* heads, int nt, int nh, int nact, int hd, float wscale,
                       float dscale, float* scores);

/* Replaces crates/backend/kernels/indexer.hip:327-335 (launch_index_topk,
 * hip_attn.rs:478-495): rows[0..min(k,nt)) = the top-k set (score descending, index
 * ascending on ties, -0.0 == +0.0) emitted ASCENDING by index. Writes nothing past
 * min(k,nt). Guards: 1001 nt<=0 or k<=0. */
int rivoli_index_topk(const float* scores, int nt, int k, unsigned int* rows);

/* Replaces crates/backend/kernels/attn.hip:279-308 (launch_attend, hip_attn.rs:101-128):
 * clat[h] = sum_t softmax_t((qabs_h.L_t + qrope_h.R_t)*scale) * L_t over the fp8 latent cache
 * (per-128 block scales) and bf16 roped keys; rows NULL = dense over 0..nr, else the nr
 * listed tokens. partial = scratch of rivoli_mla_attend_scratch_floats() floats, or NULL
 * (single split). Guards: 1001 sizes; 1002 16*(kvl+rope)*4 > 65536 or rope > 128; 1004 kvl>512 or kvl%128.
 * Any H is accepted: one CTA takes as many heads as fit its shared memory (all 64 at the model's width) and
 * larger head counts are tiled over the grid (the reference tiles them in blocks of 16). */
int rivoli_mla_attend(const float* qabs, const float* qrope, const unsigned char* Lc8,
                      const float* Lscale, const unsigned short* Rc, const unsigned int* rows, int H,
                      int nr, int kvl, int rope, int n_blocks, float scale, float* clat,
                      float* partial);

/* rivoli_mla_attend without the caller's `partial` scratch. No counterpart in the reference.
 * For callers that cannot allocate device memory (everything already handed to their own
 * arenas, a thread that must not block on the allocator, a host contract that forbids it):
 * the split partials live in a fixed 2,105,344-byte array inside the library, sized for
 * H <= 64 and kvl <= 512; larger shapes are refused with 1002. Calls nothing that allocates.
 * The first call on a device looks the array's address up (do it before any stream
 * capture). All calls on a device share the array: do not let two of them overlap on the GPU. */
int rivoli_mla_attend_static(const float* qabs, const float* qrope, const unsigned char* Lc8,
                             const float* Lscale, const unsigned short* Rc, const unsigned int* rows, int H,
                             int nr, int kvl, int rope, int n_blocks, float scale, float* clat);

/* Replaces crates/backend/kernels/attn.hip:100-103 (crates/backend/src/hip.rs:425-430). */
size_t rivoli_mla_attend_scratch_floats(int H, int kvl);

/* Replaces crates/backend/kernels/linalg.hip:403 (hip.rs device_sync): blocks until every
 * launched kernel has retired. Returns 0 or -(cudaError_t). */
int rivoli_device_sync(void);

/* ---------------------------------------------------------------------------------------
 * Part 2 - batched, paged, bf16 surface
 *
 * Pool row r = page * page_tokens + slot:
 *   latent_pool  u8  [n_pool_pages * page_tokens][kv_lora + rope_dim]  e4m3 c_kv then k_rope
 *   latent_scale f32 [n_pool_pages * page_tokens]                      absmax over the row / 448 (1 if 0)
 *   index_pool   u8  [n_pool_pages * page_tokens][index_dim]           e4m3 indexer key
 *   index_scale  f32 [n_pool_pages * page_tokens]
 *   block_table  i32 [B][max_pages_per_seq]    page id of logical page j of sequence b
 * Token t of sequence b lives at page block_table[b][t / page_tokens], slot t % page_tokens.
 * ------------------------------------------------------------------------------------- */

/* Geometry of one MLA + DSA decode layer. Plain 32-bit fields, 48 bytes, align 4; the
 * Rust mirror is #[repr(C)] and asserts the same size (cf. CompGeom,
 * crates/backend/src/abi.rs:24-45). */
typedef struct DsaGeom {
    int32_t n_heads;            /* attention query heads (64) */
    int32_t kv_lora;            /* latent width (512); multiple of 128, <= 512 */
    int32_t rope_dim;           /* roped key width (64); multiple of 16 */
    int32_t index_heads;        /* lightning-indexer heads (32) */
    int32_t index_dim;          /* indexer head dim (128); multiple of 16, <= 512 */
    int32_t page_tokens;        /* tokens per page (64); power of two */
    int32_t top_k;              /* rows attended per sequence (2048) */
    int32_t max_pages_per_seq;  /* block_table row pitch */
    int32_t n_pool_pages;       /* pages in the pool (bounds check of block_table entries) */
    float softmax_scale;        /* multiplies q.k before softmax */
    float index_wscale;         /* index_heads^-0.5 */
    float index_dscale;         /* index_dim^-0.5 */
} DsaGeom;

/* Batched form of rivoli_append_kv + rivoli_index_append (fwd.hip:51-71, indexer.hip:54-58)
 * on the paged fp8 pool. Row i (of n_rows) belongs to sequence row_seq[i] (NULL = i) and
 * is written at token position row_pos[i]. latent bf16 [n_rows][kv_lora+rope_dim],
 * index_key bf16 [n_rows][index_dim]. One absmax scale per token for the latent row (c_kv and
 * k_rope share it) and one for the indexer key.
 * Guards: 1001 n_rows<=0 / NULL; 1004/1005 geometry. A block_table entry outside the pool
 * makes the kernel skip that row and raise bit 0 of *status (device i32, may be NULL). */
int rivoli_kv_append_paged(const DsaGeom* g, const uint16_t* latent, const uint16_t* index_key,
                           const int32_t* row_seq, const int32_t* row_pos, int n_rows,
                           const int32_t* block_table, uint8_t* latent_pool, float* latent_scale,
                           uint8_t* index_pool, float* index_scale, int32_t* status, void* stream);

/* Indexer query -> e4m3 codes + one absmax scale per (sequence, head) vector.
 * q bf16 [n_vec][hd]. No reference counterpart (the reference scores f32 q against bf16
 * keys); same codec and scale rule as append. */
int rivoli_index_q_quant(const uint16_t* q, int n_vec, int hd, uint8_t* codes, float* scales,
                         void* stream);

/* Batched, paged form of rivoli_index_score (indexer.hip:60-93): for t < seq_len[b]
 *   cd = left fold over d of qcode[b][h][d]*kcode[t][d];  dot = (cd*s_q[b][h])*s_k[t]
 *   scores[b][t] = fold over h ascending of acc + (w[b][h]*wscale)*max(dot*dscale, 0)
 * in IEEE f32 with that exact order, so it is bit-reproducible. scores f32 [B][score_stride]. */
int rivoli_index_score_paged(const DsaGeom* g, const uint8_t* qcodes, const float* qscales,
                             const float* w, const uint8_t* index_pool, const float* index_scale,
                             const int32_t* block_table, const int32_t* seq_len, int B, float* scores,
                             int score_stride, void* stream);

/* Batched form of rivoli_index_topk (indexer.hip:146-257): rows u32 [B][k], the first
 * n_sel[b] = min(k, seq_len[b]) entries ascending; later entries untouched. */
int rivoli_index_topk_batched(const float* scores, int score_stride, const int32_t* seq_len, int B,
                              int k, uint32_t* rows, int32_t* n_sel, void* stream);

/* Fused indexer: q quantisation + scores + exact top-k in one call, on the tensor cores
 * where the geometry allows (index_dim 128, index_heads <= 32, 16 <= page_tokens <= 128,
 * score_stride <= 131072), otherwise through the three operators above. Replaces the chain
 * launch_index_score -> launch_index_topk (crates/backend/src/hip_attn.rs:457-495) for a
 * batch. The tensor-core scores are approximate; every token within a proven error band
 * of the k-th score is re-scored in the exact order of rivoli_index_score_paged before the
 * final cut, so rows/n_sel are IDENTICAL to rivoli_index_score_paged +
 * rivoli_index_topk_batched. index_q bf16 [B][index_heads][index_dim], w f32
 * [B][index_heads]; rows u32 [B][top_k]; scratch = rivoli_index_select_scratch_bytes(). */
size_t rivoli_index_select_scratch_bytes(const DsaGeom* g, int B, int score_stride);
int rivoli_index_select_uses_mma(const DsaGeom* g, int score_stride);
int rivoli_index_select_paged(const DsaGeom* g, const uint16_t* index_q, const float* w,
                              const uint8_t* index_pool, const float* index_scale,
                              const int32_t* block_table, const int32_t* seq_len, int B,
                              int score_stride, uint32_t* rows, int32_t* n_sel, void* scratch,
                              void* stream);
/* The first half of a decode layer-step in one call: append the step's new token of every
 * sequence (row b of latent / index_key belongs to sequence b at position row_pos[b]) and select
 * the attended rows; the append rides in the launch that prepares the indexer query, one launch
 * fewer than rivoli_kv_append_paged + rivoli_index_select_paged and bit-identical to them.
 * No counterpart in the reference, whose engine issues cache_and_absorb and the indexer launches
 * separately (crates/engine/src/glm/attn.rs:119-222). */
int rivoli_dsa_append_select_paged(const DsaGeom* g, const uint16_t* latent, const uint16_t* index_key,
                                   const int32_t* row_pos, const int32_t* block_table, uint8_t* latent_pool,
                                   float* latent_scale, uint8_t* index_pool, float* index_scale, int32_t* status,
                                   const uint16_t* index_q, const float* w, const int32_t* seq_len, int B,
                                   int score_stride, uint32_t* rows, int32_t* n_sel, void* scratch, void* stream);
/* A whole decode layer-step in one call: rivoli_dsa_append_select_paged followed by
 * rivoli_mla_attend_paged_bf16 over the selected rows (row_stride = top_k), same results. Because q is an
 * input of the call it is known to be complete before the call's first kernel starts, so the attention kernel
 * converts it while the selection kernel is still running (the separate attention entry point cannot assume
 * that and reads q only after the kernel before it has finished). min_rows_hint: a lower bound the caller's
 * scheduler knows for min(top_k, seq_len[b]) over the batch, 0 if it knows none; from 128 on no sequence can need
 * the short-context attention arm and its (otherwise empty) launch is left out. Replaces the per-layer launch
 * sequence of crates/engine/src/glm/attn.rs:119-222 (append, indexer, attend) for a batch. */
int rivoli_dsa_decode_step_paged(const DsaGeom* g, const uint16_t* latent, const uint16_t* index_key,
                                 const int32_t* row_pos, const int32_t* block_table, uint8_t* latent_pool,
                                 float* latent_scale, uint8_t* index_pool, float* index_scale, int32_t* status,
                                 const uint16_t* index_q, const float* w, const int32_t* seq_len, int B,
                                 int score_stride, uint32_t* rows, int32_t* n_sel, void* select_scratch,
                                 const uint16_t* q, uint16_t* out, float* out_m, float* out_lse,
                                 void* attend_scratch, int min_rows_hint, void* stream);
/* ---- the same step for a caller whose activations live in HOST memory ---------------------------------------
 * No counterpart in the reference, whose engine keeps activations on the device; the stream / event wrappers it
 * would build this from are crates/backend/src/gpustream.rs:16-32. A pipe owns `depth` device-side slots, three
 * non-blocking streams (upload | kernels | download) and the events that order them, all allocated in
 * rivoli_step_pipe_create; a step allocates nothing and never blocks the host. One step = ONE host-to-device copy
 * of the packed inputs, rivoli_dsa_decode_step_paged, ONE device-to-host copy of the bf16 output; the upload of
 * step i+1 and the download of step i-1 overlap the kernels of step i.
 * Packed input (pinned host memory, rivoli_step_pipe_input_bytes): latent bf16 [B][kv_lora+rope_dim], index_key
 * bf16 [B][index_dim], index_q bf16 [B][index_heads][index_dim], index_w f32 [B][index_heads], q bf16
 * [B][n_heads][kv_lora+rope_dim], each section starting on a 256-byte boundary (rivoli_step_pipe_input_offsets).
 * host_out: pinned, bf16 [B][n_heads][kv_lora]; it may be reused once rivoli_step_pipe_wait(ticket) returned.
 * row_pos / seq_len are DEVICE arrays (the caller's scheduler state), read when the step runs. */
typedef struct DsaStepState {          /* device pointers of one layer: pools, selection and scratch */
    const int32_t* block_table; uint8_t* latent_pool; float* latent_scale; uint8_t* index_pool; float* index_scale;
    int32_t* status; uint32_t* rows; int32_t* n_sel; void* select_scratch; void* attend_scratch;
    float* out_m; float* out_lse;      /* may be NULL */
    int32_t score_stride;
    int32_t min_rows_hint;             /* see rivoli_dsa_decode_step_paged; 0 = unknown */
} DsaStepState;
size_t rivoli_step_pipe_input_bytes(const DsaGeom* g, int B);
size_t rivoli_step_pipe_output_bytes(const DsaGeom* g, int B);
int rivoli_step_pipe_input_offsets(const DsaGeom* g, int B, size_t off[5]);
void* rivoli_step_pipe_create(const DsaGeom* g, int B, int depth);       /* NULL on failure; depth 1..8 */
void rivoli_step_pipe_destroy(void* pipe);
/* Returns a ticket >= 0, or -(guard code) / -(cudaError_t). */
long long rivoli_dsa_step_host(void* pipe, const DsaStepState* st, const void* host_in, void* host_out,
                               const int32_t* row_pos, const int32_t* seq_len);
int rivoli_step_pipe_wait(void* pipe, long long ticket);
int rivoli_step_pipe_drain(void* pipe);
/* ms[0] upload, ms[1] upload end -> kernels end, ms[2] kernels end -> download end, of the last use of every slot
 * (average over the slots). Synchronises the pipe. */
int rivoli_step_pipe_leg_ms(void* pipe, float ms[3]);
void* rivoli_step_pipe_stream(void* pipe, int which);                    /* 0 upload, 1 kernels, 2 download */

/* Synchronises `stream` and reports on the last rivoli_index_select_paged call (tensor-core path): 1008 if a
 * bounded device-side wait gave up, 1005 if a block-table entry inside a sequence's length pointed outside
 * the pool (that page was not read; results are undefined in both cases), else 0. */
int rivoli_index_select_status(const DsaGeom* g, int B, int score_stride, void* scratch, void* stream);
/* Diagnostics: per-sequence count of tokens the last call re-scored exactly, to HOST memory
 * host_band[B]. Synchronises `stream`. */
int rivoli_index_select_band_stats(const DsaGeom* g, int B, int score_stride, void* scratch,
                                   uint32_t* host_band, void* stream);

/* Bytes of scratch rivoli_mla_attend_paged_bf16 needs for B sequences (an error word and the
 * split partials). Zero its first 256 bytes once after allocation: the error word is sticky (first
 * failure wins) until rivoli_mla_attend_paged_status reads and clears it. */
size_t rivoli_mla_attend_paged_scratch_bytes(const DsaGeom* g, int B);

/* Batched, paged form of rivoli_mla_attend (attn.hip:119-232 + combine :241-273).
 * q bf16 [B][n_heads][kv_lora+rope_dim] (absorbed q then roped q); rows u32 [B][row_stride]
 * or NULL (dense: row j = token j); n_rows i32 [B]. out bf16 [B][n_heads][kv_lora].
 * out_m / out_lse f32 [B][n_heads] (may be NULL): max score and log-sum-exp, the partial a
 * page-range shard hands to rivoli_attend_merge_partials. scratch = the bytes above.
 * A sequence whose first row entry is the dense marker 0xFFFFFFFF is attended as if rows were NULL for it
 * (row j = token j over its first n_rows[b] tokens); this lets one call mix listed and dense sequences.
 * With the model geometry and scratch the call runs the tensor-core kernel for sequences of 128 attended
 * rows and more and the f32 CUDA-core kernel for shorter ones (two launches, disjoint sequences), so the
 * output meets 2e-2 relative / 1e-3 absolute elementwise at every row count. */
int rivoli_mla_attend_paged_bf16(const DsaGeom* g, const uint16_t* q, const uint8_t* latent_pool,
                                 const float* latent_scale, const int32_t* block_table,
                                 const uint32_t* rows, int row_stride, const int32_t* n_rows, int B,
                                 uint16_t* out, float* out_m, float* out_lse, void* scratch,
                                 void* stream);

/* 1 when rivoli_mla_attend_paged_bf16 takes the tensor-core kernel for this geometry
 * (n_heads 64, kv_lora 512, rope_dim 64, scratch given); it then returns in out_m a softmax
 * reference point m <= lse rather than the exact maximum (merging needs only out and lse). */
int rivoli_mla_attend_paged_uses_mma(const DsaGeom* g);
/* The rows a layer serves under the one-step-stale selection (crates/engine/src/indexer.rs:14-63: what token t
 * serves is what token t-1 stored; nothing stored = dense over the whole prefix), batched: per sequence mode 0 =
 * the previous token's rows verbatim, 1 = this token's fresh rows, 2 = dense (out_rows[b][0] = the dense marker,
 * out_n[b] = seq_len[b]). All arrays on the device; rows u32 [B][k]. */
int rivoli_stale_compose_rows(const uint32_t* prev_rows, const int32_t* prev_n, const uint32_t* cur_rows,
                              const int32_t* cur_n, const int32_t* mode, const int32_t* seq_len, int B, int k,
                              uint32_t* out_rows, int32_t* out_n, void* stream);
/* Synchronises `stream`; 1008 if a bounded device-side wait of the last tensor-core
 * attention call on `scratch` gave up (output undefined), else 0. */
int rivoli_mla_attend_paged_status(const DsaGeom* g, void* scratch, void* stream);

/* Merge G shards' normalised partials (attn.hip:241-273 with (m_s, l_s) = (lse_g, 1)):
 * weight_g = exp(lse_g - max lse), ascending g. part_out bf16 [G][n_vec][kvl],
 * part_lse f32 [G][n_vec], out bf16 [n_vec][kvl]. */
int rivoli_attend_merge_partials(const uint16_t* part_out, const float* part_lse, int G, int n_vec,
                                 int kvl, uint16_t* out, void* stream);

/* ---- page-range sharded decode step (one long context split over the GPUs of a box) ----------------------
 * No counterpart in the reference (single GPU); the merge is its split combine (attn.hip:241-273) across GPUs.
 * Every rank holds a page range of every sequence in its OWN pools at local positions 0..n-1 (local_len[b]
 * tokens of sequence b; rank order = ascending token order). The step's new token is appended by the rank that
 * owns the last range (rivoli_kv_append_paged) before the step. Three phases around two exchanges:
 *   A  rivoli_shard_candidates: local selection -> rows_l u32 [B][top_k] (ascending local indices) and the
 *      candidate buffer (rivoli_shard_candidate_bytes): [B][top_k] f32 EXACT scores of rows_l (-inf past n_l[b]),
 *      then n_l i32 [B];
 *   -- all-gather of the candidate buffers, rank-major --
 *   B  rivoli_shard_cut_attend: the exact global top-k over the world * top_k candidates (ties -> lower rank, then
 *      lower local index = lower global index), this rank's surviving rows -> rows_att / n_mine, local partial
 *      attention -> the partial buffer (rivoli_shard_partial_bytes): out bf16 [B][n_heads][kv_lora] normalised
 *      within the shard, then lse f32 [B][n_heads];
 *   -- all-gather of the partial buffers, rank-major --
 *   C  rivoli_shard_merge: weight_g = exp(lse_g - max lse), ascending g -> out bf16 [B][n_heads][kv_lora], the same
 *      on every rank.
 * rivoli_shard_step_paged runs A, ncclAllGather, B, ncclAllGather, C on the caller's communicator (an ncclComm_t
 * passed as void*; NULL allowed when world == 1) and stream: two collectives per step. NCCL is loaded at run time;
 * 1008 if it cannot be, 1100 + ncclResult_t if a collective fails. Needs index_dim 128 and index_heads <= 32
 * (1004 otherwise). shard_scratch = rivoli_shard_scratch_bytes(); select_scratch / attend_scratch as for the
 * single-GPU operators. Remote data reaches a GPU only through NCCL into that scratch. */
size_t rivoli_shard_candidate_bytes(const DsaGeom* g, int B);
size_t rivoli_shard_partial_bytes(const DsaGeom* g, int B);
size_t rivoli_shard_scratch_bytes(const DsaGeom* g, int B, int world);
int rivoli_shard_candidates(const DsaGeom* g, const uint16_t* index_q, const float* w, const uint8_t* index_pool,
                            const float* index_scale, const int32_t* block_table, const int32_t* local_len, int B,
                            int score_stride, uint32_t* rows_l, void* select_scratch, void* cand, void* stream);
int rivoli_shard_cut_attend(const DsaGeom* g, const void* all_cand, int rank, int world, const uint32_t* rows_l,
                            const uint16_t* q, const uint8_t* latent_pool, const float* latent_scale,
                            const int32_t* block_table, int B, uint32_t* rows_att, int32_t* n_mine, void* part,
                            void* shard_scratch, void* attend_scratch, void* stream);
int rivoli_shard_merge(const DsaGeom* g, const void* all_part, int world, int B, uint16_t* out, void* stream);
int rivoli_shard_step_paged(const DsaGeom* g, void* comm, int rank, int world, const uint16_t* index_q,
                            const float* w, const uint16_t* q, const uint8_t* latent_pool, const float* latent_scale,
                            const uint8_t* index_pool, const float* index_scale, const int32_t* block_table,
                            const int32_t* local_len, int B, int score_stride, uint32_t* rows_l, uint32_t* rows_att,
                            int32_t* n_mine, uint16_t* out, void* select_scratch, void* attend_scratch,
                            void* shard_scratch, void* stream);
/* Communicator helpers for a host that holds no ncclComm_t yet: rank 0 makes the 128-byte id, passes it to the
 * other ranks by its own means, and every rank calls comm_create (a collective call). */
int rivoli_shard_nccl_unique_id(void* id128);
int rivoli_shard_nccl_comm_create(const void* id128, int rank, int world, void** comm);
int rivoli_shard_nccl_comm_destroy(void* comm);

/* CUDA-core (f32 accumulate) implementation of rivoli_mla_attend_paged_bf16, same contract.
 * No reference counterpart beyond attn.hip:119-232 itself: it is the cross-check of the
 * tensor-core kernel and serves geometries that kernel does not cover. */
size_t rivoli_attend_simt_scratch_bytes(const DsaGeom* g, int B);
int rivoli_attend_simt_paged_bf16(const DsaGeom* g, const uint16_t* q, const uint8_t* latent_pool,
                                  const float* latent_scale, const int32_t* block_table,
                                  const uint32_t* rows, int row_stride, const int32_t* n_rows, int B,
                                  uint16_t* out, float* out_m, float* out_lse, void* scratch,
                                  void* stream);

/* ---------------------------------------------------------------------------------------
 * Part 3 - host-side page allocator (no device work)
 *
 * The reference keeps contiguous KV slabs (crates/engine/src/glm/engine.rs:77-83) and has
 * no pager; the nearest idiom is its expert arena's LIFO free list
 * (crates/core/src/arena.rs:131-149). alloc pops the tail of the free list, release pushes
 * a sequence's pages logical page 0 first, so page tables are a pure function of the call
 * history. reserve: 0 ok, 1001 bad sequence, 1002 block-table row full, 1007 pool exhausted.
 * ------------------------------------------------------------------------------------- */
void* rivoli_pagepool_create(int n_pages, int n_seqs, int max_pages_per_seq, int page_tokens);
void rivoli_pagepool_destroy(void* pool);
void rivoli_pagepool_shuffle(void* pool, uint64_t seed);
int rivoli_pagepool_reserve(void* pool, int seq, int n_tokens);
int rivoli_pagepool_release(void* pool, int seq);
int rivoli_pagepool_n_free(const void* pool);
int rivoli_pagepool_seq_pages(const void* pool, int seq);
const int32_t* rivoli_pagepool_block_table(const void* pool);   /* [n_seqs][max_pages_per_seq], -1 unmapped */
const int32_t* rivoli_pagepool_free_list(const void* pool);     /* [n_free] */

/* ---- kv_b projections either side of attention (the step after the cache path) ------------------
 * kv_b: e4m3 codes [H*(nope+vh) rows][kvl cols], scale[(row / block) * ceil(kvl / block) + col / block];
 * head h owns rows [h*(nope+vh), +nope) (absorb) and the next vh rows (value).
 * rivoli_mla_absorb_fp8 / rivoli_mla_value_fp8 replace crates/backend/kernels/mla.hip:192-231 (same
 * arguments and guards: 1001 non-positive size, 1003 block not a power of two, 1004 nrow not 1 or 2,
 * value only: 1002 kvl % 4 != 0); outputs are the left folds of the reference's host tests, bit for bit. */
int rivoli_mla_absorb_fp8(const float* q, const unsigned char* kvb, const float* kvb_scale, int H, int qh, int nope,
                          int vh, int kvl, int block, int nrow, float* qabs);
int rivoli_mla_value_fp8(const float* clat, const unsigned char* kvb, const float* kvb_scale, int H, int nope, int vh,
                         int kvl, int block, int nrow, float* ctx);
/* Batched decode form, no counterpart in the reference. q bf16 [B][H][qh] (nope values to absorb, then
 * the rope segment) -> q_abs bf16 [B][H][kvl + rope]: the absorbed query followed by the rope segment
 * bit for bit, i.e. the row rivoli_mla_attend_paged_bf16 consumes (the reference's gather_rope repack,
 * crates/backend/kernels/fwd.hip:73-84, folded in). clat bf16 [B][H][kvl] (the attention output)
 * -> ctx bf16 [B][H][vh]. Tensor-core kernels (tcgen05, bf16 x exact-bf16 codes, f32 accumulate, block
 * scales applied per scale run in the epilogue) for 128-blocks, kvl <= 512, nope <= 256, multiples of
 * 64; CUDA-core kernels otherwise or when force_simt != 0. 1002: qh < nope + rope; 1005: alignment. */
int rivoli_mla_absorb_batched_bf16(const uint16_t* q, const unsigned char* kvb, const float* kvb_scale, int H, int qh,
                                   int nope, int vh, int kvl, int rope, int block, int B, uint16_t* q_abs,
                                   int force_simt, void* stream);
int rivoli_mla_value_batched_bf16(const uint16_t* clat, const unsigned char* kvb, const float* kvb_scale, int H,
                                  int nope, int vh, int kvl, int block, int B, uint16_t* ctx, int force_simt,
                                  void* stream);
/* Synchronises `stream`; 1008 if a bounded wait of a tensor-core projection gave up since the last call. */
int rivoli_kvb_proj_status(void* stream);

/* ---- indexer front end: what produces the indexer's key, queries and head weights ------------------
 * rivoli_gemv_fp8 (+ _splitk), rivoli_layernorm, rivoli_rope_interleave replace
 * crates/backend/kernels/linalg.hip:305-342, indexer.hip:259-266, activation.hip:551-559 (same arguments and
 * guards). y[r][o] = sum_i (e4m3(W[o][i]) * scale[(o/block) * ceil(i_dim/block) + i/block]) * x[r][i] in the
 * fold order of crates/artifact/src/quant/fp8.rs:32-42; layernorm with var = E[x^2] - mean^2; RoPE pairs
 * (2j, 2j+1) -> (j, seg/2 + j) at angle pos * theta^(-2j/seg) computed in f64. */
int rivoli_gemv_fp8(const float* x, const unsigned char* packed, const float* scale, int o_dim, int i_dim, int block,
                    int nrow, float* y);
int rivoli_gemv_fp8_splitk(const float* x, const unsigned char* packed, const float* scale, int o_dim, int i_dim,
                           int block, int nrow, float* y);
int rivoli_layernorm(const float* x, const float* w, const float* b, int n, float eps, float* y);
int rivoli_rope_interleave(float* base, int count, int stride, int seg, int pos, double theta);
/* Batched decode form, no counterpart in the reference: for every sequence b at position pos[b]
 *   index_key[b]   = bf16(rope(layernorm(wk . x[b])))              [index_dim]
 *   index_q[b][h]  = bf16(rope((wq_b . q_resid[b])[h]))            [index_heads][index_dim]
 *   index_w[b]     = weights_proj . x[b]                           [index_heads] f32
 * x bf16 [B][hidden], q_resid bf16 [B][q_lora]; the three weight matrices are e4m3 with block x block
 * scales; the rotation covers [rope_off, rope_off + rope_seg) of every index_dim-wide vector. The outputs
 * are the rows rivoli_kv_append_paged / rivoli_index_select_paged take. scratch =
 * rivoli_index_frontend_scratch_bytes() (split-K partial sums; the split is fixed by the geometry and
 * summed in order, so results are reproducible). The GEMMs run on the tensor cores (tcgen05 kind::f16, weights
 * as bf16(code * scale)) for 128-blocks, contraction lengths multiple of 128 and output counts multiple of 128
 * (or of 16 up to 128); on CUDA cores otherwise or when force_simt != 0. */
typedef struct IndexFrontGeom {
    int32_t hidden, q_lora, index_heads, index_dim, rope_off, rope_seg, block;
    float eps;       /* LayerNorm epsilon (the reference: 1e-6, crates/engine/src/indexer.rs:12) */
    double theta;    /* RoPE base */
} IndexFrontGeom;
size_t rivoli_index_frontend_scratch_bytes(const IndexFrontGeom* g, int B);
int rivoli_index_frontend_bf16(const IndexFrontGeom* g, const uint16_t* x, const uint16_t* q_resid, const int32_t* pos,
                               int B, const unsigned char* wk, const float* wk_scale, const float* knorm_w,
                               const float* knorm_b, const unsigned char* wq_b, const float* wq_b_scale,
                               const unsigned char* wproj, const float* wproj_scale, uint16_t* index_key,
                               uint16_t* index_q, float* index_w, void* scratch, int force_simt, void* stream);
/* Synchronises `stream`; 1008 if a bounded wait of the tensor-core front end gave up since the last call. */
int rivoli_index_frontend_status(void* stream);

/* ---- V4 cousin path: block indexer, scored block selection, MQA sparse attention with a sink --------
 *
 * The first three are the reference's own symbols with identical signatures and guard codes
 * (f32 activations holding bf16 values, one sequence). */

/* crates/backend/kernels/blockindex.hip:263-282 (kernel :97-138). In place on `rows` rows of width d:
 * natural-order Walsh-Hadamard butterfly * 1/sqrt(d), bf16 store, fp4 (e2m1) block-32 quantise-dequantise
 * with a power-of-two scale, bf16 store. Bit-identical to the host rule. 1001 rows/d <= 0, 1002 d > 256,
 * 1003 d not a power of two, 1004 d % 32 != 0. */
int rivoli_act_quant_f4_rotated(float* x, int rows, int d, void* stream);

/* crates/backend/kernels/blockindex.hip:284-306 (kernel :234-261).
 * score[t][c] = bf16( sum_h bf16( relu(bf16(q[t][h] . kv[c])) * w[t][h] ) ); the dot and the head sum are
 * ascending f32 folds with one rounding per operation (no fused multiply-add), so the result is
 * bit-identical to the host fold. 1001 s/heads/hd <= 0, 1005 n_comp <= 0. */
int rivoli_index_score_blocks(const float* q, const float* kv, const float* w, float* score, int s, int n_comp,
                              int heads, int hd, void* stream);

/* crates/backend/kernels/attn.hip:442-465 (kernel :358-440). o[t][head] = softmax over the slots
 * idxs[t][0..topk) (-1 = masked) of q[t][head] . kv[idx] * scale, times kv[idx]; sink[head] joins the
 * softmax DENOMINATOR only (max-shifted). Output rounded to bf16. A query with every slot masked writes
 * NaN. 1001 non-positive sizes, 1002 d > 1024, 1006 (d + topk) floats + reduction scratch over 64 KiB. */
int rivoli_gather_attn_shared_kv(const float* q, const float* kv, const float* sink, const int* idxs, int m, int h,
                                 int d, int topk, float scale, float* o, void* stream);

/* Batched decode form over bf16 storage (no counterpart in the reference, whose V4 engine is one sequence
 * at a time: crates/engine/src/v4/select.rs:78-86). Per sequence b:
 *   kv_cache[b]  bf16 [window + max_comp][head_dim]: ring slots, then the compressed rows in block order;
 *   index_kv[b]  bf16 [max_comp][index_dim]: the indexer's compressed rows (already spread);
 *   pos[b] = position of the query token (already written to the ring); n_comp = (pos+1) / ratio. */
typedef struct V4Geom {
    int32_t n_heads, head_dim, window, index_heads, index_dim, index_topk, ratio, max_comp;
    float softmax_scale;
} V4Geom;

/* Selection rows sel[b][window + index_topk] (crates/engine/src/v4/select.rs:153-232,395-447):
 * the ring in oldest-first order (-1 past the live slots before it fills), then the compressed columns:
 * every closed block in order while n_comp <= index_topk, otherwise the index_topk best by score
 * (total order on f32, ties toward the lower block), ascending, each shifted by `window`; -1 pads the row.
 * index_q bf16 [B][index_heads][index_dim] (already spread), index_w f32 [B][index_heads].
 * scratch = rivoli_v4_select_scratch_bytes(): the score rows f32 [B][max_comp] of the sequences that ranked
 * (readable after the call), then one flag per sequence.
 * Scores are bit-exact. With index_dim == 128 they are computed on the integer tensor cores (four chained
 * mma.m16n8k32.s8 per dot product, exact) for rows of the form the spread produces (integer multiples of a row unit,
 * block scales at most 3 binades apart), for which the host's ordered f32 fold is exact as well; a cached row
 * outside that has its column re-scored by the ordered CUDA-core fold, a query row outside it sends the whole
 * sequence there (force_fold != 0 sends every sequence there; the flag word of a
 * sequence reads 1 for "whole sequence", 2 for "some columns"). Indices are bit-exact. 1001 bad sizes / null scratch,
 * 1002 index_heads > 64 or index_dim > 128 or max_comp > 16384 or index_topk > 4096, 1004 index_dim % 32 != 0. */
size_t rivoli_v4_select_scratch_bytes(const V4Geom* g, int n_seqs);
int rivoli_v4_select_blocks_bf16(const V4Geom* g, int n_seqs, const int32_t* pos, const uint16_t* index_q,
                                 const float* index_w, const uint16_t* index_kv, const unsigned char* packed,
                                 const uint32_t* packed_exp, int32_t* sel, void* scratch, int force_fold, void* stream);

/* Optional second form of the indexer's compressed rows, written ONCE when a row enters the cache, so that the
 * scorer does not convert every row from bf16 on every step: packed int8 [B][max_comp][128] (the row in units of
 * 2^(e - 130), e = the smallest biased exponent any non-empty block's largest magnitude has) and packed_exp u32
 * [B][max_comp] (e; 0 = the row is all zeros; 0xff = the row is not of that form: blocks more than 3 binades apart,
 * a value that is not a multiple of the unit, magnitudes outside 2^-40 .. 2^40). Packs rows
 * [row_begin[b], row_end[b]) of every sequence (row_begin may be null = 0; max_rows = the largest count, sizes the
 * grid). Pass both arrays to rivoli_v4_select_blocks_bf16 (or two nulls); index_kv is still read by the ordered
 * fold. 1001 nulls / sizes, 1002 index_dim != 128. */
int rivoli_v4_index_pack_bf16(const V4Geom* g, int n_seqs, const int32_t* row_begin, const int32_t* row_end,
                              int max_rows, const uint16_t* index_kv, unsigned char* packed, uint32_t* packed_exp,
                              void* stream);

/* out[b][head] bf16 = sparse attention of q[b] bf16 [n_heads][head_dim] over kv_cache[b] rows sel[b][0..cols)
 * with the sink in the denominator. n_heads == 64 and head_dim == 512 run on the tensor cores (one CTA per
 * sequence: the gathered rows are staged once in shared memory and shared by all heads); other shapes on
 * CUDA cores. 1001 bad sizes, 1002 head_dim > 1024, 1006 cols too large for the CUDA-core staging. */
int rivoli_v4_sparse_attend_bf16(const V4Geom* g, int n_seqs, const uint16_t* q, const uint16_t* kv_cache,
                                 const float* sink, const int32_t* sel, int cols, uint16_t* out, int force_simt,
                                 void* stream);

/* ---- V4 KV compressor, decode arm (crates/backend/kernels/kvcompress.hip; struct layouts of
 * crates/backend/src/abi.rs:24-45) -------------------------------------------------------------------- */
typedef struct CompGeom {
    int32_t ratio;   /* positions pooled per block */
    int32_t coff;    /* 1 + overlap */
    int32_t d;       /* this compressor's head_dim */
    int32_t cd;      /* coff * d: width of the projected rows and of ape's rows */
    int32_t ents;    /* coff * ratio: entries in one pooling window */
    int32_t rd;      /* rope_head_dim: only the LAST rd dims of a pooled row are rotated */
    float eps;       /* norm_eps */
} CompGeom;
typedef struct CompFinish {
    const float* norm;   /* [d] RMSNorm gain */
    const float* freqs;  /* [positions][rd]: (cos, sin) pairs */
    float* out;          /* [d] the pooled, normed, rotated row (before the finishing quantisation) */
} CompFinish;

/* crates/backend/kernels/mla.hip:527-550 (kernel :319-338): fp8 (e4m3, round to nearest even) quantise-dequantise
 * of the first n values of each row in blocks of `block`, power-of-two scale, amax floor 1e-4. Bit-identical to
 * the host rule. 1001 sizes, 1002 out of place with a tail, 1004 n % block. */
int rivoli_act_quant_f8_prefix(const float* src, float* dst, int rows, int row_stride, int n, int block, void* stream);
/* kvcompress.hip `rivoli_kv_compress_deposit`: s projected rows [s][cd] (kv, score) into the pooling state
 * [ents][cd]: with overlap the last full block becomes the overlap half; the s % ratio rows of the open block
 * land from slot0 on; score rows get ape added. 1000 null geometry, 1001-1004/1010 geometry, 1005 s <= 0, 1008 slot0. */
int rivoli_kv_compress_deposit(const float* kv, const float* score, const float* ape, float* kv_state,
                               float* score_state, const CompGeom* p, int s, int slot0, void* stream);
/* kvcompress.hip `rivoli_kv_compress_prefill`: blocks 0 .. nblk-1 of a prompt that starts at position 0, from its
 * projected rows kv, score [s][cd]: each block pooled over its own rows and (with overlap) the previous block's,
 * finished at position b * ratio -> f->out[b][d]. 1006 nblk <= 0. Same tolerance as the decode arm. */
int rivoli_kv_compress_prefill(const float* kv, const float* score, const float* ape, const CompFinish* f,
                               const CompGeom* p, int nblk, void* stream);
/* kvcompress.hip `rivoli_kv_compress_decode`: pool the state (softmax over the entry axis per feature), bf16 store,
 * RMSNorm, rotate the last rd dims at the block's first position, bf16 store -> f->out; then the overlap half of the
 * state moves down. 1007 start_pos <= 0, 1009 (start_pos + 1) % ratio != 0. Tolerance: expf and the norm's
 * reduction order differ from the host's by rounding. */
int rivoli_kv_compress_decode(float* kv_state, float* score_state, const CompFinish* f, const CompGeom* p,
                              int start_pos, void* stream);
/* Batched decode step (no counterpart in the reference: crates/engine/src/v4/kvcompress.rs drives one sequence):
 * per sequence b, deposit the token's projected rows kv_proj[b], score_proj[b] ([cd] f32) at slot pos[b] % ratio of
 * its state ([B][ents][cd] f32); if the block closes, pool + norm + rotate as above, finish with the spread
 * (rotate != 0: the indexer's compressor, blockindex.hip:97-138) or the fp8 block-64 quantisation of the d - rd
 * un-rotated dims (the attention compressor, crates/oracles/src/v4oracle/compress.rs:235-247), and store the row as
 * bf16 at cache[(b * cache_rows + cache_row0 + pos[b] / ratio) * d]. prequant (optional) receives the row before
 * the finishing quantisation, [B][d] f32. packed / packed_exp (optional, both or neither; rotate != 0 and d == 128)
 * receive the same row in the scorer's int8 + block-exponent form (see rivoli_v4_index_pack_bf16), at row
 * b * cache_rows + cache_row0 + pos[b] / ratio of those arrays. */
int rivoli_v4_compress_step_bf16(const CompGeom* p, int n_seqs, const int32_t* pos, const float* kv_proj,
                                 const float* score_proj, const float* ape, float* kv_state, float* score_state,
                                 const float* norm, const float* freqs, int rotate, uint16_t* cache, int cache_rows,
                                 int cache_row0, float* prequant, unsigned char* packed, uint32_t* packed_exp,
                                 void* stream);

/* ---- measurement hook ------------------------------------------------------------------------------------------
 * events[0..5): cudaEvent_t handles that the following rivoli_dsa_decode_step_paged / rivoli_dsa_append_select_paged
 * calls record on their stream: 0 before the prologue kernel (append + query preparation), 1 before the scorer,
 * 2 before the selection, 3 before the attention, 4 after it; a benchmark reads each kernel's own duration from
 * them. The records take away the programmatic overlap between the kernels. NULL switches the hook off (the
 * default). No counterpart in the reference. */
void rivoli_dsa_step_set_timing_events(void* const* events);

/* ---- test hooks (exercised by the GPU tests; not for production callers) ----------------------------------
 * Overrides for the tensor-core attention's NEXT launches, host side only, no counterpart in the reference.
 * min_rows >= 0 replaces the 128-row threshold below which a sequence goes to the CUDA-core kernel (0 = every
 * sequence on the tensor cores; -1 restores the default). withhold != 0: the next launch leaves out one barrier
 * arrival, so its bounded waits run out: the launch still returns, rivoli_mla_attend_paged_status reports 1008
 * and later launches are unaffected (this is how the give-up path of the waits is tested; nothing faults).
 * max_polls > 0 sets the poll limit of the bounded waits (<= 0 restores the default). */
void rivoli_attend_mma_test_hook(int min_rows, int withhold, int max_polls);
/* Forces the thread-block cluster size of the following selection launches (1, 2, 4 or 8; anything else restores
 * the library's own plan), so that a test can run every cluster size at any batch size. */
void rivoli_index_select_test_cluster(int cluster);

/* Library build tag, e.g. "sm_100a". */
const char* rivoli_kernels_arch(void);

#ifdef __cplusplus
}
#endif
#endif /* RIVOLI_KERNELS_H */
