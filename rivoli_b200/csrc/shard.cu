// Page-range sharded decode step (one long context split over the GPUs of a box): every rank holds a page
// range of every sequence in its own pools at local positions 0 .. n-1, and a layer-step is
//
//   A. local selection (tensor-core scorer + exact cluster selection) and the EXACT scores of the local
//      candidates -> one small buffer per rank;
//   -- all-gather of the candidates (NCCL) --
//   B. the exact global cut, decided identically on every rank from the gathered lists (every token of the
//      global top-k is in its shard's local top-k; ranks are concatenated in ascending token order, so "lower
//      position wins a tie" is "lower global index wins a tie"), this rank's surviving rows, local partial
//      attention -> normalised partial out (bf16) and log-sum-exp per (sequence, head);
//   -- all-gather of the partials (NCCL) --
//   C. merge in ascending rank order, w_g = exp(lse_g - max lse): the reference's split combine
//      (crates/backend/kernels/attn.hip:241-273) across GPUs.
//
// The three phases are entry points of their own (a host with another transport, or a test that emulates the
// ranks on one GPU, calls them around its own exchange); rivoli_shard_step_paged strings them together with two
// ncclAllGather calls on the caller's communicator and stream. NCCL is looked up at run time (dlopen), so the
// library loads on a machine without it and only these entry points then return 1008. Remote data reaches this
// GPU through NCCL into local buffers only.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>

#include "codec.cuh"
#include "common.cuh"
#include "index_rescore.cuh"

extern "C" void rivoli_index_select_query_codes(const DsaGeom* g, int B, int score_stride, void* scratch,
                                                const uint8_t** qcodes, const float** qscales);

namespace {

constexpr int SH_THREADS = 512, SH_WARPS = SH_THREADS / 32, SH_TOK = 4;

size_t up256(size_t x) { return (x + 255) / 256 * 256; }
size_t cand_bytes(const DsaGeom* g, int B) { return up256((size_t)B * g->top_k * 4 + (size_t)B * 4); }
size_t part_bytes(const DsaGeom* g, int B) {
    return up256((size_t)B * g->n_heads * g->kv_lora * 2 + (size_t)B * g->n_heads * 4);
}

// ---- A: exact scores of the local candidates ------------------------------------------------------------------
__global__ void __launch_bounds__(SH_THREADS)
shard_rescore_kernel(DsaGeom g, const uint8_t* __restrict__ qcodes, const float* __restrict__ qscales,
                     const float* __restrict__ w, const uint8_t* __restrict__ index_pool,
                     const float* __restrict__ index_scale, const int32_t* __restrict__ block_table,
                     const uint32_t* __restrict__ rows, const int32_t* __restrict__ n_sel, float* __restrict__ cand) {
    extern __shared__ __align__(16) float sr_smem[];
    uint32_t* qf = reinterpret_cast<uint32_t*>(sr_smem);   // [RS_HD / 4][32] packed q codes
    float* kfw = sr_smem + (RS_HD / 4) * 32;               // [SH_WARPS][SH_TOK][RS_HD]
    const int b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nh = g.index_heads, k = g.top_k;
    const int per_cta = SH_WARPS * SH_TOK * 4;             // candidate slots of one CTA
    const int j0 = blockIdx.x * per_cta;
    const int n = min(max(n_sel[b], 0), k);
    float* out = cand + (size_t)b * k;
    for (int j = j0 + tid; j < min(k, j0 + per_cta); j += SH_THREADS)
        if (j >= n) out[j] = -INFINITY;                    // dead slots never beat a live candidate
    if (j0 >= n) return;
    rv_rescore_stage_q(qcodes + (size_t)b * nh * RS_HD, nh, qf);
    __syncthreads();
    const float my_sq = lane < nh ? qscales[(size_t)b * nh + lane] : 0.0f;
    const float my_wh = lane < nh ? __fmul_rn(w[(size_t)b * nh + lane], g.index_wscale) : 0.0f;
    rv_rescore_listed<SH_WARPS, SH_TOK>(rows + (size_t)b * k + j0, (uint32_t)min(per_cta, n - j0), qf,
                                        kfw + warp * (SH_TOK * RS_HD), block_table + (size_t)b * g.max_pages_per_seq, g,
                                        index_pool, index_scale, my_sq, my_wh,
                                        [&](uint32_t pos, float score) { out[j0 + pos] = score; });
}

// ---- B: the gathered candidates as one score row per sequence, [rank 0 | rank 1 | ...] --------------------------
__global__ void shard_cat_kernel(const uint8_t* __restrict__ all_cand, size_t rank_stride, int world, int B, int k,
                                 float* __restrict__ cat, int32_t* __restrict__ cat_len) {
    const int b = blockIdx.y;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < world * k; i += gridDim.x * blockDim.x) {
        const int gk = i / k, j = i - gk * k;
        const float* sc = reinterpret_cast<const float*>(all_cand + (size_t)gk * rank_stride);
        const int32_t* nn = reinterpret_cast<const int32_t*>(all_cand + (size_t)gk * rank_stride + (size_t)B * k * 4);
        cat[(size_t)b * world * k + i] = j < nn[b] ? sc[(size_t)b * k + j] : -INFINITY;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) cat_len[b] = world * k;
}

// This rank's survivors of the global cut: the selected positions are ascending, this rank's candidates occupy
// [rank * k, (rank + 1) * k), so its survivors are a contiguous run of `sel_pos` and stay in ascending local order.
// Padding (-inf) is picked only when fewer than k live candidates exist and is dropped by its score.
__global__ void __launch_bounds__(1024)
shard_mine_kernel(const float* __restrict__ cat, const uint32_t* __restrict__ sel_pos, const int32_t* __restrict__ n_glob,
                  const uint32_t* __restrict__ rows_l, int rank, int world, int k, uint32_t* __restrict__ rows_att,
                  int32_t* __restrict__ n_mine) {
    __shared__ int s_first, s_count;
    const int b = blockIdx.x;
    if (threadIdx.x == 0) { s_first = 0x7fffffff; s_count = 0; }
    __syncthreads();
    const int n = min(max(n_glob[b], 0), k);
    const uint32_t lo = (uint32_t)rank * k, hi = lo + k;
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
        const uint32_t p = sel_pos[(size_t)b * k + j];
        if (p >= lo && p < hi && cat[(size_t)b * world * k + p] > -INFINITY) { atomicMin(&s_first, j); atomicAdd(&s_count, 1); }
    }
    __syncthreads();
    const int first = s_first, cnt = s_count;
    for (int i = threadIdx.x; i < cnt; i += blockDim.x)
        rows_att[(size_t)b * k + i] = rows_l[(size_t)b * k + (sel_pos[(size_t)b * k + first + i] - lo)];
    if (threadIdx.x == 0) n_mine[b] = cnt;
}

// ---- C: merge of the gathered partials, one warp per (sequence, head) vector ------------------------------------
__global__ void __launch_bounds__(256)
shard_merge_kernel(const uint8_t* __restrict__ all_part, size_t rank_stride, size_t lse_off, int G, int n_vec, int kvl,
                   uint16_t* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int v = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (v >= n_vec) return;
    auto lse = [&](int s) { return reinterpret_cast<const float*>(all_part + (size_t)s * rank_stride + lse_off)[v]; };
    auto po = [&](int s) { return reinterpret_cast<const uint16_t*>(all_part + (size_t)s * rank_stride) + (size_t)v * kvl; };
    float m_g = -INFINITY;
    for (int s = 0; s < G; ++s) m_g = fmaxf(m_g, lse(s));
    float wsum = 0.0f;
    for (int s = 0; s < G; ++s) wsum += isfinite(m_g) ? expf(lse(s) - m_g) : 0.0f;
    const float inv = wsum > 0.0f ? 1.0f / wsum : 0.0f;
    for (int i = lane; i < kvl; i += 32) {
        float sum = 0.0f;
        for (int s = 0; s < G; ++s) {
            const float wgt = isfinite(m_g) ? expf(lse(s) - m_g) : 0.0f;
            sum += rv_bf16_to_f32(po(s)[i]) * wgt;
        }
        out[(size_t)v * kvl + i] = rv_f32_to_bf16(sum * inv);
    }
}

// ---- NCCL, resolved at run time ----------------------------------------------------------------------------------
struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    bool ok = false;
};
NcclApi& nccl() {
    static NcclApi api = [] {
        NcclApi a;
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);   // an already loaded copy (same soname) is reused
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (h) {
            a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
            a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
            a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
            a.AllGather = reinterpret_cast<decltype(a.AllGather)>(dlsym(h, "ncclAllGather"));
            a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllGather;
        }
        return a;
    }();
    return api;
}

struct ShardScratch { float* cat; int32_t* cat_len; uint32_t* sel_pos; int32_t* n_glob; uint8_t* all_cand; uint8_t* all_part; uint8_t* cand; uint8_t* part; };
ShardScratch carve_shard(const DsaGeom* g, int B, int world, void* scratch, size_t* total) {
    uint8_t* p = static_cast<uint8_t*>(scratch);
    size_t off = 0;
    auto take = [&](size_t n) { uint8_t* r = p ? p + off : nullptr; off += up256(n); return r; };
    ShardScratch s;
    s.cat = reinterpret_cast<float*>(take((size_t)B * world * g->top_k * 4));
    s.cat_len = reinterpret_cast<int32_t*>(take((size_t)B * 4));
    s.sel_pos = reinterpret_cast<uint32_t*>(take((size_t)B * g->top_k * 4));
    s.n_glob = reinterpret_cast<int32_t*>(take((size_t)B * 4));
    s.cand = take(cand_bytes(g, B));
    s.part = take(part_bytes(g, B));
    s.all_cand = take((size_t)world * cand_bytes(g, B));
    s.all_part = take((size_t)world * part_bytes(g, B));
    *total = off;
    return s;
}

}  // namespace

RIVOLI_API size_t rivoli_shard_candidate_bytes(const DsaGeom* g, int B) { return (g && B > 0) ? cand_bytes(g, B) : 0; }
RIVOLI_API size_t rivoli_shard_partial_bytes(const DsaGeom* g, int B) { return (g && B > 0) ? part_bytes(g, B) : 0; }
RIVOLI_API size_t rivoli_shard_scratch_bytes(const DsaGeom* g, int B, int world) {
    if (!g || B <= 0 || world <= 0) return 0;
    size_t total = 0;
    carve_shard(g, B, world, nullptr, &total);
    return total;
}

// Phase A. cand (rivoli_shard_candidate_bytes) = [B][top_k] f32 exact scores of rows_l (-inf past n_l[b]) followed
// by n_l i32 [B]. rows_l u32 [B][top_k] receives the local selection (ascending local indices).
RIVOLI_API int rivoli_shard_candidates(const DsaGeom* g, const uint16_t* index_q, const float* w,
                                       const uint8_t* index_pool, const float* index_scale, const int32_t* block_table,
                                       const int32_t* local_len, int B, int score_stride, uint32_t* rows_l,
                                       void* select_scratch, void* cand, void* stream) {
    if (int e = rv_check_geom(g)) return e;
    if (B <= 0 || !cand || !rows_l || !select_scratch) return 1001;
    if (g->index_dim != RS_HD || g->index_heads > 32) return 1004;
    cudaStream_t st = (cudaStream_t)stream;
    float* cs = static_cast<float*>(cand);
    int32_t* n_l = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(cand) + (size_t)B * g->top_k * 4);
    if (int e = rivoli_index_select_paged(g, index_q, w, index_pool, index_scale, block_table, local_len, B, score_stride,
                                          rows_l, n_l, select_scratch, stream))
        return e;
    const uint8_t* qcodes; const float* qscales;
    rivoli_index_select_query_codes(g, B, score_stride, select_scratch, &qcodes, &qscales);
    const size_t smem = ((size_t)(RS_HD / 4) * 32 + (size_t)SH_WARPS * SH_TOK * RS_HD) * 4;
    const int per_cta = SH_WARPS * SH_TOK * 4;
    rv_drain_error();
    cudaFuncSetAttribute(shard_rescore_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    shard_rescore_kernel<<<dim3((g->top_k + per_cta - 1) / per_cta, B), SH_THREADS, smem, st>>>(
        *g, qcodes, qscales, w, index_pool, index_scale, block_table, rows_l, n_l, cs);
    return rv_launch_status();
}

// Phase B. all_cand = `world` candidate buffers, rank-major. part (rivoli_shard_partial_bytes) = this rank's
// normalised partial out bf16 [B][n_heads][kv_lora] followed by lse f32 [B][n_heads]. rows_att / n_mine receive this
// rank's surviving rows (ascending local indices) and their count.
RIVOLI_API int rivoli_shard_cut_attend(const DsaGeom* g, const void* all_cand, int rank, int world,
                                       const uint32_t* rows_l, const uint16_t* q, const uint8_t* latent_pool,
                                       const float* latent_scale, const int32_t* block_table, int B,
                                       uint32_t* rows_att, int32_t* n_mine, void* part, void* shard_scratch,
                                       void* attend_scratch, void* stream) {
    if (int e = rv_check_geom(g)) return e;
    if (B <= 0 || world <= 0 || rank < 0 || rank >= world || !all_cand || !rows_l || !rows_att || !n_mine || !part ||
        !shard_scratch)
        return 1001;
    if ((long long)world * g->top_k > (1ll << 24)) return 1002;   // the cut runs over world * top_k candidates
    cudaStream_t st = (cudaStream_t)stream;
    size_t total = 0;
    ShardScratch s = carve_shard(g, B, world, shard_scratch, &total);
    const int k = g->top_k;
    rv_drain_error();
    shard_cat_kernel<<<dim3((world * k + 255) / 256, B), 256, 0, st>>>(static_cast<const uint8_t*>(all_cand), cand_bytes(g, B),
                                                                        world, B, k, s.cat, s.cat_len);
    if (int e = rv_launch_status()) return e;
    if (int e = rivoli_index_topk_batched(s.cat, world * k, s.cat_len, B, k, s.sel_pos, s.n_glob, stream)) return e;
    shard_mine_kernel<<<B, 1024, 0, st>>>(s.cat, s.sel_pos, s.n_glob, rows_l, rank, world, k, rows_att, n_mine);
    if (int e = rv_launch_status()) return e;
    uint16_t* po = static_cast<uint16_t*>(part);
    float* pl = reinterpret_cast<float*>(static_cast<uint8_t*>(part) + (size_t)B * g->n_heads * g->kv_lora * 2);
    return rivoli_mla_attend_paged_bf16(g, q, latent_pool, latent_scale, block_table, rows_att, k, n_mine, B, po, nullptr,
                                        pl, attend_scratch, stream);
}

// Phase C. all_part = `world` partial buffers, rank-major; out bf16 [B][n_heads][kv_lora], identical on every rank.
RIVOLI_API int rivoli_shard_merge(const DsaGeom* g, const void* all_part, int world, int B, uint16_t* out, void* stream) {
    if (int e = rv_check_geom(g)) return e;
    if (B <= 0 || world <= 0 || world > 64 || !all_part || !out) return 1001;
    const int n_vec = B * g->n_heads;
    rv_drain_error();
    shard_merge_kernel<<<(n_vec + 7) / 8, 256, 0, (cudaStream_t)stream>>>(
        static_cast<const uint8_t*>(all_part), part_bytes(g, B), (size_t)n_vec * g->kv_lora * 2, world, n_vec, g->kv_lora, out);
    return rv_launch_status();
}

// The whole step on the caller's NCCL communicator: A, all-gather, B, all-gather, C. comm may be NULL when
// world == 1 (no exchange). 1008 if NCCL cannot be loaded; an NCCL failure returns 1100 + ncclResult_t.
RIVOLI_API int rivoli_shard_step_paged(const DsaGeom* g, void* comm, int rank, int world, const uint16_t* index_q,
                                       const float* w, const uint16_t* q, const uint8_t* latent_pool,
                                       const float* latent_scale, const uint8_t* index_pool, const float* index_scale,
                                       const int32_t* block_table, const int32_t* local_len, int B, int score_stride,
                                       uint32_t* rows_l, uint32_t* rows_att, int32_t* n_mine, uint16_t* out,
                                       void* select_scratch, void* attend_scratch, void* shard_scratch, void* stream) {
    if (int e = rv_check_geom(g)) return e;
    if (B <= 0 || world <= 0 || !shard_scratch) return 1001;
    if (world > 1 && (!comm || !nccl().ok)) return 1008;
    cudaStream_t st = (cudaStream_t)stream;
    size_t total = 0;
    ShardScratch s = carve_shard(g, B, world, shard_scratch, &total);
    uint8_t* my_cand = world > 1 ? s.cand : s.all_cand;       // with one rank the "gathered" buffer is the rank's own
    uint8_t* my_part = world > 1 ? s.part : s.all_part;
    if (int e = rivoli_shard_candidates(g, index_q, w, index_pool, index_scale, block_table, local_len, B, score_stride,
                                        rows_l, select_scratch, my_cand, stream))
        return e;
    if (world > 1) {
        const ncclResult_t r = nccl().AllGather(my_cand, s.all_cand, cand_bytes(g, B), ncclUint8, (ncclComm_t)comm, st);
        if (r != ncclSuccess) return 1100 + (int)r;
    }
    if (int e = rivoli_shard_cut_attend(g, s.all_cand, rank, world, rows_l, q, latent_pool, latent_scale, block_table, B,
                                        rows_att, n_mine, my_part, shard_scratch, attend_scratch, stream))
        return e;
    if (world > 1) {
        const ncclResult_t r = nccl().AllGather(my_part, s.all_part, part_bytes(g, B), ncclUint8, (ncclComm_t)comm, st);
        if (r != ncclSuccess) return 1100 + (int)r;
    }
    return rivoli_shard_merge(g, s.all_part, world, B, out, stream);
}

// Communicator helpers for hosts that do not hold an ncclComm_t yet: rank 0 makes the 128-byte id, every rank gets
// it by its own means and creates its communicator (collective call: every rank must make it).
RIVOLI_API int rivoli_shard_nccl_unique_id(void* id128) {
    if (!id128) return 1001;
    if (!nccl().ok) return 1008;
    ncclUniqueId id;
    const ncclResult_t r = nccl().GetUniqueId(&id);
    if (r != ncclSuccess) return 1100 + (int)r;
    memcpy(id128, &id, sizeof(id));
    return 0;
}
RIVOLI_API int rivoli_shard_nccl_comm_create(const void* id128, int rank, int world, void** comm) {
    if (!id128 || !comm || world <= 0 || rank < 0 || rank >= world) return 1001;
    if (!nccl().ok) return 1008;
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    ncclComm_t c = nullptr;
    const ncclResult_t r = nccl().CommInitRank(&c, world, id, rank);
    if (r != ncclSuccess) return 1100 + (int)r;
    *comm = c;
    return 0;
}
RIVOLI_API int rivoli_shard_nccl_comm_destroy(void* comm) {
    if (!comm) return 0;
    if (!nccl().ok) return 1008;
    const ncclResult_t r = nccl().CommDestroy((ncclComm_t)comm);
    return r == ncclSuccess ? 0 : 1100 + (int)r;
}
