// Lightning-indexer selection on the tensor cores, with an exactness guarantee.
//
// The indexer reads 132 bytes per cached token and spends 8192 FLOP on them (~62 FLOP/B),
// so only tensor cores keep it HBM-bound. But an MMA does not accumulate in the fixed
// order the reference's score is defined in, so its scores can differ from the exact ones
// in the last bits, which would move top-k indices at the cut. This file therefore does:
//
//   1. index_q_prepare_kernel   q -> e4m3 codes + per-head scale (bit-exact codec), plus one
//                               error-bound constant per sequence. On the fused decode path
//                               (rivoli_dsa_append_select_paged) the same work runs in
//                               step_prologue_kernel, whose extra blocks append the step's tokens.
//   2. index_score_mma_kernel   approximate scores a_t for every cached token: fp8 keys are
//                               streamed page by page by TMA (one 2-D box per page) into swizzled
//                               shared memory and consumed by tcgen05.mma kind::f8f6f4
//                               (tokens = M 128, heads = N 32, dims = K 128), accumulators
//                               in TMEM, scale/ReLU/head-weight epilogue from TMEM.
//   3. index_select_cluster_kernel (index_select.cu)  per sequence, one thread-block cluster: locate
//                               the bin of the k-th approximate score A_k with one histogram pass;
//                               every token within 2*eps of that bin is re-scored in
//                               the exact order (sequential f32 fold, identical to
//                               rivoli_index_score_paged); tokens above the band are in,
//                               below are out; the final exact top-k (ties -> lower index)
//                               is emitted ascending.
//
// Why this yields the exact top-k set: with |a_t - o_t| <= eps for the exact scores o_t,
// the k-th largest values satisfy |A_k - E_k| <= eps, so a_t > A_k + 2 eps implies
// o_t > E_k (selected) and a_t < A_k - 2 eps implies o_t < E_k (not selected); everything
// else is decided on exact scores. eps per sequence = max key scale * sum_h |w_h ws| ds
// s_q[h] ||qcode_h||_2 * sqrt(hd) * 448 * 2^-16: a Cauchy-Schwarz bound on sum |q_d k_d|
// times 2^-16 relative error. The sequential fold's own worst case is hd * 2^-24 = 2^-17
// of sum |q_d k_d|; the tensor core measured 2^-21.9 on full-range random codes.
#include "codec.cuh"
#include "common.cuh"
#include "quant.cuh"
#include "tc_common.cuh"
#include "index_select.hpp"
#include "tmap.hpp"

namespace {

constexpr int IM_TILE = 128;       // tokens per MMA tile (M)
constexpr int IM_HD = 128;         // index dim = one 128-byte swizzle row
constexpr int IM_NPAD = 32;        // heads padded to N = 32
constexpr int IM_NS = 6;           // key-tile stages in flight
constexpr int IM_NACC = 4;         // TMEM accumulators (32 columns each)
constexpr int IM_TPI = 16;         // most tiles per work item (a launch picks fewer when the batch is small: IndexMmaArgs::tpi)
constexpr int IM_THREADS = 192;    // warps 0-3 epilogue, 4 producer, 5 MMA
constexpr int IM_STAGE_BYTES = IM_TILE * IM_HD;   // 16 KiB
constexpr int IM_Q_BYTES = IM_NPAD * IM_HD;       // 4 KiB
constexpr float IM_EPS_REL = 1.52587890625e-05f;  // 2^-16
constexpr int IM_ERR_BAD_PAGE = 1005;             // error word: a block-table entry inside seq_len lies outside the pool

struct IndexMmaArgs {
    DsaGeom g;
    const uint8_t* qcodes; const float* qscales; const float* w;
    const uint8_t* index_pool; const float* index_scale; const int32_t* block_table; const int32_t* seq_len;
    float* scores; int score_stride; int B;
    int* err;              // device error word (0 = ok)
    int tpi;               // tiles per work item, 1 .. IM_TPI: small enough that every persistent CTA gets work
};

// ---------------------------------------------------------------------------------------------
// 1. q quantisation + per-sequence error-bound constant. One CTA per sequence, one warp per head.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void
index_q_prepare_block(int b, const uint16_t* __restrict__ q, const float* __restrict__ w, int nh, int hd, float wscale,
                      float dscale, uint8_t* __restrict__ codes, float* __restrict__ scales, float* __restrict__ cb,
                      int* __restrict__ err, float* term) {
    const int h = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (h < nh) {
        const size_t v = (size_t)b * nh + h;
        // same codec path as rivoli_index_q_quant: 16 values per lane, absmax scale, e4m3 codes
        float f[16];
        const bool act = lane * 16 < hd;
        if (act) {
            const uint4* p = reinterpret_cast<const uint4*>(q + v * hd + lane * 16);
            const uint4 p0 = p[0], p1 = p[1];
            const uint32_t ww[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) { f[2 * i] = __uint_as_float(ww[i] << 16); f[2 * i + 1] = __uint_as_float(ww[i] & 0xffff0000u); }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) f[i] = 0.0f;
        }
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
        amax = rv_warp_max(amax);
        const float scl = rv_scale_from_amax(amax);
        float n2 = 0.0f;
        if (act) {
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint16_t lo = rv_f32x2_to_e4m3x2(__fdiv_rn(f[4 * i], scl), __fdiv_rn(f[4 * i + 1], scl));
                const uint16_t hi = rv_f32x2_to_e4m3x2(__fdiv_rn(f[4 * i + 2], scl), __fdiv_rn(f[4 * i + 3], scl));
                o[i] = (uint32_t)lo | ((uint32_t)hi << 16);
                const float2 a = rv_e4m3x2_to_f32x2(lo), c = rv_e4m3x2_to_f32x2(hi);
                n2 += a.x * a.x + a.y * a.y + c.x * c.x + c.y * c.y;
            }
            *reinterpret_cast<uint4*>(codes + v * hd + lane * 16) = make_uint4(o[0], o[1], o[2], o[3]);
        }
        n2 = rv_warp_sum(n2);
        if (lane == 0) {
            scales[v] = scl;
            term[h] = fabsf(w[v] * wscale) * dscale * scl * sqrtf(n2);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        for (int i = 0; i < nh; ++i) s += term[i];
        // ||kcode||_2 <= sqrt(hd) * 448; 1.01 covers the roundings of this very sum
        cb[b] = s * sqrtf((float)hd) * 448.0f * IM_EPS_REL * 1.01f;
        if (b == 0) *err = 0;   // the scorer's error word starts clean on every call
    }
}

__global__ void __launch_bounds__(1024)
index_q_prepare_kernel(const uint16_t* __restrict__ q, const float* __restrict__ w, int nh, int hd, float wscale,
                       float dscale, uint8_t* __restrict__ codes, float* __restrict__ scales, float* __restrict__ cb,
                       int* __restrict__ err) {
    __shared__ float term[32];
    rv_grid_dep_trigger();   // the scorer may set itself up while this runs; it waits before reading these outputs
    index_q_prepare_block(blockIdx.x, q, w, nh, hd, wscale, dscale, codes, scales, cb, err, term);
}

// Decode-step prologue in one launch: blocks [0, B) prepare the indexer query of sequence b,
// blocks [B, B + ceil(B/32)) append the step's new token of 32 sequences each (one warp per row).
// The two halves touch disjoint memory.
struct AppendArgs {
    const uint16_t* latent; const uint16_t* index_key; const int32_t* row_pos; const int32_t* block_table;
    uint8_t* latent_pool; float* latent_scale; uint8_t* index_pool; float* index_scale; int32_t* status;
};

__global__ void __launch_bounds__(1024)
step_prologue_kernel(DsaGeom g, AppendArgs ap, int B, const uint16_t* __restrict__ q, const float* __restrict__ w,
                     uint8_t* __restrict__ codes, float* __restrict__ scales, float* __restrict__ cb,
                     int* __restrict__ err) {
    __shared__ float term[32];
    rv_grid_dep_trigger();   // the scorer may set itself up while this runs; it waits before reading these outputs
    if ((int)blockIdx.x < B) {
        index_q_prepare_block(blockIdx.x, q, w, g.index_heads, g.index_dim, g.index_wscale, g.index_dscale, codes, scales,
                              cb, err, term);
        return;
    }
    const int row = ((int)blockIdx.x - B) * 32 + (threadIdx.x >> 5);
    if (row >= B) return;
    append_row_paged(g, ap.latent, ap.index_key, row, row, ap.row_pos[row], ap.block_table, ap.latent_pool,
                     ap.latent_scale, ap.index_pool, ap.index_scale, ap.status, threadIdx.x & 31);
}

// ---------------------------------------------------------------------------------------------
// 2. approximate scores on the tensor cores (persistent CTAs, warp specialised)
// ---------------------------------------------------------------------------------------------
struct ImBarriers {
    uint64_t full[IM_NS], empty[IM_NS], tfull[IM_NACC], tempty[IM_NACC], qfree[2];
};

__global__ void __launch_bounds__(IM_THREADS)
index_score_mma_kernel(IndexMmaArgs A, const __grid_constant__ CUtensorMap tm_keys,
                       const __grid_constant__ CUtensorMap tm_q) {
    extern __shared__ __align__(1024) uint8_t im_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(im_smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* s_keys = smem;                                   // IM_NS x 16 KiB
    uint8_t* s_q = smem + IM_NS * IM_STAGE_BYTES;             // 2 x 4 KiB
    __shared__ ImBarriers bars;
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_flag;
    __shared__ float s_wh[IM_NPAD];
    __shared__ int s_pg[IM_TPI * (IM_TILE / 16)];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const DsaGeom& g = A.g;
    const int nh = g.index_heads, P = g.page_tokens;

    if (tid == 0) {
        for (int i = 0; i < IM_NS; ++i) { tc::mbar_init(&bars.full[i], 1); tc::mbar_init(&bars.empty[i], 1); }
        for (int i = 0; i < IM_NACC; ++i) { tc::mbar_init(&bars.tfull[i], 1); tc::mbar_init(&bars.tempty[i], 4); }
        tc::mbar_init(&bars.qfree[0], 1); tc::mbar_init(&bars.qfree[1], 1);
        tc::mbar_init_fence();
        abort_flag = 0;
    }
    // q tiles start zeroed: rows >= nh are never loaded and must contribute exact zeros
    for (int i = tid; i < 2 * IM_Q_BYTES / 16; i += IM_THREADS) reinterpret_cast<uint4*>(s_q)[i] = make_uint4(0, 0, 0, 0);
    if (warp == 5) tc::tmem_alloc<IM_NACC * 32>(&tmem_base_s);
    tc::fence_proxy_async();
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    rv_grid_dep_trigger();   // the selection kernel may be scheduled; it waits for this grid before reading scores
    rv_grid_dep_wait();      // query codes, head scales and this step's appended keys come from the kernel before

    const int tpi = A.tpi;
    const int max_tiles = (A.score_stride + IM_TILE - 1) / IM_TILE;
    const int chunks = (max_tiles + tpi - 1) / tpi;
    const int n_items = A.B * chunks;

    if (warp == 4) {
        // ------------------------------ producer: TMA page loads ----------------------------------
        // A page is P rows x 128 bytes, contiguous in the pool; one 2-D TMA box per page lands it in
        // shared memory already in the 128-byte-swizzled K-major form the MMA consumes. The whole
        // warp fetches an item's page ids once; lane 0 then issues one instruction per page.
        int it = 0, items_done = 0;
        bool ok = true;
        const int ppt = IM_TILE / P;  // pages per tile (16 <= P <= 128)
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int b = item / chunks, c = item - b * chunks;
            const int nt = min(A.seq_len[b], A.score_stride);
            const int tile_end = min((c + 1) * tpi, (nt + IM_TILE - 1) / IM_TILE);
            if (c * tpi >= tile_end) continue;
            const int first_lp = c * tpi * ppt;
            __syncwarp();
            for (int j = lane; j < tpi * ppt; j += 32) {
                const int lp = first_lp + j;
                int pg = -1;
                const bool live = lp < g.max_pages_per_seq && lp * P < nt;
                if (live) pg = A.block_table[(size_t)b * g.max_pages_per_seq + lp];
                const bool bad = pg < 0 || pg >= g.n_pool_pages;
                // A page inside the sequence that the table does not map into the pool is never loaded (its
                // tokens get scores of whatever the stage held) and the call is flagged, as the append does.
                if (live && bad) atomicCAS(A.err, 0, IM_ERR_BAD_PAGE);
                s_pg[j] = bad ? -1 : pg;
            }
            __syncwarp();
            const int qb = items_done & 1;
            for (int tile = c * tpi; tile < tile_end && ok; ++tile) {
                const int s = it % IM_NS;
                ok = tc::mbar_wait_warp(&bars.empty[s], ((it / IM_NS) & 1) ^ 1, &abort_flag, 11);
                if (!ok) break;
                const bool first = tile == c * tpi;
                if (first) {
                    ok = tc::mbar_wait_warp(&bars.qfree[qb], ((items_done >> 1) & 1) ^ 1, &abort_flag, 12);
                    if (!ok) break;
                }
                if (lane == 0) {
                    const int pbase = (tile - c * tpi) * ppt;
                    uint32_t bytes = first ? (uint32_t)nh * IM_HD : 0u;
                    for (int p2 = 0; p2 < ppt; ++p2) bytes += s_pg[pbase + p2] >= 0 ? (uint32_t)P * IM_HD : 0u;
                    tc::mbar_arrive_expect_tx(&bars.full[s], bytes);
                    if (first)  // this sequence's q codes ride the first tile's barrier
                        tc::tma_load_2d(tc::smem_u32(s_q + qb * IM_Q_BYTES), &tm_q, 0, b * nh, &bars.full[s]);
                    for (int p2 = 0; p2 < ppt; ++p2) {
                        const int pg = s_pg[pbase + p2];
                        if (pg >= 0)
                            tc::tma_load_2d(tc::smem_u32(s_keys + s * IM_STAGE_BYTES + p2 * P * IM_HD), &tm_keys, 0,
                                            pg * P, &bars.full[s]);
                    }
                }
                __syncwarp();
                ++it;
            }
            ++items_done;
        }
    } else if (warp == 5) {
        // ------------------------------ MMA issuer ------------------------------------------------
        int it = 0, items_done = 0;
        bool ok = true;
        const uint32_t idesc = tc::idesc_e4m3(IM_TILE, IM_NPAD, 0, 0);
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int b = item / chunks, c = item - b * chunks;
            const int nt = min(A.seq_len[b], A.score_stride);
            const int tile_end = min((c + 1) * tpi, (nt + IM_TILE - 1) / IM_TILE);
            const int qb = items_done & 1;
            for (int tile = c * tpi; tile < tile_end && ok; ++tile) {
                const int s = it % IM_NS, a = it % IM_NACC;
                ok = tc::mbar_wait_warp(&bars.full[s], (it / IM_NS) & 1, &abort_flag, 21) &&
                     tc::mbar_wait_warp(&bars.tempty[a], ((it / IM_NACC) & 1) ^ 1, &abort_flag, 22);
                if (!ok) break;
                tc::tc_fence_after();
                if (lane == 0) {
                    const uint32_t ka = tc::smem_u32(s_keys + s * IM_STAGE_BYTES), qa = tc::smem_u32(s_q + qb * IM_Q_BYTES);
#pragma unroll
                    for (int k = 0; k < IM_HD / 32; ++k)
                        tc::mma_f8(tmem + a * 32, tc::smem_desc_sw128(ka + k * 32, 16, 1024),
                                   tc::smem_desc_sw128(qa + k * 32, 16, 1024), idesc, k > 0);
                    tc::mma_commit(&bars.empty[s]);
                    tc::mma_commit(&bars.tfull[a]);
                    if (tile == tile_end - 1) tc::mma_commit(&bars.qfree[qb]);
                }
                __syncwarp();
                ++it;
            }
            if (c * tpi < tile_end) ++items_done;      // items without tiles never touched a q buffer
        }
    } else {
        // ------------------------------ epilogue: TMEM -> scores --------------------------------
        int it = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int b = item / chunks, c = item - b * chunks;
            const int nt = min(A.seq_len[b], A.score_stride);
            const int tile_end = min((c + 1) * tpi, (nt + IM_TILE - 1) / IM_TILE);
            if (c * tpi >= tile_end) continue;
            tc::named_barrier(1, 128);  // previous item's constants are no longer read
            if (tid < IM_NPAD) {
                // a_t / s_k = sum_h (w_h ws s_q[h] ds) * max(cd_h, 0): the exact formula up to a few
                // roundings (s_q, s_k, ds > 0 commute with the ReLU); the band covers them
                s_wh[tid] = tid < nh ? A.w[(size_t)b * nh + tid] * g.index_wscale * A.qscales[(size_t)b * nh + tid] *
                                           g.index_dscale : 0.0f;
            }
            tc::named_barrier(1, 128);
            for (int tile = c * tpi; tile < tile_end && ok; ++tile) {
                const int a = it % IM_NACC;
                const int t = tile * IM_TILE + tid;
                ok = tc::mbar_wait_warp(&bars.tfull[a], (it / IM_NACC) & 1, &abort_flag, 31);
                if (!ok) break;
                tc::tc_fence_after();
                uint32_t r[32];
                tc::tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + a * 32, r);
                tc::tmem_ld_wait();
                tc::tc_fence_before();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&bars.tempty[a]);
                if (t < nt) {
                    float acc = 0.0f;
#pragma unroll
                    for (int h = 0; h < IM_NPAD; ++h) acc = fmaf(s_wh[h], fmaxf(__uint_as_float(r[h]), 0.0f), acc);
                    A.scores[(size_t)b * A.score_stride + t] = acc;   // the key scale s_k[t] is applied by the selector
                }
                ++it;
            }
        }
    }

    tc::tc_fence_before();
    __syncthreads();
    if (warp == 5) tc::tmem_dealloc<IM_NACC * 32>(tmem);
    if (tid == 0 && abort_flag) atomicCAS(A.err, 0, abort_flag);
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct SelectScratch {
    uint8_t* qcodes; float* qscales; float* cb; int* err; unsigned int* stats; float* scores;
};

SelectScratch carve(const DsaGeom* g, int B, int score_stride, void* scratch, size_t* total) {
    uint8_t* p = static_cast<uint8_t*>(scratch);
    size_t off = 0;
    SelectScratch s;
    auto take = [&](size_t n) { uint8_t* r = p ? p + off : nullptr; off += align_up(n, 256); return r; };
    s.qcodes = take((size_t)B * g->index_heads * g->index_dim);
    s.qscales = reinterpret_cast<float*>(take((size_t)B * g->index_heads * 4));
    s.cb = reinterpret_cast<float*>(take((size_t)B * 4));
    s.err = reinterpret_cast<int*>(take(4));
    s.stats = reinterpret_cast<unsigned int*>(take((size_t)B * 8));
    s.scores = reinterpret_cast<float*>(take((size_t)B * score_stride * 4));
    *total = off;
    return s;
}

constexpr int SEL_MAX_NT = 8 * 512 * 32;   // what one cluster of the selection kernel covers

bool mma_geometry_ok(const DsaGeom* g, int score_stride) {
    return g->index_dim == IM_HD && g->index_heads <= IM_NPAD && g->page_tokens >= 16 && g->page_tokens <= IM_TILE &&
           score_stride <= SEL_MAX_NT;
}

}  // namespace

RIVOLI_API size_t rivoli_index_select_scratch_bytes(const DsaGeom* g, int B, int score_stride) {
    if (!g || B <= 0 || score_stride <= 0) return 0;
    size_t total = 0;
    carve(g, B, score_stride, nullptr, &total);
    return total;
}

// 1 if rivoli_index_select_paged takes the tensor-core path for this geometry, else 0.
RIVOLI_API int rivoli_index_select_uses_mma(const DsaGeom* g, int score_stride) {
    return (g && mma_geometry_ok(g, score_stride)) ? 1 : 0;
}

RIVOLI_API int rivoli_kv_append_paged(const DsaGeom* g, const uint16_t* latent, const uint16_t* index_key,
                                      const int32_t* row_seq, const int32_t* row_pos, int n_rows,
                                      const int32_t* block_table, uint8_t* latent_pool, float* latent_scale,
                                      uint8_t* index_pool, float* index_scale, int32_t* status, void* stream);

// `ap` != NULL: the step's append (one new token per sequence) rides in the same launch as the
// query preparation.
static int select_impl(const DsaGeom* g, const AppendArgs* ap, const uint16_t* index_q, const float* w,
                       const uint8_t* index_pool, const float* index_scale,
                       const int32_t* block_table, const int32_t* seq_len, int B,
                       int score_stride, uint32_t* rows, int32_t* n_sel, void* scratch,
                       void* stream) {
    if (int e = rv_check_geom(g)) return e;
    if (B <= 0 || score_stride <= 0 || !index_q || !w || !index_pool || !index_scale || !block_table || !seq_len ||
        !rows || !n_sel || !scratch)
        return 1001;
    if ((((uintptr_t)index_pool | (uintptr_t)index_q | (uintptr_t)scratch) & 15)) return 1005;
    if ((long long)score_stride > (long long)g->max_pages_per_seq * g->page_tokens) return 1002;
    cudaStream_t st = (cudaStream_t)stream;
    size_t total = 0;
    SelectScratch s = carve(g, B, score_stride, scratch, &total);
    const int nh = g->index_heads, hd = g->index_dim;

    if (!mma_geometry_ok(g, score_stride)) {
        // geometries outside the tensor-core kernel: the exact CUDA-core scorer + exact top-k
        if (ap)
            if (int e = rivoli_kv_append_paged(g, ap->latent, ap->index_key, nullptr, ap->row_pos, B, ap->block_table,
                                               ap->latent_pool, ap->latent_scale, ap->index_pool, ap->index_scale,
                                               ap->status, stream))
                return e;
        int e = rivoli_index_q_quant(index_q, B * nh, hd, s.qcodes, s.qscales, stream);
        if (e) return e;
        e = rivoli_index_score_paged(g, s.qcodes, s.qscales, w, index_pool, index_scale, block_table, seq_len, B,
                                     s.scores, score_stride, stream);
        if (e) return e;
        return rivoli_index_topk_batched(s.scores, score_stride, seq_len, B, g->top_k, rows, n_sel, stream);
    }

    rv_drain_error();
    rv_stage_event(0, st);
    if (ap)
        step_prologue_kernel<<<B + (B + 31) / 32, 1024, 0, st>>>(*g, *ap, B, index_q, w, s.qcodes, s.qscales, s.cb,
                                                                 s.err);
    else
        index_q_prepare_kernel<<<B, 32 * nh, 0, st>>>(index_q, w, nh, hd, g->index_wscale, g->index_dscale, s.qcodes,
                                                       s.qscales, s.cb, s.err);
    if (int e = rv_launch_status()) return e;

    IndexMmaArgs ma{*g, s.qcodes, s.qscales, w, index_pool, index_scale, block_table, seq_len,
                    s.scores, score_stride, B, s.err, IM_TPI};
    const size_t smem1 = (size_t)IM_NS * IM_STAGE_BYTES + 2 * IM_Q_BYTES + 1024;
    cudaFuncSetAttribute(index_score_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int max_tiles = (score_stride + IM_TILE - 1) / IM_TILE;
    // work items of 16 tiles; when that leaves SMs without any item (a small batch), smaller items: about four per SM
    // (measured: 17.9 -> 15.2 us at batch 16 x 16,384 tokens, while batches that already fill the chip lose 10 % to the
    // per-item set-up with smaller items)
    if ((long long)B * ((max_tiles + IM_TPI - 1) / IM_TPI) >= 6LL * sms) {
        ma.tpi = IM_TPI / 2;   // plenty of items: halves of them even out the last round (measured: 160.6 -> 158.6 us per step at batch 128 x 16,384)
    } else if ((long long)B * ((max_tiles + IM_TPI - 1) / IM_TPI) < sms) {
        long long tpi = (long long)B * max_tiles / (4LL * sms);
        ma.tpi = (int)(tpi < 2 ? 2 : (tpi > IM_TPI ? IM_TPI : tpi));
    }
    const int n_items = B * ((max_tiles + ma.tpi - 1) / ma.tpi);
    const int grid = n_items < 2 * sms ? n_items : 2 * sms;
    CUtensorMap tm_keys, tm_q;
    if (int e = rivoli::make_tmap_rows_sw128(&tm_keys, index_pool, (uint64_t)g->n_pool_pages * g->page_tokens, IM_HD,
                                             (uint32_t)g->page_tokens))
        return e;
    if (int e = rivoli::make_tmap_rows_sw128(&tm_q, s.qcodes, (uint64_t)B * nh, IM_HD, (uint32_t)nh)) return e;
    rv_stage_event(1, st);
    rv_launch_dependent(index_score_mma_kernel, dim3(grid), dim3(IM_THREADS), smem1, st, ma, tm_keys, tm_q);
    if (int e = rv_launch_status()) return e;
    rv_stage_event(2, st);

    const SelArgs ra{*g, s.scores, score_stride, seq_len, s.qcodes, s.qscales, w, s.cb,
                     index_pool, index_scale, block_table, rows, n_sel, g->top_k, s.stats,
                     (score_stride % 4 == 0 && ((uintptr_t)index_scale & 15) == 0 && g->page_tokens % 4 == 0) ? 1 : 0};
    return rivoli::launch_index_select_cluster(ra, B, st);
}

RIVOLI_API int rivoli_index_select_paged(const DsaGeom* g, const uint16_t* index_q, const float* w,
                                         const uint8_t* index_pool, const float* index_scale,
                                         const int32_t* block_table, const int32_t* seq_len, int B,
                                         int score_stride, uint32_t* rows, int32_t* n_sel, void* scratch,
                                         void* stream) {
    return select_impl(g, nullptr, index_q, w, index_pool, index_scale, block_table, seq_len, B, score_stride, rows,
                       n_sel, scratch, stream);
}

// Decode step, first half: append the step's token of every sequence (row b belongs to sequence
// b, position row_pos[b]) AND select the attended rows, with the append riding in the launch
// that prepares the indexer query. Same results as rivoli_kv_append_paged followed by
// rivoli_index_select_paged.
RIVOLI_API int rivoli_dsa_append_select_paged(const DsaGeom* g, const uint16_t* latent, const uint16_t* index_key,
                                              const int32_t* row_pos, const int32_t* block_table,
                                              uint8_t* latent_pool, float* latent_scale, uint8_t* index_pool,
                                              float* index_scale, int32_t* status, const uint16_t* index_q,
                                              const float* w, const int32_t* seq_len, int B, int score_stride,
                                              uint32_t* rows, int32_t* n_sel, void* scratch, void* stream) {
    if (int e = rv_check_geom(g)) return e;
    if (B <= 0 || !latent || !index_key || !row_pos || !block_table || !latent_pool || !latent_scale || !index_pool ||
        !index_scale)
        return 1001;
    if ((g->rope_dim % 4) != 0 || ((g->kv_lora + g->rope_dim) % 16) != 0) return 1004;
    if ((((uintptr_t)latent | (uintptr_t)index_key | (uintptr_t)latent_pool | (uintptr_t)index_pool) & 15) ||
        ((uintptr_t)latent_scale & 3))
        return 1005;
    const AppendArgs ap{latent, index_key, row_pos, block_table, latent_pool, latent_scale, index_pool, index_scale, status};
    return select_impl(g, &ap, index_q, w, index_pool, index_scale, block_table, seq_len, B, score_stride, rows, n_sel,
                       scratch, stream);
}

// Where the last rivoli_index_select_paged call on `scratch` left the query codes and their scales (both paths
// of that call fill them): read by the page-range shard step, which re-scores its candidates exactly.
extern "C" void rivoli_index_select_query_codes(const DsaGeom* g, int B, int score_stride, void* scratch,
                                                const uint8_t** qcodes, const float** qscales) {
    size_t total = 0;
    SelectScratch s = carve(g, B, score_stride, scratch, &total);
    *qcodes = s.qcodes;
    *qscales = s.qscales;
}

// Reads back the tensor-core scorer's error word and clears it: 1005 = a block-table entry inside a
// sequence's length pointed outside the pool (rows undefined), 1008 = a bounded wait gave up.
// Synchronises the stream.
RIVOLI_API int rivoli_index_select_status(const DsaGeom* g, int B, int score_stride, void* scratch, void* stream) {
    if (!g || !scratch) return 1001;
    size_t total = 0;
    SelectScratch s = carve(g, B, score_stride, scratch, &total);
    int h = 0;
    cudaError_t e = cudaMemcpyAsync(&h, s.err, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return -(int)e;
    if (h) cudaMemsetAsync(s.err, 0, sizeof(int), (cudaStream_t)stream);
    return h == IM_ERR_BAD_PAGE ? 1005 : (h ? 1008 : 0);
}

// Diagnostics: copies the per-sequence band sizes of the last call (tokens re-scored
// exactly) to host memory. Synchronises the stream.
RIVOLI_API int rivoli_index_select_band_stats(const DsaGeom* g, int B, int score_stride, void* scratch,
                                              uint32_t* host_band, void* stream) {
    if (!g || !scratch || !host_band || B <= 0) return 1001;
    size_t total = 0;
    SelectScratch s = carve(g, B, score_stride, scratch, &total);
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaMemcpy2D(host_band, 4, s.stats, 8, 4, (size_t)B, cudaMemcpyDeviceToHost);
    return e == cudaSuccess ? 0 : -(int)e;
}

