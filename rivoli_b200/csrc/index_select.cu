// Exact top-k selection over the tensor-core scorer's approximate scores: one thread-block CLUSTER per
// sequence, so a sequence's tokens are spread over up to 8 SMs whatever the batch size is.
//
// Input: a_t (approximate score of token t, without the key scale) from index_score_mma_kernel, with
// |a_t * s_k[t] - o_t| <= eps for the exact score o_t. With A_k the k-th largest approximate score,
// a_t > A_k + 2 eps implies "selected" and a_t < A_k - 2 eps implies "not selected" (|A_k - E_k| <= eps for
// the exact k-th value E_k); the band in between is re-scored in the exact fold order of
// rivoli_index_score_paged and ranked exactly (ties -> lower index). The rows written are therefore
// IDENTICAL to exact scoring + exact top-k (contract and tie rule: crates/backend/kernels/indexer.hip:143-257,
// crates/core/src/routing.rs:42-61).
//
// Layout: CTA `r` of a cluster of C owns the CH = EPT * 512 consecutive tokens [r * CH, (r + 1) * CH), thread t
// the EPT consecutive tokens from r * CH + t * EPT, keys in registers. What the CTAs of a cluster exchange
// goes through distributed shared memory (plain loads / stores on mapped addresses), mostly PUSHED into the
// reader's memory so that a CTA needs nobody else's memory after its last cluster barrier.
//
//   1. keys; cluster-wide min / max key and max key scale (eps).
//   2. ONE histogram pass over 4096 bins spread linearly in value between the smallest and the largest score:
//      the distribution decides the bin width, so the bin of the k-th value holds a handful of tokens on
//      score-like data. Histograms are all-reduced slice by slice, the k-th bin is found by a suffix scan.
//   3. classification against the band [smallest score of that bin - 2 eps, largest + 2 eps]; band tokens
//      are listed per CTA.
//   4. exact re-score of the CTA's own band tokens (a warp takes 4 at a time, lane = head), the lists are
//      gathered cluster-wide, every band token is ranked against all of them.
//   5. ascending write-out: counts are exchanged, each CTA compacts its own contiguous token range.
//
// A batch that fills the chip by itself runs this kernel as ONE CTA of 1024 threads per sequence (a cluster of one):
// for that shape the exchanges, the cluster barriers and the list copies are compiled out (SOLO below).
//
// If the band does not fit the list (tie-dominated scores: thousands of tokens at the cut) the cluster takes
// the slow path instead: every band token is re-scored chunk by chunk, the exact keys replace the approximate
// ones in the registers, and an exact 4 x 8-bit radix selection runs over the whole cluster.
#include <cooperative_groups.h>

#include "codec.cuh"
#include "common.cuh"
#include "index_rescore.cuh"
#include "index_select.hpp"
#include "topk_core.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int SEL_MAX_WARPS = 32;   // CTAs of 512 threads (clusters of 2 to 8) or of 1024 threads (one CTA per sequence)
constexpr int SEL_BINS = 4096;
constexpr int SEL_LIST = 2048;     // band tokens per SEQUENCE the fast path holds (and per chunk on the slow path)
constexpr int SEL_TOK = 4;         // band tokens a warp re-scores per pass
constexpr int SEL_HD = RS_HD;      // index dim (one code word per lane)

struct SelXc {                     // per-CTA exchange block; slot q of an array is written by rank q (its own copy in phase 1)
    uint32_t kmin[SEL_MAX_CLUSTER], kmax[SEL_MAX_CLUSTER], skmax[SEL_MAX_CLUSTER];
    uint32_t slice_tot[SEL_MAX_CLUSTER];
    uint32_t bmin[SEL_MAX_CLUSTER], bmax[SEL_MAX_CLUSTER];
    uint32_t n_in[SEL_MAX_CLUSTER], n_band[SEL_MAX_CLUSTER];
    uint32_t n_out[SEL_MAX_CLUSTER];
    uint32_t cnt_gt[SEL_MAX_CLUSTER], cnt_eq[SEL_MAX_CLUSTER];
    uint32_t red[2][SEL_MAX_WARPS];
    uint32_t red3[2][3][SEL_MAX_WARPS];
    uint32_t wcnt[SEL_MAX_WARPS];
    uint32_t list_n;
    uint32_t bstar, n_above;
    uint32_t pivot, need;
};

// Block-wide reductions over NW warps, one barrier per call (double-buffered partials as in topk_core.cuh).
template <int NW>
__device__ __forceinline__ uint32_t sel_block_sum(uint32_t v, SelXc& xc, int& buf) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = __reduce_add_sync(0xffffffffu, v);
    if (lane == 0) xc.red[buf][warp] = v;
    __syncthreads();
    const uint32_t t = __reduce_add_sync(0xffffffffu, lane < NW ? xc.red[buf][lane] : 0u);
    buf ^= 1;
    return t;
}
template <int NW>
__device__ __forceinline__ uint32_t sel_block_max(uint32_t v, SelXc& xc, int& buf) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = __reduce_max_sync(0xffffffffu, v);
    if (lane == 0) xc.red[buf][warp] = v;
    __syncthreads();
    const uint32_t t = __reduce_max_sync(0xffffffffu, lane < NW ? xc.red[buf][lane] : 0u);
    buf ^= 1;
    return t;
}
template <int NW>
__device__ __forceinline__ uint32_t sel_block_min(uint32_t v, SelXc& xc, int& buf) {
    return ~sel_block_max<NW>(~v, xc, buf);
}

// min, max and a second max over the block in ONE barrier.
template <int NW>
__device__ __forceinline__ void sel_block_minmaxmax(uint32_t& mn, uint32_t& mx, uint32_t& mx2, SelXc& xc, int& buf) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    mn = __reduce_min_sync(0xffffffffu, mn);
    mx = __reduce_max_sync(0xffffffffu, mx);
    mx2 = __reduce_max_sync(0xffffffffu, mx2);
    if (lane == 0) { xc.red3[buf][0][warp] = mn; xc.red3[buf][1][warp] = mx; xc.red3[buf][2][warp] = mx2; }
    __syncthreads();
    mn = __reduce_min_sync(0xffffffffu, lane < NW ? xc.red3[buf][0][lane] : 0xffffffffu);
    mx = __reduce_max_sync(0xffffffffu, lane < NW ? xc.red3[buf][1][lane] : 0u);
    mx2 = __reduce_max_sync(0xffffffffu, lane < NW ? xc.red3[buf][2][lane] : 0u);
    buf ^= 1;
}

// Exclusive prefix of `v` over the block in thread order (one barrier).
template <int NW>
__device__ __forceinline__ uint32_t sel_block_excl(uint32_t v, SelXc& xc) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) xc.wcnt[warp] = incl;
    __syncthreads();
    const uint32_t cw = lane < NW ? xc.wcnt[lane] : 0u;
    const uint32_t pre = __reduce_add_sync(0xffffffffu, lane < warp ? cw : 0u);
    __syncthreads();                                   // wcnt may be rewritten by the next call
    return pre + incl - v;
}

template <int EPT, int NT>
__global__ void __launch_bounds__(NT, (NT == 512 && EPT <= 16) ? 2 : 1)
index_select_cluster_kernel(SelArgs A) {
    constexpr int NW = NT / 32;
    // A CTA of 1024 threads is launched only as a cluster of ONE (a batch that fills the chip by itself): every
    // exchange between CTAs and every cluster barrier falls away at compile time, and with them most of the block
    // barriers, which is what this latency-bound kernel is made of.
    constexpr bool SOLO = NT == 1024;
    cg::cluster_group cluster = cg::this_cluster();
    const int C = SOLO ? 1 : (int)cluster.dim_blocks().x, r = SOLO ? 0 : (int)cluster.block_rank();
    extern __shared__ __align__(16) uint32_t sel_smem[];
    __shared__ SelXc xc;
    uint32_t* qf = sel_smem;                                              // [SEL_HD / 4][32] packed q codes, [word][head]
    float* kfw = reinterpret_cast<float*>(qf + (SEL_HD / 4) * 32);        // [NW][SEL_TOK][SEL_HD] key rows as f32
    uint32_t* hist = reinterpret_cast<uint32_t*>(kfw + NW * SEL_TOK * SEL_HD);   // [SEL_BINS]; later `dec`
    uint32_t* l_tok = hist + SEL_BINS;                                    // [SEL_LIST] this CTA's band tokens
    uint32_t* l_key = l_tok + SEL_LIST;                                   // [SEL_LIST] their exact keys
    uint32_t* a_tok = l_key + SEL_LIST;                                   // [SEL_LIST] the cluster's band, gathered
    uint32_t* a_key = a_tok + SEL_LIST;                                   // [SEL_LIST]
    uint32_t* red_hist = a_tok;                                           // [SEL_BINS / C] reduced histogram slice (phase 2)
    uint32_t* slice = l_tok;                                              // [SEL_BINS / C] the slice holding the k-th bin

    const DsaGeom& g = A.g;
    constexpr int hd = SEL_HD;
    const int nh = g.index_heads, P = g.page_tokens;
    const int b = (int)blockIdx.x / C, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    rv_grid_dep_trigger();   // the next kernel may set itself up; it waits for this grid before reading rows
    rv_grid_dep_wait();      // scores, query codes and the error constant come from the kernels before
    const int nt = min(A.seq_len[b], A.score_stride);
    const int kk = min(A.k, nt);
    uint32_t* out = A.rows + (size_t)b * A.k;
    if (r == 0 && tid == 0) A.n_sel[b] = kk > 0 ? kk : 0;
    if (kk <= 0) return;                                                  // uniform over the cluster
    constexpr int CH = EPT * NT;
    const int i0 = r * CH + tid * EPT;
    const int nvalid = max(0, min(EPT, nt - i0));
    if (kk == nt) {                                                       // everything is selected: the identity
#pragma unroll
        for (int j = 0; j < EPT; ++j)
            if (j < nvalid) out[i0 + j] = (uint32_t)(i0 + j);
        if (r == 0 && tid == 0 && A.stats) { A.stats[b * 2] = 0; A.stats[b * 2 + 1] = (unsigned)nt; }
        return;
    }

    // ---- 1. approximate keys: (unscaled tensor-core score) * key scale of the token --------------------------
    const float* s = A.scores + (size_t)b * A.score_stride;
    const int32_t* bt = A.block_table + (size_t)b * g.max_pages_per_seq;
    uint32_t key[EPT];
    float skm = 0.0f;
    {
        float sc[EPT], sk[EPT];
        if (A.vec_ok && nvalid == EPT) {
            size_t rr[EPT / 4];
#pragma unroll
            for (int j4 = 0; j4 < EPT / 4; ++j4) {
                const int i = i0 + j4 * 4;
                int pg = bt[i / P];
                pg = (pg < 0 || pg >= g.n_pool_pages) ? 0 : pg;
                rr[j4] = (size_t)pg * P + (i & (P - 1));
            }
#pragma unroll
            for (int j4 = 0; j4 < EPT / 4; ++j4) {
                const float4 a = *reinterpret_cast<const float4*>(s + i0 + j4 * 4);
                const float4 c = *reinterpret_cast<const float4*>(A.index_scale + rr[j4]);
                sc[j4 * 4] = a.x; sc[j4 * 4 + 1] = a.y; sc[j4 * 4 + 2] = a.z; sc[j4 * 4 + 3] = a.w;
                sk[j4 * 4] = c.x; sk[j4 * 4 + 1] = c.y; sk[j4 * 4 + 2] = c.z; sk[j4 * 4 + 3] = c.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                const int i = i0 + j;
                sc[j] = 0.0f; sk[j] = 0.0f;
                if (j < nvalid) {
                    int pg = bt[i / P];
                    pg = (pg < 0 || pg >= g.n_pool_pages) ? 0 : pg;
                    sc[j] = s[i];
                    sk[j] = A.index_scale[(size_t)pg * P + (i & (P - 1))];
                }
            }
        }
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            key[j] = j < nvalid ? topk_key(sc[j] * sk[j]) : 0u;
            skm = fmaxf(skm, sk[j]);
        }
    }
    rv_rescore_stage_q(A.qcodes + (size_t)b * nh * hd, nh, qf);
    for (int i = tid; i < SEL_BINS; i += NT) hist[i] = 0u;
    if (tid == 0) xc.list_n = 0;
    int buf = 0;
    uint32_t kmin = 0xffffffffu, kmax = 0u;
    float sk_max = 0.0f;
    {
        uint32_t mn = 0xffffffffu, mx = 0u;
#pragma unroll
        for (int j = 0; j < EPT; ++j)
            if (j < nvalid) { mn = min(mn, key[j]); mx = max(mx, key[j]); }
        uint32_t sm = __float_as_uint(skm);                                      // scales are >= 0: bit order = value order
        sel_block_minmaxmax<NW>(mn, mx, sm, xc, buf);                            // (also orders the zeroing above before the histogram)
        if constexpr (SOLO) {
            kmin = mn; kmax = mx; sk_max = __uint_as_float(sm);
        } else {
            if (tid == 0) { xc.kmin[r] = mn; xc.kmax[r] = mx; xc.skmax[r] = sm; }
            // [1] The first exchange is a PULL: a CTA may touch another CTA's shared memory only once that CTA is known
            // to be running, which its arrival at this barrier proves. Every later exchange pushes.
            cluster.sync();
            for (int q = 0; q < C; ++q) {
                const SelXc* src = cluster.map_shared_rank(&xc, q);
                kmin = min(kmin, src->kmin[q]); kmax = max(kmax, src->kmax[q]);
                sk_max = fmaxf(sk_max, __uint_as_float(src->skmax[q]));
            }
        }
    }
    const float eps = sk_max * A.cb[b];

    // ---- 2. one histogram pass: 4096 bins spread linearly IN VALUE between the smallest and the largest score ----
    // bin(v) = min(4095, int((v - vmin) * inv_w)) is monotone in v, which is all the selection needs: tokens in
    // higher bins than the k-th value's are above it, tokens in lower bins below. (Bins linear in the key BITS
    // would be logarithmic in value: 6 % wide around 1.0.) A degenerate range (all scores equal, or a span
    // that overflows) gives inv_w = 0 and one bin; the slow path below takes such inputs.
    const float vmin = topk_unkey(kmin), vmax = topk_unkey(kmax);
    float inv_w = (float)SEL_BINS / (vmax - vmin);
    if (!(inv_w > 0.0f) || !(inv_w < 3.0e38f)) inv_w = 0.0f;
    auto bin_of = [&](uint32_t k) -> uint32_t {
        const float t = (topk_unkey(k) - vmin) * inv_w;
        return (uint32_t)fminf(t, (float)(SEL_BINS - 1));
    };
    {
        // consecutive tokens often share a bin (runs of ReLU zeros): one shared-memory atomic per run
        uint32_t cur = 0xffffffffu, run = 0u;
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            if (j < nvalid) {
                const uint32_t bin = bin_of(key[j]);
                if (bin != cur) { if (run) atomicAdd(&hist[cur], run); cur = bin; run = 0u; }
                ++run;
            }
        }
        if (run) atomicAdd(&hist[cur], run);
    }
    __syncthreads();
    int SL = SEL_BINS;                                                        // bins of the slice that holds the k-th value
    int s_star = 0;
    uint32_t above = 0u;                                                      // tokens in slices above the k-th value's
    uint32_t slice_total = (uint32_t)nt;                                      // tokens in that slice
    const uint32_t* slice_c = hist;
    if constexpr (!SOLO) {
        cluster.sync();                                                       // [2] every CTA's histogram is complete
        SL = SEL_BINS / C;                                                    // rank r reduces bins [r * SL, (r + 1) * SL)
        {
            uint32_t tot = 0u;
            for (int i = tid; i < SL; i += NT) {
                uint32_t v = 0u;
                for (int q = 0; q < C; ++q) v += cluster.map_shared_rank(hist, q)[r * SL + i];
                red_hist[i] = v;
                tot += v;
            }
            tot = sel_block_sum<NW>(tot, xc, buf);
            if (tid < C) cluster.map_shared_rank(&xc, tid)->slice_tot[r] = tot;
        }
        __syncthreads();
        cluster.sync();                                                       // [3] reduced slices and their totals
        for (int q = C - 1; q >= 0; --q) {
            if (above + xc.slice_tot[q] >= (uint32_t)kk) { s_star = q; break; }
            above += xc.slice_tot[q];
        }
        {
            const uint32_t* src = cluster.map_shared_rank(red_hist, s_star);
            for (int i = tid; i < SL; i += NT) slice[i] = src[i];
        }
        __syncthreads();
        slice_total = xc.slice_tot[s_star];
        slice_c = slice;
    }
    {
        // suffix scan over the slice: thread t owns bins [t * per, (t + 1) * per), per = ceil(SL / 512)
        const int per = (SL + NT - 1) / NT;
        uint32_t mine = 0u;
        for (int j = 0; j < per; ++j) { const int i = tid * per + j; if (i < SL) mine += slice_c[i]; }
        const uint32_t before = sel_block_excl<NW>(mine, xc);                     // bins below this thread's
        const uint32_t total = slice_total;
        uint32_t acc = above + (total - before - mine);                       // tokens in bins above this thread's
        for (int j = per - 1; j >= 0; --j) {
            const int i = tid * per + j;
            if (i < SL) {
                const uint32_t h = slice_c[i];
                if (acc < (uint32_t)kk && (uint32_t)kk <= acc + h) { xc.bstar = (uint32_t)(s_star * SL + i); xc.n_above = acc; }
                acc += h;
            }
        }
    }
    __syncthreads();
    const uint32_t bstar = xc.bstar;

    // ---- 3. classification: surely selected / band (re-scored exactly) / surely not -------------------------
    // The k-th approximate score is one of the tokens of bin `bstar`: it lies between the smallest and the
    // largest key found there (exact bounds, no reasoning about the rounding of bin_of needed).
    uint32_t k_lo, k_hi;
    {
        uint32_t mn = 0xffffffffu, mx = 0u;
#pragma unroll
        for (int j = 0; j < EPT; ++j)
            if (j < nvalid && bin_of(key[j]) == bstar) { mn = min(mn, key[j]); mx = max(mx, key[j]); }
        uint32_t unused = 0u;
        sel_block_minmaxmax<NW>(mn, mx, unused, xc, buf);
        if constexpr (!SOLO) {
            if (tid < C) {
                SelXc* dst = cluster.map_shared_rank(&xc, tid);
                dst->bmin[r] = mn; dst->bmax[r] = mx;
            }
            cluster.sync();                                                   // [3b]
            mn = 0xffffffffu; mx = 0u;
            for (int q = 0; q < C; ++q) { mn = min(mn, xc.bmin[q]); mx = max(mx, xc.bmax[q]); }
        }
        const float lo_f = topk_unkey(mn) - 2.0f * eps, hi_f = topk_unkey(mx) + 2.0f * eps;
        k_lo = lo_f == lo_f ? topk_key(lo_f) : 0u;
        k_hi = hi_f == hi_f ? topk_key(hi_f) : 0xffffffffu;
    }
    uint32_t m_in = 0u, m_band = 0u;
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        if (j < nvalid) {
            if (key[j] > k_hi) m_in |= 1u << j;
            else if (key[j] >= k_lo) m_band |= 1u << j;
        }
    }
    {   // this CTA's count of surely selected tokens: the warp sums meet at the barrier that closes the list
        const uint32_t v = __reduce_add_sync(0xffffffffu, (uint32_t)__popc(m_in));
        if (lane == 0) xc.red[buf][warp] = v;
    }
    uint32_t my_pos;                                                          // list position of this thread's first band token
    {
        const uint32_t cnt = (uint32_t)__popc(m_band);
        uint32_t incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        uint32_t wbase = 0u;
        if (lane == 31 && incl) wbase = atomicAdd(&xc.list_n, incl);          // order inside the list is irrelevant
        wbase = __shfl_sync(0xffffffffu, wbase, 31);
        my_pos = wbase + incl - cnt;
        uint32_t pos = my_pos;
#pragma unroll
        for (int j = 0; j < EPT; ++j)
            if (m_band & (1u << j)) { if (pos < SEL_LIST) l_tok[pos] = (uint32_t)(i0 + j); ++pos; }
    }
    __syncthreads();
    const uint32_t n_in_mine = __reduce_add_sync(0xffffffffu, lane < NW ? xc.red[buf][lane] : 0u);
    buf ^= 1;
    const uint32_t n_band_mine = xc.list_n;
    uint32_t n_in = n_in_mine, n_band = n_band_mine;
    if constexpr (!SOLO) {
        if (tid < C) {
            SelXc* dst = cluster.map_shared_rank(&xc, tid);
            dst->n_in[r] = n_in_mine; dst->n_band[r] = n_band_mine;
        }
        cluster.sync();                                                       // [4] (also: nobody reads red_hist any more)
        n_in = 0u; n_band = 0u;
        for (int q = 0; q < C; ++q) { n_in += xc.n_in[q]; n_band += xc.n_band[q]; }
    }

    // this lane's head constants for the exact re-score (nh <= 32)
    const float my_sq = lane < nh ? A.qscales[(size_t)b * nh + lane] : 0.0f;
    const float my_wh = lane < nh ? __fmul_rn(A.w[(size_t)b * nh + lane], g.index_wscale) : 0.0f;
    // Exact key of the first `ln` listed tokens -> l_key[position] (0 and ~0 are reserved for "surely out" / "surely in").
    auto rescore = [&](uint32_t ln) {
        rv_rescore_listed<NW, SEL_TOK>(l_tok, ln, qf, kfw + warp * (SEL_TOK * hd), bt, g, A.index_pool, A.index_scale,
                                              my_sq, my_wh, [&](uint32_t pos, float score) {
            uint32_t ku = topk_key(score);
            l_key[pos] = ku == 0xffffffffu ? 0xfffffffeu : (ku == 0u ? 1u : ku);
        });
    };
    // ascending write-out of this CTA's tokens whose bit is set in `sel`, from slot `base` on (one barrier)
    auto write_out = [&](uint32_t sel, uint32_t base) {
        uint32_t pos = base + sel_block_excl<NW>((uint32_t)__popc(sel), xc);
#pragma unroll
        for (int j = 0; j < EPT; ++j)
            if (sel & (1u << j)) out[pos++] = (uint32_t)(i0 + j);
    };

    if (n_band <= (uint32_t)SEL_LIST) {
        // ---- 4. common case: the whole band fits the list --------------------------------------------------
        rescore(n_band_mine);
        __syncthreads();
        const uint32_t* all_tok = l_tok;                                      // the cluster's band: a lone CTA's own lists
        const uint32_t* all_key = l_key;
        if constexpr (!SOLO) {
            cluster.sync();                                                   // [5] every CTA's exact band keys
            uint32_t off = 0u;
            for (int q = 0; q < C; ++q) {
                const uint32_t nq = xc.n_band[q];
                const uint32_t* st = cluster.map_shared_rank(l_tok, q);
                const uint32_t* sk2 = cluster.map_shared_rank(l_key, q);
                for (uint32_t i = tid; i < nq; i += NT) { a_tok[off + i] = st[i]; a_key[off + i] = sk2[i]; }
                off += nq;
            }
            __syncthreads();
            all_tok = a_tok; all_key = a_key;
        }
        // rank each of this CTA's band tokens among ALL band tokens by (exact key descending, index ascending)
        uint32_t* dec = hist;
        const uint32_t take = (uint32_t)kk - n_in;   // >= 1: fewer than kk tokens lie above the band
        for (uint32_t q2 = warp; q2 < n_band_mine; q2 += NW) {
            const uint32_t kq = l_key[q2], tq = l_tok[q2];
            uint32_t c = 0;
            for (uint32_t j2 = lane; j2 < n_band; j2 += 32) {
                const uint32_t kj = all_key[j2];
                c += (kj > kq || (kj == kq && all_tok[j2] < tq)) ? 1u : 0u;
            }
            c = __reduce_add_sync(0xffffffffu, c);
            if (lane == 0) dec[q2] = c < take ? 1u : 0u;
        }
        __syncthreads();
        uint32_t sel = m_in;
        {
            uint32_t pos = my_pos;
#pragma unroll
            for (int j = 0; j < EPT; ++j)
                if (m_band & (1u << j)) { if (dec[pos]) sel |= 1u << j; ++pos; }
        }
        uint32_t base = 0u;
        if constexpr (!SOLO) {
            const uint32_t n_out_mine = sel_block_sum<NW>((uint32_t)__popc(sel), xc, buf);
            if (tid < C) cluster.map_shared_rank(&xc, tid)->n_out[r] = n_out_mine;
            cluster.sync();                                                   // [6] counts; nobody reads our lists any more
            for (int q = 0; q < r; ++q) base += xc.n_out[q];
        }
        write_out(sel, base);
        if (r == 0 && tid == 0 && A.stats) { A.stats[b * 2] = n_band; A.stats[b * 2 + 1] = n_in; }
        return;
    }

    // ---- slow path (tie-dominated scores): the band does not fit the list --------------------------------------
    // Exact keys replace the approximate ones in the registers: surely-in -> all ones, surely-out -> 0, band ->
    // exact key (re-scored in chunks of SEL_LIST consecutive tokens, so a chunk's band always fits the list).
    for (int c0 = r * CH; c0 < min(nt, (r + 1) * CH); c0 += SEL_LIST) {
        __syncthreads();
        if (tid == 0) xc.list_n = 0;
        __syncthreads();
        const bool mine = i0 >= c0 && i0 < c0 + SEL_LIST;                 // EPT divides SEL_LIST: a thread's tokens share a chunk
        uint32_t pos0 = 0u;
        if (mine && m_band) {
            pos0 = atomicAdd(&xc.list_n, (uint32_t)__popc(m_band));
            uint32_t pos = pos0;
#pragma unroll
            for (int j = 0; j < EPT; ++j)
                if (m_band & (1u << j)) l_tok[pos++] = (uint32_t)(i0 + j);
        }
        __syncthreads();
        rescore(xc.list_n);
        __syncthreads();
        if (mine) {
            uint32_t pos = pos0;
#pragma unroll
            for (int j = 0; j < EPT; ++j)
                if (m_band & (1u << j)) key[j] = l_key[pos++];
        }
    }
#pragma unroll
    for (int j = 0; j < EPT; ++j)
        if (j < nvalid && !(m_band & (1u << j))) key[j] = ((m_in >> j) & 1u) ? 0xffffffffu : 0u;
    // exact cluster-wide radix selection, four 8-bit digits, MSB first; per-warp histograms so that ties never
    // serialise a CTA on one bin; whist aliases `hist`, the CTA's digit histogram goes to a_tok[0..256)
    uint32_t pivot = 0u, mask = 0u, need = (uint32_t)kk;
    uint32_t* whist = hist;                                                   // [NW][256]
    for (int sh2 = 24; sh2 >= 0; sh2 -= 8) {
        __syncthreads();
        for (int i = tid; i < NW * 256; i += NT) whist[i] = 0u;
        __syncthreads();
#pragma unroll
        for (int j = 0; j < EPT; ++j)
            if (j < nvalid && (key[j] & mask) == pivot) atomicAdd(&whist[warp * 256 + ((key[j] >> sh2) & 0xffu)], 1u);
        __syncthreads();
        if (tid < 256) {
            uint32_t t = 0;
#pragma unroll
            for (int w2 = 0; w2 < NW; ++w2) t += whist[w2 * 256 + tid];
            a_tok[tid] = t;
        }
        __syncthreads();
        cluster.sync();                                                       // every CTA's digit histogram
        if (tid < 256) {
            uint32_t t = 0;
            for (int q = 0; q < C; ++q) t += cluster.map_shared_rank(a_tok, q)[tid];
            a_key[tid] = t;
        }
        __syncthreads();
        if (warp == 0) {
            // lane owns bins 8 * lane .. 8 * lane + 7; acc = entries in strictly higher bins
            uint32_t h[8], tot = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) { h[j] = a_key[lane * 8 + j]; tot += h[j]; }
            uint32_t incl = tot;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_down_sync(0xffffffffu, incl, o);
                if (lane + o < 32) incl += v;
            }
            uint32_t acc = incl - tot;
#pragma unroll
            for (int j = 7; j >= 0; --j) {
                if (acc < need && need <= acc + h[j]) {
                    xc.pivot = pivot | ((uint32_t)(lane * 8 + j) << sh2);
                    xc.need = need - acc;
                }
                acc += h[j];
            }
        }
        __syncthreads();
        pivot = xc.pivot;
        need = xc.need;
        mask |= 0xffu << sh2;
        cluster.sync();                                                       // a_tok may be rewritten by the next digit
    }
    // `need` of the tokens tied at the pivot are taken, in ascending global index = ascending rank, then thread
    uint32_t sel_gt = 0u, sel_eq = 0u;
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        if (j < nvalid) {
            if (key[j] > pivot) sel_gt |= 1u << j;
            else if (key[j] == pivot) sel_eq |= 1u << j;
        }
    }
    const uint32_t gt_mine = sel_block_sum<NW>((uint32_t)__popc(sel_gt), xc, buf);
    const uint32_t eq_mine = sel_block_sum<NW>((uint32_t)__popc(sel_eq), xc, buf);
    if (tid < C) {
        SelXc* dst = cluster.map_shared_rank(&xc, tid);
        dst->cnt_gt[r] = gt_mine; dst->cnt_eq[r] = eq_mine;
    }
    cluster.sync();
    uint32_t base = 0u, eq_before = 0u;
    for (int q = 0; q < r; ++q) {
        const uint32_t left = need > eq_before ? need - eq_before : 0u;
        base += xc.cnt_gt[q] + min(xc.cnt_eq[q], left);
        eq_before += xc.cnt_eq[q];
    }
    const uint32_t need_mine = need > eq_before ? need - eq_before : 0u;        // ties this CTA may still take
    const uint32_t eq_excl = sel_block_excl<NW>((uint32_t)__popc(sel_eq), xc);      // ties in this CTA before this thread's
    uint32_t sel = sel_gt;
    {
        uint32_t e = eq_excl;
#pragma unroll
        for (int j = 0; j < EPT; ++j)
            if (sel_eq & (1u << j)) { if (e < need_mine) sel |= 1u << j; ++e; }
    }
    write_out(sel, base);
    if (r == 0 && tid == 0 && A.stats) { A.stats[b * 2] = n_band; A.stats[b * 2 + 1] = 0; }
}

}  // namespace

namespace rivoli {

static int g_sel_cluster_override = 0;

bool select_cluster_plan(int B, int score_stride, int* cluster, int* ept, int* threads) {
    // A batch that fills the chip by itself (one CTA per SM) takes ONE CTA of 1024 threads per sequence: no exchange
    // between CTAs at all. Smaller batches spread a sequence over a cluster of 2 to 8 CTAs of 512 threads, about two
    // CTAs per SM at most.
    int C = 1, NT = 512;
    if ((long long)B * 4 < 3 * 148)   // from three quarters of the SMs on, one CTA per sequence (measured at batch 128: 161 against 166 us per step with clusters of 2)
        while (C < SEL_MAX_CLUSTER && (long long)B * C * 2 <= 2 * 148) C *= 2;
    if (g_sel_cluster_override > 0) C = g_sel_cluster_override;
    if (C == 1 && (long long)1024 * 16 >= score_stride) NT = 1024;   // 16 keys per thread fit the 64 registers of a 1024-thread CTA
    for (;;) {
        for (int e = 4; e <= 32; e *= 2)
            if ((long long)C * NT * e >= score_stride) { *cluster = C; *ept = e; *threads = NT; return true; }
        if (C >= SEL_MAX_CLUSTER) return false;
        C *= 2;
        NT = 512;
    }
}

}  // namespace rivoli

// Test hook: force the cluster size of the following selection launches (1, 2, 4 or 8; 0 = the plan's own choice),
// so that every cluster size can be exercised at any batch size.
extern "C" __attribute__((visibility("default"))) void rivoli_index_select_test_cluster(int cluster) {
    rivoli::g_sel_cluster_override = (cluster == 1 || cluster == 2 || cluster == 4 || cluster == 8) ? cluster : 0;
}

namespace rivoli {

int launch_index_select_cluster(const SelArgs& a, int B, cudaStream_t st) {
    int C = 1, ept = 4, nt = 512;
    if (!select_cluster_plan(B, a.score_stride, &C, &ept, &nt)) return 1002;
    const size_t smem = ((size_t)(SEL_HD / 4) * 32 + (size_t)(nt / 32) * SEL_TOK * SEL_HD + SEL_BINS + 4 * SEL_LIST) * 4;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(B * C)); cfg.blockDim = dim3((unsigned)nt); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = (unsigned)C; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 2;
    rv_drain_error();
#define RV_SEL(EPT, NT)                                                                                                   \
    do {                                                                                                                  \
        cudaFuncSetAttribute(index_select_cluster_kernel<EPT, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        (void)cudaLaunchKernelEx(&cfg, index_select_cluster_kernel<EPT, NT>, a);                                          \
    } while (0)
    if (nt == 1024) {
        if (ept == 4) RV_SEL(4, 1024);
        else if (ept == 8) RV_SEL(8, 1024);
        else if (ept == 16) RV_SEL(16, 1024);
        else return 1002;   // the plan takes 1024-thread CTAs only up to 16 keys per thread
    } else {
        if (ept == 4) RV_SEL(4, 512);
        else if (ept == 8) RV_SEL(8, 512);
        else if (ept == 16) RV_SEL(16, 512);
        else RV_SEL(32, 512);
    }
#undef RV_SEL
    return rv_launch_status();
}

}  // namespace rivoli
