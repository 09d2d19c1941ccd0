/*
 * CPU oracle for the V4 cousin of the decode path: Hadamard + fp4 spread, block scorer,
 * scored block selection, and MQA sparse attention with a per-head sink.
 *
 * TEST INFRASTRUCTURE ONLY (same rule as rivoli_oracle.c): nothing in the product package
 * links, loads or calls this file.
 *
 * Each function restates one piece of the reference's host algorithm and cites the
 * reference file:line it follows (paths relative to the reference project root).
 *
 * Pinning status:
 *   - e2m1 codec, power-of-two scale rounding, the Sylvester basis order of the Hadamard,
 *     the f32-accumulate-then-round score rule (1.125 case) and the selection tie / order /
 *     padding rules are pinned by literal values recorded in the reference's tests
 *     (crates/engine/tests/kernel_v4_indexer.rs:689-726,
 *      crates/engine/src/v4/select.rs:534-541,681-707,714-740).
 *   - sparse attention has no literal expected values in the reference (its tests compare
 *     against captures its Rust oracle produces at run time); the fold order of
 *     crates/oracles/src/v4oracle/attention.rs:119-201 is restated statement for statement
 *     and is "unpinned" beyond that.
 *
 * Compile with -ffp-contract=off: every fold here rounds once per operation.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

uint16_t orc_f32_to_bf16(float x);
float orc_bf16_to_f32(uint16_t b);

static inline float rbf16(float x) { return orc_bf16_to_f32(orc_f32_to_bf16(x)); }
static inline uint32_t fbits(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float bitsf(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

/* ---- e2m1 (fp4) element codec: crates/oracles/src/v4oracle/numerics.rs:158-186 -------------- */
ORC_API float orc_e2m1_decode(uint8_t nib) {
    static const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    const float m = mag[nib & 7];
    return (nib & 8) ? -m : m;
}

/* Nearest code; a value on a midpoint goes to the code with the even mantissa bit. */
ORC_API uint8_t orc_e2m1_encode(float x) {
    static const float mid[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
    const float a = fabsf(x);
    unsigned code = 0;
    for (int i = 0; i < 7; ++i) code += (a > mid[i] || (a == mid[i] && (i & 1))) ? 1u : 0u;
    return (uint8_t)((signbit(x) ? 8u : 0u) | code);
}

/* Smallest power of two >= amax * max_inv, by exponent-field arithmetic:
 * crates/oracles/src/v4oracle/numerics.rs:202-218. */
ORC_API float orc_fast_round_scale(float amax, float max_inv) {
    const uint32_t b = fbits(amax * max_inv);
    const int e = (int)((b >> 23) & 0xffu) - 127 + ((b & 0x7fffffu) ? 1 : 0);
    return bitsf((uint32_t)(e + 127) << 23);
}

/* Block-32 fp4 quantise-dequantise in place: numerics.rs:245-298 (amax floor 6 * 2^-126). */
static void fp4_act_quant(float* row, int n) {
    const float FP4_MAX = 6.0f;
    const float floor_ = FP4_MAX * bitsf(1u << 23);
    for (int b0 = 0; b0 < n; b0 += 32) {
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(row[b0 + i]));
        amax = fmaxf(amax, floor_);
        const float s = orc_fast_round_scale(amax, 1.0f / FP4_MAX);
        for (int i = 0; i < 32; ++i) {
            float q = row[b0 + i] / s;
            q = q < -FP4_MAX ? -FP4_MAX : (q > FP4_MAX ? FP4_MAX : q);
            row[b0 + i] = orc_e2m1_decode(orc_e2m1_encode(q)) * s;
        }
    }
}

/* Natural-order (Sylvester) Walsh-Hadamard butterfly, then 1/sqrt(n): numerics.rs:324-353. */
ORC_API void orc_v4_hadamard(float* row, int n) {
    for (int h = 1; h < n; h <<= 1)
        for (int i = 0; i < n; i += 2 * h)
            for (int j = i; j < i + h; ++j) {
                const float a = row[j], b = row[j + h];
                row[j] = a + b;
                row[j + h] = a - b;
            }
    const float scale = 1.0f / sqrtf((float)n);
    for (int i = 0; i < n; ++i) row[i] *= scale;
}

/* The indexer's spread on `rows` rows of width d: Hadamard, bf16 store, fp4 block-32
 * simulation, bf16 store. crates/oracles/src/v4oracle/forward.rs:1130-1138;
 * device form crates/backend/kernels/blockindex.hip:97-138. Returns the launcher's guard. */
ORC_API int orc_v4_spread(float* x, int rows, int d) {
    if (rows <= 0 || d <= 0) return 1001;
    if (d > 256) return 1002;
    if (d & (d - 1)) return 1003;
    if (d % 32) return 1004;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        float* row = x + (size_t)r * d;
        orc_v4_hadamard(row, d);
        for (int i = 0; i < d; ++i) row[i] = rbf16(row[i]);
        fp4_act_quant(row, d);
        for (int i = 0; i < d; ++i) row[i] = rbf16(row[i]);
    }
    return 0;
}

/* score[t][c] = bf16( sum_h bf16( relu(bf16(q[t][h] . kv[c])) * w[t][h] ) ), the dot and the
 * head sum both ascending f32 folds: crates/engine/tests/kernel_v4_indexer.rs:437-460,
 * device form crates/backend/kernels/blockindex.hip:234-261. */
ORC_API int orc_v4_index_score_blocks(const float* q, const float* kv, const float* w, float* score,
                                      int s, int n_comp, int heads, int hd) {
    if (s <= 0 || heads <= 0 || hd <= 0) return 1001;
    if (n_comp <= 0) return 1005;
#pragma omp parallel for collapse(2) schedule(static)
    for (int t = 0; t < s; ++t)
        for (int c = 0; c < n_comp; ++c) {
            const float* kvr = kv + (size_t)c * hd;
            float acc = 0.0f;
            for (int hh = 0; hh < heads; ++hh) {
                const float* qh = q + ((size_t)t * heads + hh) * hd;
                float dot = 0.0f;
                for (int i = 0; i < hd; ++i) dot += qh[i] * kvr[i];
                dot = rbf16(dot);
                dot = fmaxf(dot, 0.0f);
                acc += rbf16(dot * w[(size_t)t * heads + hh]);
            }
            score[(size_t)t * n_comp + c] = rbf16(acc);
        }
    return 0;
}

/* f32 total order (sign-magnitude bits), the order Rust's total_cmp defines. */
static inline uint32_t total_key(float v) {
    const uint32_t b = fbits(v);
    return b ^ ((uint32_t)((int32_t)b >> 31) | 0x80000000u);
}
typedef struct { uint32_t key; int32_t idx; } sel_ent;
static int sel_cmp(const void* pa, const void* pb) {
    const sel_ent* a = (const sel_ent*)pa; const sel_ent* b = (const sel_ent*)pb;
    if (a->key != b->key) return a->key > b->key ? -1 : 1;
    return a->idx < b->idx ? -1 : (a->idx > b->idx ? 1 : 0);
}
static int i32_cmp(const void* pa, const void* pb) {
    const int32_t a = *(const int32_t*)pa, b = *(const int32_t*)pb;
    return a < b ? -1 : (a > b ? 1 : 0);
}

/* One ranked row: the best min(k, limit) of the first `limit` blocks by score (descending,
 * ties toward the lower index), emitted ascending, shifted by `offset`, padded with -1 out to
 * `width`. crates/engine/src/v4/select.rs:153-190 (limit = n_comp at decode,
 * min((t+1)/ratio, n_comp) for prefill row t). */
ORC_API void orc_v4_scored_row(const float* scores, int limit, int k, int offset, int width, int32_t* out) {
    sel_ent* e = (sel_ent*)malloc(sizeof(sel_ent) * (size_t)(limit > 0 ? limit : 1));
    for (int i = 0; i < limit; ++i) { e[i].key = total_key(scores[i]); e[i].idx = i; }
    qsort(e, (size_t)limit, sizeof(sel_ent), sel_cmp);
    const int n = k < limit ? k : limit;
    for (int i = 0; i < n; ++i) out[i] = e[i].idx;
    qsort(out, (size_t)n, sizeof(int32_t), i32_cmp);
    for (int i = 0; i < n; ++i) out[i] += offset;
    for (int i = n; i < width; ++i) out[i] = -1;
    free(e);
}

/* Decode-time window row: the ring read oldest-first once it is full, live slots then -1
 * padding before that. crates/engine/src/v4/select.rs:195-218 (decode arms). */
ORC_API void orc_v4_window_row(int win, int start_pos, int32_t* out) {
    if (start_pos >= win - 1) {
        const int cut = start_pos % win;
        int n = 0;
        for (int i = cut + 1; i < win; ++i) out[n++] = i;
        for (int i = 0; i <= cut; ++i) out[n++] = i;
    } else {
        for (int j = 0; j < win; ++j) out[j] = j <= start_pos ? j : -1;
    }
}

/* MQA sparse attention over one shared entry per position that is both key and value, gathered
 * by an explicit index list (-1 = masked), with sink[h] added to the softmax denominator only.
 * Fold order of crates/oracles/src/v4oracle/attention.rs:119-201: logits are ascending f32
 * dots times scale; the sum and the value accumulation ascend over live slots; the output is
 * stored bf16-rounded. A query whose slots are all masked writes NaN (the device contract,
 * crates/backend/kernels/attn.hip:346-352). */
ORC_API int orc_v4_sparse_attn(const float* q, const float* kv, const float* sink, const int32_t* idxs,
                               int m, int h, int d, int topk, float scale, float* o) {
    if (m <= 0 || h <= 0 || d <= 0 || topk <= 0) return 1001;
#pragma omp parallel
    {
        float* lg = (float*)malloc(sizeof(float) * (size_t)topk);
        float* acc = (float*)malloc(sizeof(float) * (size_t)d);
#pragma omp for collapse(2) schedule(static)
        for (int t = 0; t < m; ++t)
            for (int hh = 0; hh < h; ++hh) {
                const float* qh = q + ((size_t)t * h + hh) * d;
                const int32_t* ix = idxs + (size_t)t * topk;
                float* orow = o + ((size_t)t * h + hh) * d;
                float mx = -INFINITY;
                for (int j = 0; j < topk; ++j) {
                    if (ix[j] < 0) { lg[j] = -INFINITY; continue; }
                    const float* k = kv + (size_t)ix[j] * d;
                    float a = 0.0f;
                    for (int i = 0; i < d; ++i) a += qh[i] * k[i];
                    lg[j] = a * scale;
                    mx = fmaxf(mx, lg[j]);
                }
                if (!isfinite(mx)) {
                    for (int i = 0; i < d; ++i) orow[i] = NAN;
                    continue;
                }
                float sum = 0.0f;
                for (int i = 0; i < d; ++i) acc[i] = 0.0f;
                for (int j = 0; j < topk; ++j) {
                    if (ix[j] < 0) continue;
                    const float e = expf(lg[j] - mx);
                    sum += e;
                    const float* k = kv + (size_t)ix[j] * d;
                    for (int i = 0; i < d; ++i) acc[i] += e * k[i];
                }
                sum += expf(sink[hh] - mx);
                for (int i = 0; i < d; ++i) orow[i] = rbf16(acc[i] / sum);
            }
        free(lg);
        free(acc);
    }
    return 0;
}

/* ---- batched decode step over bf16 storage (the layout the CUDA path uses) ------------------
 * Per sequence b at position pos[b] (the query token's own position, already written):
 *   n_comp = (pos+1) / ratio closed blocks;
 *   compressed columns = all of them in order when n_comp <= index_topk
 *     (crates/engine/src/v4/select.rs:224-232), else the scored top index_topk (:153-190);
 *   row = [window ring order | compressed + window], width window + index_topk, -1 padded;
 *   out = sparse attention over kv_cache[b] ([window + max_comp][d]).
 * Values are bf16 in storage and widened exactly, so this equals the f32 functions above on
 * the widened arrays. `sel` receives the assembled rows, `score` (optional) the score rows. */
typedef struct {
    int32_t n_heads, head_dim, window, index_heads, index_dim, index_topk, ratio, max_comp;
    float softmax_scale;
} orc_v4_geom;

ORC_API void orc_v4_decode_step_bf16(const orc_v4_geom* g, int n_seqs, const int32_t* pos, const uint16_t* q,
                                     const uint16_t* kv_cache, const float* sink, const uint16_t* iq,
                                     const float* iw, const uint16_t* ikv, int32_t* sel, float* score_out,
                                     uint16_t* out) {
    const int H = g->n_heads, D = g->head_dim, W = g->window, IH = g->index_heads, ID = g->index_dim;
    const int K = g->index_topk, cols = W + K;
    const size_t kv_rows = (size_t)W + (size_t)g->max_comp;
    for (int b = 0; b < n_seqs; ++b) {
        int32_t* row = sel + (size_t)b * cols;
        orc_v4_window_row(W, pos[b], row);
        const int n_comp = (pos[b] + 1) / g->ratio;
        if (n_comp <= K) {
            for (int c = 0; c < K; ++c) row[W + c] = c < n_comp ? W + c : -1;
        } else {
            float* qf = (float*)malloc(sizeof(float) * (size_t)IH * ID);
            float* kf = (float*)malloc(sizeof(float) * (size_t)n_comp * ID);
            float* sc = (float*)malloc(sizeof(float) * (size_t)n_comp);
            for (int i = 0; i < IH * ID; ++i) qf[i] = orc_bf16_to_f32(iq[(size_t)b * IH * ID + i]);
            for (size_t i = 0; i < (size_t)n_comp * ID; ++i)
                kf[i] = orc_bf16_to_f32(ikv[(size_t)b * g->max_comp * ID + i]);
            orc_v4_index_score_blocks(qf, kf, iw + (size_t)b * IH, sc, 1, n_comp, IH, ID);
            if (score_out) memcpy(score_out + (size_t)b * g->max_comp, sc, sizeof(float) * (size_t)n_comp);
            orc_v4_scored_row(sc, n_comp, K, W, K, row + W);
            free(qf); free(kf); free(sc);
        }
    }
    /* attention: widen one sequence at a time */
    float* qf = (float*)malloc(sizeof(float) * (size_t)H * D);
    float* kf = (float*)malloc(sizeof(float) * kv_rows * D);
    float* of = (float*)malloc(sizeof(float) * (size_t)H * D);
    for (int b = 0; b < n_seqs; ++b) {
        const int n_comp = (pos[b] + 1) / g->ratio;
        const size_t live = (size_t)W + (size_t)n_comp;
        for (int i = 0; i < H * D; ++i) qf[i] = orc_bf16_to_f32(q[(size_t)b * H * D + i]);
        for (size_t i = 0; i < live * D; ++i) kf[i] = orc_bf16_to_f32(kv_cache[(size_t)b * kv_rows * D + i]);
        orc_v4_sparse_attn(qf, kf, sink, sel + (size_t)b * cols, 1, H, D, cols, g->softmax_scale, of);
        for (int i = 0; i < H * D; ++i) out[(size_t)b * H * D + i] = orc_f32_to_bf16(of[i]);
    }
    free(qf); free(kf); free(of);
}

/* ---- KV compressor, decode arm -----------------------------------------------------------------
 * crates/oracles/src/v4oracle/compress.rs:42-200 (decode branch :131-174, finish :176-200);
 * device form crates/backend/kernels/kvcompress.hip (deposit, decode, pool_row, finish_row). */
typedef struct {
    int32_t ratio, coff, d, cd, ents, rd;
    float eps;
} orc_comp_geom;

static int comp_guard(const orc_comp_geom* p) {
    if (p->ratio <= 1 || p->d <= 0 || p->rd <= 0 || p->coff < 1 || p->coff > 2) return 1001;
    if (p->rd > p->d || (p->rd & 1)) return 1002;
    if (p->cd != p->coff * p->d || p->ents != p->coff * p->ratio) return 1003;
    if (p->ents > 128) return 1004;
    if ((p->coff == 2) != (p->ratio == 4)) return 1010;
    return 0;
}

/* One decode token: score += ape[slot], then both rows land in slot (state_off + slot) of the state.
 * compress.rs:131-144. */
ORC_API int orc_v4_compress_deposit_token(const float* kv, const float* score, const float* ape, float* kv_state,
                                          float* score_state, const orc_comp_geom* p, int start_pos) {
    const int g = comp_guard(p);
    if (g) return g;
    const int slot = start_pos % p->ratio, state_off = p->coff == 2 ? p->ratio : 0;
    const size_t dst = (size_t)(state_off + slot) * p->cd;
    for (int e = 0; e < p->cd; ++e) {
        kv_state[dst + e] = kv[e];
        score_state[dst + e] = score[e] + ape[(size_t)slot * p->cd + e];
    }
    return 0;
}

/* e4m3 with round-to-nearest-even everywhere (the V4 rule: numerics.rs:45-140), as a round trip. */
static float e4m3_rne_roundtrip(float x) {
    if (x != x) return NAN;
    const float a = fabsf(x);
    const float sgn = signbit(x) ? -1.0f : 1.0f;
    if (a >= 464.0f) return sgn * 448.0f;
    if (a <= 1.0f / 1024.0f) return sgn * 0.0f;
    int e;
    (void)frexpf(a, &e);
    e -= 1;                                   /* a = 1.m * 2^e */
    const float q = e < -6 ? 1.0f / 512.0f : ldexpf(1.0f, e - 3);   /* spacing of the grid around a */
    const float r = nearbyintf(a / q) * q;   /* default rounding mode: nearest even; a / q is exact */
    return sgn * (r > 448.0f ? 448.0f : r);
}

/* fp8 block quantise-dequantise of the first n values of each row, power-of-two scale, amax floor 1e-4:
 * numerics.rs:245-285, device form crates/backend/kernels/mla.hip:319-338. src == dst allowed. */
ORC_API int orc_act_quant_f8_prefix(const float* src, float* dst, int rows, int row_stride, int n, int block) {
    if (rows <= 0 || n <= 0 || block <= 0 || row_stride < n) return 1001;
    if (src != dst && n != row_stride) return 1002;
    if (n % block) return 1004;
    for (int r = 0; r < rows; ++r)
        for (int b0 = 0; b0 < n; b0 += block) {
            const float* seg = src + (size_t)r * row_stride + b0;
            float* out = dst + (size_t)r * row_stride + b0;
            float amax = 0.0f;
            for (int i = 0; i < block; ++i) amax = fmaxf(amax, fabsf(seg[i]));
            amax = fmaxf(amax, 1e-4f);
            const float s = orc_fast_round_scale(amax, 1.0f / 448.0f);
            for (int i = 0; i < block; ++i) {
                float q = seg[i] / s;
                q = q < -448.0f ? -448.0f : (q > 448.0f ? 448.0f : q);
                out[i] = e4m3_rne_roundtrip(q) * s;
            }
        }
    return 0;
}

/* Pool the `ents` state entries into one row per feature (softmax over the ENTRY axis, entries below
 * `ratio` contribute their first d dims, the others their last d when coff == 2), bf16 store, RMSNorm
 * with bf16 store, adjacent-pair rotation of the last rd dims at the block's FIRST position, bf16 store;
 * then the overlap half of the state moves down. compress.rs:145-193. `freqs` holds (cos, sin) pairs,
 * rd/2 per position. Writes the d-wide row BEFORE the final quantisation into `out`. */
ORC_API int orc_v4_compress_decode(float* kv_state, float* score_state, const float* norm, const float* freqs,
                                   float* out, const orc_comp_geom* p, int start_pos) {
    const int g = comp_guard(p);
    if (g) return g;
    if (start_pos <= 0) return 1007;
    if ((start_pos + 1) % p->ratio != 0) return 1009;
    const int d = p->d, cd = p->cd, ents = p->ents, overlap = p->coff == 2;
    for (int e = 0; e < d; ++e) {
        float m = -INFINITY;
        for (int j = 0; j < ents; ++j) {
            const int half = (overlap && j >= p->ratio) ? d : 0;
            m = fmaxf(m, score_state[(size_t)j * cd + half + e]);
        }
        if (!isfinite(m)) { out[e] = 0.0f; continue; }
        float s = 0.0f;
        for (int j = 0; j < ents; ++j) {
            const int half = (overlap && j >= p->ratio) ? d : 0;
            s += expf(score_state[(size_t)j * cd + half + e] - m);
        }
        float acc = 0.0f;
        for (int j = 0; j < ents; ++j) {
            const int half = (overlap && j >= p->ratio) ? d : 0;
            acc += kv_state[(size_t)j * cd + half + e] * (expf(score_state[(size_t)j * cd + half + e] - m) / s);
        }
        out[e] = acc;
    }
    if (overlap) {
        const size_t n = (size_t)p->ratio * cd;
        memmove(kv_state, kv_state + n, n * sizeof(float));
        memmove(score_state, score_state + n, n * sizeof(float));
    }
    for (int e = 0; e < d; ++e) out[e] = rbf16(out[e]);
    float var = 0.0f;
    for (int e = 0; e < d; ++e) var += out[e] * out[e];
    const float rs = 1.0f / sqrtf(var / (float)d + p->eps);
    for (int e = 0; e < d; ++e) out[e] = rbf16(norm[e] * (out[e] * rs));
    const int pos = (start_pos / p->ratio) * p->ratio;
    float* seg = out + (d - p->rd);
    for (int i = 0; i < p->rd / 2; ++i) {
        const float c = freqs[(size_t)pos * p->rd + 2 * i], sn = freqs[(size_t)pos * p->rd + 2 * i + 1];
        const float a = seg[2 * i], b = seg[2 * i + 1];
        seg[2 * i] = a * c - b * sn;
        seg[2 * i + 1] = a * sn + b * c;
    }
    for (int e = 0; e < d; ++e) out[e] = rbf16(out[e]);
    return 0;
}

/* ---- KV compressor, prefill arm: crates/oracles/src/v4oracle/compress.rs:52-128 ------------------
 * kv, score: [s][cd] projected rows of a prompt that starts at position 0. */

/* State left behind by a prompt of s tokens (compress.rs:57-79): with overlap the last FULL block's rows
 * (scores + ape) become the overlap half; the s % ratio rows of the open block land from slot 0. */
ORC_API int orc_v4_compress_deposit_prefill(const float* kv, const float* score, const float* ape, float* kv_state,
                                            float* score_state, const orc_comp_geom* p, int s) {
    const int g = comp_guard(p);
    if (g) return g;
    if (s <= 0) return 1005;
    const int ratio = p->ratio, cd = p->cd, overlap = p->coff == 2;
    const int remainder = s % ratio, cutoff = s - remainder, state_off = overlap ? ratio : 0;
    if (overlap && cutoff >= ratio)
        for (int j = 0; j < ratio; ++j)
            for (int e = 0; e < cd; ++e) {
                const size_t src = (size_t)(cutoff - ratio + j) * cd + e;
                kv_state[(size_t)j * cd + e] = kv[src];
                score_state[(size_t)j * cd + e] = score[src] + ape[(size_t)j * cd + e];
            }
    for (int j = 0; j < remainder; ++j)
        for (int e = 0; e < cd; ++e) {
            const size_t src = (size_t)(cutoff + j) * cd + e, dst = (size_t)(state_off + j) * cd + e;
            kv_state[dst] = kv[src];
            score_state[dst] = score[src] + ape[(size_t)j * cd + e];
        }
    return 0;
}

/* The finish shared by both arms: bf16 store, RMSNorm + bf16, adjacent-pair rotation at `pos`, bf16. */
static void comp_finish_row(float* out, const float* norm, const float* freqs, const orc_comp_geom* p, int pos) {
    const int d = p->d;
    for (int e = 0; e < d; ++e) out[e] = rbf16(out[e]);
    float var = 0.0f;
    for (int e = 0; e < d; ++e) var += out[e] * out[e];
    const float rs = 1.0f / sqrtf(var / (float)d + p->eps);
    for (int e = 0; e < d; ++e) out[e] = rbf16(norm[e] * (out[e] * rs));
    float* seg = out + (d - p->rd);
    for (int i = 0; i < p->rd / 2; ++i) {
        const float c = freqs[(size_t)pos * p->rd + 2 * i], sn = freqs[(size_t)pos * p->rd + 2 * i + 1];
        const float a = seg[2 * i], b = seg[2 * i + 1];
        seg[2 * i] = a * c - b * sn;
        seg[2 * i + 1] = a * sn + b * c;
    }
    for (int e = 0; e < d; ++e) out[e] = rbf16(out[e]);
}

/* Blocks 0 .. nblk-1 of the prompt, each pooled over its ratio rows (second halves) and, with overlap, the
 * previous block's rows (first halves; absent for block 0), scores + ape per position within the block;
 * finished at position b * ratio. out: [nblk][d] rows before the final quantisation. compress.rs:83-128. */
ORC_API int orc_v4_compress_prefill(const float* kv, const float* score, const float* ape, const float* norm,
                                    const float* freqs, float* out, const orc_comp_geom* p, int nblk) {
    const int g = comp_guard(p);
    if (g) return g;
    if (nblk <= 0) return 1006;
    const int ratio = p->ratio, d = p->d, cd = p->cd, ents = p->ents, overlap = p->coff == 2;
    for (int b = 0; b < nblk; ++b) {
        float* row = out + (size_t)b * d;
        for (int e = 0; e < d; ++e) {
            float sc[128], kvv[128];
            int live[128];
            for (int j = 0; j < ents; ++j) {
                int sblk, src_j, half;
                live[j] = 1;
                if (!overlap) { sblk = b; src_j = j; half = 0; }
                else if (j >= ratio) { sblk = b; src_j = j - ratio; half = d; }
                else if (b > 0) { sblk = b - 1; src_j = j; half = 0; }
                else { live[j] = 0; sc[j] = -INFINITY; kvv[j] = 0.0f; continue; }
                const size_t src = (size_t)(sblk * ratio + src_j) * cd + half + e;
                kvv[j] = kv[src];
                sc[j] = score[src] + ape[(size_t)src_j * cd + half + e];
            }
            float m = -INFINITY;
            for (int j = 0; j < ents; ++j) m = fmaxf(m, sc[j]);
            if (!isfinite(m)) { row[e] = 0.0f; continue; }
            float s = 0.0f;
            for (int j = 0; j < ents; ++j) s += expf(sc[j] - m);
            float acc = 0.0f;
            for (int j = 0; j < ents; ++j) acc += kvv[j] * (expf(sc[j] - m) / s);
            row[e] = acc;
            (void)live;
        }
        comp_finish_row(row, norm, freqs, p, b * ratio);
    }
    return 0;
}
