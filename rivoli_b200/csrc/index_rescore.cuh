// Exact lightning-indexer score of LISTED tokens, in the fold order of rivoli_index_score_paged (bit-identical to it):
//   cd = left fold over d of qcode[h][d] * kcode[t][d]   (each product of two e4m3 values is exact in f32, so the fused
//        multiply-add IS the reference's acc + q * k: crates/engine/tests/indexer_kernel.rs:237-249)
//   dot = (cd * s_q[h]) * s_k[t];  term_h = (w[h] * wscale) * max(dot * dscale, 0);  score = fold over h ascending.
// A warp takes TOK tokens per pass (their loads are in flight together and they share the decoded q values), lane = head
// (index_heads <= 32), index_dim = 128 (one 4-code word per lane).
#pragma once

#include <type_traits>

#include "codec.cuh"
#include "common.cuh"

constexpr int RS_HD = 128;

// q codes of one sequence, PACKED as they lie in memory (word w of head h = its dims 4w .. 4w+3), transposed to
// [word][head] in shared memory (lane = head on both sides: no bank conflicts). qf holds (RS_HD / 4) * 32 words. The fold
// decodes a word into its four f32 values on the fly (exactly: every e4m3 value is an f32): one shared-memory load per
// four dims instead of four. All threads of the CTA call it; the caller synchronises afterwards.
__device__ __forceinline__ void rv_rescore_stage_q(const uint8_t* __restrict__ qcodes_seq, int nh, uint32_t* qf) {
    for (int e = threadIdx.x; e < 32 * (RS_HD / 4); e += blockDim.x) {
        const int h = e & 31, d4 = e >> 5;
        qf[d4 * 32 + h] = h < nh ? *reinterpret_cast<const uint32_t*>(qcodes_seq + (size_t)h * RS_HD + d4 * 4) : 0u;
    }
}

// Scores the tokens toks[0 .. ln): a pass covers WARPS * TOK of them, warp w taking positions base + w, base + WARPS + w, ...
// kf = this WARP's staging of TOK key rows as f32 (TOK * RS_HD floats). my_sq / my_wh = this lane's head scale and
// weight * wscale (0 for lanes >= nh). emit(position, score) is called by one lane per token.
template <int WARPS, int TOK, class Emit>
__device__ __forceinline__ void rv_rescore_listed(const uint32_t* toks, uint32_t ln, const uint32_t* qf, float* kf,
                                                  const int32_t* __restrict__ bt, const DsaGeom& g,
                                                  const uint8_t* __restrict__ index_pool,
                                                  const float* __restrict__ index_scale, float my_sq, float my_wh,
                                                  Emit emit) {
    static_assert(TOK <= 4, "the fold below is specialised for up to four tokens");
    constexpr int hd = RS_HD;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nh = g.index_heads, P = g.page_tokens;
    for (uint32_t base = 0; base < ln; base += WARPS * TOK) {
        if (base + warp >= ln) break;
        const int n_here = min(TOK, (int)((ln - base - warp + WARPS - 1) / WARPS));   // warp-uniform, >= 1
        uint32_t cw[TOK];
        float skv[TOK];
#pragma unroll
        for (int e = 0; e < TOK; ++e) {
            cw[e] = 0u; skv[e] = 0.0f;
            if (e < n_here) {
                const int t = (int)toks[base + e * WARPS + warp];
                int pg = bt[t / P];
                pg = (pg < 0 || pg >= g.n_pool_pages) ? 0 : pg;
                const size_t rr = (size_t)pg * P + (t & (P - 1));
                cw[e] = *reinterpret_cast<const uint32_t*>(index_pool + rr * hd + lane * 4);
                skv[e] = index_scale[rr];
            }
        }
#pragma unroll
        for (int e = 0; e < TOK; ++e) {
            const float2 x = rv_e4m3x2_to_f32x2((uint16_t)(cw[e] & 0xffff)), y = rv_e4m3x2_to_f32x2((uint16_t)(cw[e] >> 16));
            *reinterpret_cast<float4*>(kf + e * hd + lane * 4) = make_float4(x.x, x.y, y.x, y.y);
        }
        __syncwarp();
        float cd[TOK];
#pragma unroll
        for (int e = 0; e < TOK; ++e) cd[e] = 0.0f;
        auto fold = [&](auto ntok) {
            constexpr int NT = decltype(ntok)::value < TOK ? decltype(ntok)::value : TOK;
#pragma unroll 4
            for (int d = 0; d < hd; d += 4) {
                const uint32_t qc = qf[(d >> 2) * 32 + lane];
                const float2 qlo = rv_e4m3x2_to_f32x2((uint16_t)(qc & 0xffff)), qhi = rv_e4m3x2_to_f32x2((uint16_t)(qc >> 16));
                const float q0f = qlo.x, q1f = qlo.y, q2f = qhi.x, q3f = qhi.y;
#pragma unroll
                for (int e = 0; e < NT; ++e) {
                    const float4 k4 = *reinterpret_cast<const float4*>(kf + e * hd + d);   // broadcast read
                    cd[e] = fmaf(q0f, k4.x, cd[e]);
                    cd[e] = fmaf(q1f, k4.y, cd[e]);
                    cd[e] = fmaf(q2f, k4.z, cd[e]);
                    cd[e] = fmaf(q3f, k4.w, cd[e]);
                }
            }
        };
        if (n_here >= TOK) fold(std::integral_constant<int, TOK>{});
        else if (n_here == 1) fold(std::integral_constant<int, 1>{});
        else if (n_here == 2) fold(std::integral_constant<int, 2>{});
        else fold(std::integral_constant<int, 3>{});
        __syncwarp();
#pragma unroll
        for (int e = 0; e < TOK; ++e) {
            const float dot = __fmul_rn(__fmul_rn(cd[e], my_sq), skv[e]);
            float rr = __fmul_rn(dot, g.index_dscale);
            rr = rr > 0.0f ? rr : 0.0f;
            kf[e * hd + lane] = __fmul_rn(my_wh, rr);
        }
        __syncwarp();
        if (lane < n_here) {
            float acc = 0.0f;
            for (int h = 0; h < nh; ++h) acc = __fadd_rn(acc, kf[lane * hd + h]);
            emit(base + lane * WARPS + warp, acc);
        }
        __syncwarp();
    }
}
