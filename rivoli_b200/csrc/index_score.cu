// Lightning-indexer scores on CUDA cores, in the reference's exact arithmetic order.
//
//   rivoli_index_score        : the reference operator (f32 q, bf16 key slab, one sequence;
//                               crates/backend/kernels/indexer.hip:60-93).
//   rivoli_index_score_paged  : batched, paged, fp8 keys and fp8 q. Bit-reproducible:
//                               the code dot is a left fold over d (each product of two e4m3
//                               values is exact in f32, so fma(q,k,acc) IS round(acc + q*k)),
//                               scales are applied to the finished dot, heads fold ascending.
//
// The paged kernel is a register-tiled f32 "GEMM" (tokens x heads x dims) whose k-loop is
// sequential per output, which is what keeps the fold order fixed. It is the definitional
// path: ~62 FLOP per key byte means CUDA cores cannot keep up with HBM here; the
// tensor-core scorer uses this kernel's arithmetic only for the tokens near the top-k cut.
#include "codec.cuh"
#include "common.cuh"

// ------------------------------------------------------------------------------------------
// Reference layout. One warp per cached token; lanes split hd; heads fold in list order on
// lane 0 so the per-token sum has the reference's head order. The per-head dot is a
// shuffle-tree sum (the reference's own kernel also differs from its host fold here, and
// holds the comparison to 1e-5 relative: crates/engine/tests/indexer_kernel.rs:340-356).
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
index_score_slab_kernel(const float* __restrict__ q, const float* __restrict__ w,
                        const unsigned short* __restrict__ kcache, const unsigned int* __restrict__ heads,
                        int nt, int nact, int hd, float wscale, float dscale, float* __restrict__ scores) {
    extern __shared__ float kf[];  // [8 warps][hd]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * 8 + warp;
    if (t >= nt) return;
    float* krow = kf + (size_t)warp * hd;
    for (int i = lane; i < hd; i += 32) krow[i] = rv_bf16_to_f32(kcache[(size_t)t * hd + i]);
    __syncwarp();
    float acc = 0.0f;
    for (int a = 0; a < nact; ++a) {
        const int h = heads ? (int)heads[a] : a;
        const float* qh = q + (size_t)h * hd;
        float part = 0.0f;
        for (int i = lane; i < hd; i += 32) part = fmaf(qh[i], krow[i], part);
        part = rv_warp_sum(part);
        const float r = fmaxf(__fmul_rn(part, dscale), 0.0f);
        acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(w[h], wscale), r));
    }
    if (lane == 0) scores[t] = acc;
}

RIVOLI_API int rivoli_index_score(const float* q, const float* w, const unsigned short* kcache,
                                  const unsigned int* heads, int nt, int nh, int nact, int hd,
                                  float wscale, float dscale, float* scores) {
    if (nt <= 0 || nh <= 0 || nact <= 0 || nact > nh || hd <= 0) return 1001;
    // Same bounds the reference's launcher states (block = next pow2 >= nact, <= 1024;
    // staging (hd + block) floats <= 64 KiB), so the same shapes are accepted and rejected.
    int bd = 1;
    while (bd < nact) bd <<= 1;
    if (bd < 32) bd = 32;
    if (bd > 1024) return 1002;
    if (((size_t)hd + bd) * sizeof(float) > 65536) return 1002;
    const size_t smem = (size_t)8 * hd * sizeof(float);
    rv_drain_error();
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(index_score_slab_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    index_score_slab_kernel<<<(nt + 7) / 8, 256, smem>>>(q, w, kcache, heads, nt, nact, hd, wscale, dscale, scores);
    return rv_launch_status();
}

// ------------------------------------------------------------------------------------------
// Paged exact scorer. CTA = 128 threads = 128 tokens of one sequence.
//   thread (tx = tid % 32, ty = tid / 32) owns tokens 4*tx..4*tx+3 and heads ty*HPW..+HPW-1
//   dims are staged 64 at a time: kf[64][128] (token minor) and qf[64][4*HPW] (head minor)
// ------------------------------------------------------------------------------------------
constexpr int IS_TOK = 128;   // tokens per CTA
constexpr int IS_DCH = 64;    // dims per staged chunk

template <int HPW>
__global__ void __launch_bounds__(128)
index_score_paged_kernel(DsaGeom g, const uint8_t* __restrict__ qcodes, const float* __restrict__ qscales,
                         const float* __restrict__ w, const uint8_t* __restrict__ index_pool,
                         const float* __restrict__ index_scale, const int32_t* __restrict__ block_table,
                         const int32_t* __restrict__ seq_len, float* __restrict__ scores, int score_stride) {
    constexpr int NHP = 4 * HPW;  // padded head count
    constexpr int CST = NHP + 1;  // odd pitch of the per-(token, head) contribution tile
    __shared__ __align__(16) float smem[IS_DCH * IS_TOK + IS_DCH * NHP];
    float (*kf)[IS_TOK] = reinterpret_cast<float (*)[IS_TOK]>(smem);
    float (*qf)[NHP] = reinterpret_cast<float (*)[NHP]>(smem + IS_DCH * IS_TOK);
    // After the k-loop both tiles are dead: cs overlays the front, sks sits at the very end.
    float* cs = smem;
    float* sks = smem + IS_DCH * IS_TOK + IS_DCH * NHP - IS_TOK;
    static_assert(IS_TOK * CST <= IS_DCH * IS_TOK + IS_DCH * NHP - IS_TOK, "epilogue tiles overlap");
    const int b = blockIdx.y, t0 = blockIdx.x * IS_TOK, tid = threadIdx.x;
    const int nt = seq_len[b];
    if (t0 >= nt) return;
    const int nh = g.index_heads, hd = g.index_dim;
    const int tx = tid & 31, ty = tid >> 5;

    // This thread stages token t0 + tid.
    const int t = t0 + tid;
    const uint8_t* krow = nullptr;
    float sk = 0.0f;
    if (t < nt) {
        const int page = block_table[(size_t)b * g.max_pages_per_seq + t / g.page_tokens];
        const size_t r = (size_t)page * g.page_tokens + (t & (g.page_tokens - 1));
        krow = index_pool + r * hd;
        sk = index_scale[r];
    }

    float acc[4][HPW];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < HPW; ++j) acc[i][j] = 0.0f;

    for (int d0 = 0; d0 < hd; d0 += IS_DCH) {
        const int dn = min(IS_DCH, hd - d0);
        __syncthreads();
        // keys: 16 codes at a time from this thread's row
        for (int c = 0; c < dn; c += 16) {
            uint4 p = make_uint4(0, 0, 0, 0);
            if (krow) p = *reinterpret_cast<const uint4*>(krow + d0 + c);
            const uint32_t wv[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float2 a = rv_e4m3x2_to_f32x2((uint16_t)(wv[k] & 0xffff));
                float2 bq = rv_e4m3x2_to_f32x2((uint16_t)(wv[k] >> 16));
                kf[c + 4 * k + 0][tid] = a.x; kf[c + 4 * k + 1][tid] = a.y;
                kf[c + 4 * k + 2][tid] = bq.x; kf[c + 4 * k + 3][tid] = bq.y;
            }
        }
        // q: [dn][NHP], zero for padded heads
        for (int e = tid; e < dn * NHP; e += 128) {
            const int d = e / NHP, h = e % NHP;
            float v = 0.0f;
            if (h < nh) v = rv_e4m3_to_f32(qcodes[((size_t)b * nh + h) * hd + d0 + d]);
            qf[d][h] = v;
        }
        __syncthreads();
        for (int d = 0; d < dn; ++d) {
            const float4 kv = *reinterpret_cast<const float4*>(&kf[d][tx * 4]);
            float qv[HPW];
#pragma unroll
            for (int j = 0; j < HPW; j += 2) {
                const float2 q2 = *reinterpret_cast<const float2*>(&qf[d][ty * HPW + j]);
                qv[j] = q2.x; qv[j + 1] = q2.y;
            }
#pragma unroll
            for (int j = 0; j < HPW; ++j) {
                acc[0][j] = fmaf(qv[j], kv.x, acc[0][j]);
                acc[1][j] = fmaf(qv[j], kv.y, acc[1][j]);
                acc[2][j] = fmaf(qv[j], kv.z, acc[2][j]);
                acc[3][j] = fmaf(qv[j], kv.w, acc[3][j]);
            }
        }
    }
    __syncthreads();
    // Per-(token, head) contribution into smem, then a sequential fold over heads.
    sks[tid] = sk;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < HPW; ++j) {
        const int h = ty * HPW + j;
        if (h < nh) {
            const float sq = qscales[(size_t)b * nh + h];
            const float wh = __fmul_rn(w[(size_t)b * nh + h], g.index_wscale);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int tl = tx * 4 + i;
                const float dot = __fmul_rn(__fmul_rn(acc[i][j], sq), sks[tl]);
                float r = __fmul_rn(dot, g.index_dscale);
                r = r > 0.0f ? r : 0.0f;
                cs[tl * CST + h] = __fmul_rn(wh, r);
            }
        }
    }
    __syncthreads();
    if (t < nt) {
        float s = 0.0f;
        for (int h = 0; h < nh; ++h) s = __fadd_rn(s, cs[tid * CST + h]);
        scores[(size_t)b * score_stride + t] = s;
    }
}

RIVOLI_API int rivoli_index_score_paged(const DsaGeom* g, const uint8_t* qcodes, const float* qscales,
                                        const float* w, const uint8_t* index_pool,
                                        const float* index_scale, const int32_t* block_table,
                                        const int32_t* seq_len, int B, float* scores, int score_stride,
                                        void* stream) {
    if (int e = rv_check_geom(g)) return e;
    if (B <= 0 || score_stride <= 0 || !qcodes || !qscales || !w || !index_pool || !index_scale ||
        !block_table || !seq_len || !scores)
        return 1001;
    if ((uintptr_t)index_pool & 15) return 1005;
    if ((long long)score_stride > (long long)g->max_pages_per_seq * g->page_tokens) return 1002;
    dim3 grid((score_stride + IS_TOK - 1) / IS_TOK, B);
    cudaStream_t st = (cudaStream_t)stream;
    rv_drain_error();
#define RV_LAUNCH_IS(HPW)                                                                         \
    index_score_paged_kernel<HPW><<<grid, 128, 0, st>>>(*g, qcodes, qscales, w, index_pool,       \
                                                         index_scale, block_table, seq_len, scores, \
                                                         score_stride)
    if (g->index_heads <= 8) RV_LAUNCH_IS(2);
    else if (g->index_heads <= 16) RV_LAUNCH_IS(4);
    else if (g->index_heads <= 32) RV_LAUNCH_IS(8);
    else RV_LAUNCH_IS(16);
#undef RV_LAUNCH_IS
    return rv_launch_status();
}
