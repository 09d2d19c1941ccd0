// Indexer front end: the operators that produce what the lightning indexer consumes,
//   k   = rope(layernorm(wk . x))            index key    (crates/backend/kernels/indexer.hip:1-13)
//   q_h = rope((wq_b . q_resid)[h])           index queries
//   w   = weights_proj . x                    head weights
// with wk / wq_b / weights_proj fp8-e4m3 block-scaled.
//
//   rivoli_gemv_fp8, rivoli_layernorm, rivoli_rope_interleave : the reference's single-token f32
//       operators (linalg.hip:324-342, indexer.hip:22-50,259-266, activation.hip:337-371,551-559), same
//       arguments and guards. The GEMV folds in the order of the reference's host arithmetic
//       (crates/artifact/src/quant/fp8.rs:32-42), bit for bit.
//   rivoli_index_frontend_bf16 : the batched decode form - three block-scaled GEMMs over the batch
//       written as split-K partial sums (deterministic: a fixed split, summed in order), then one
//       per-sequence epilogue kernel that reduces the partials, applies LayerNorm to the key, rotates
//       key and queries at the sequence's position and stores bf16 - the rows rivoli_kv_append_paged and
//       rivoli_index_select_paged take.
#include "codec.cuh"
#include "common.cuh"

namespace {

__device__ __forceinline__ int if_shift(int block) { return 31 - __clz(block); }

template <int R>
__global__ void __launch_bounds__(256)
gemv_fp8_kernel(const float* __restrict__ x, const uint8_t* __restrict__ packed, const float* __restrict__ scale,
                int o_dim, int i_dim, int block, float* __restrict__ y) {
    const int o = blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= o_dim) return;
    const int bsh = if_shift(block), sc_cols = (i_dim + block - 1) / block;
    const uint8_t* row = packed + (size_t)o * i_dim;
    const float* srow = scale + (size_t)(o >> bsh) * sc_cols;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;
    for (int i = 0; i < i_dim; ++i) {
        const float ws = __fmul_rn(rv_e4m3_to_f32(row[i]), srow[i >> bsh]);
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = __fadd_rn(acc[r], __fmul_rn(ws, x[(size_t)r * i_dim + i]));
    }
#pragma unroll
    for (int r = 0; r < R; ++r) y[(size_t)r * o_dim + o] = acc[r];
}

// One block; sums in f64 (the reference's host test removes the summation-order error the same way),
// then the reference's f32 formula with var = E[x^2] - mean^2.
__global__ void __launch_bounds__(256)
layernorm_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b, int n,
                 float eps, float* __restrict__ y) {
    __shared__ double ss[256], sq[256];
    const int t = threadIdx.x;
    double s = 0.0, q = 0.0;
    for (int i = t; i < n; i += 256) { const double v = (double)x[i]; s += v; q += v * v; }
    ss[t] = s; sq[t] = q;
    __syncthreads();
    for (int st = 128; st > 0; st >>= 1) {
        if (t < st) { ss[t] += ss[t + st]; sq[t] += sq[t + st]; }
        __syncthreads();
    }
    const float mean = (float)(ss[0] / (double)n);
    const float var = __fsub_rn((float)(sq[0] / (double)n), __fmul_rn(mean, mean));
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, eps)));
    for (int i = t; i < n; i += 256) y[i] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(x[i], mean), inv), w[i]), b[i]);
}

__device__ __forceinline__ void rope_pair(float a, float b, int j, int seg, int pos, double theta, float* lo, float* hi) {
    const double ang = (double)pos * pow(theta, -2.0 * (double)j / (double)seg);
    const float cs = (float)cos(ang), sn = (float)sin(ang);
    *lo = __fsub_rn(__fmul_rn(a, cs), __fmul_rn(b, sn));
    *hi = __fadd_rn(__fmul_rn(b, cs), __fmul_rn(a, sn));
}

__global__ void rope_interleave_kernel(float* __restrict__ base, int stride, int seg, int pos, double theta) {
    const int s = blockIdx.x, j = threadIdx.x, half = seg / 2;
    float* v = base + (size_t)s * stride;
    const float a = v[2 * j], b = v[2 * j + 1];
    __syncthreads();   // every pair is read before any element is written: in place, race free
    rope_pair(a, b, j, seg, pos, theta, &v[j], &v[half + j]);
}

// ---------------------------------------------------------------------------------------------
// Batched front end.
// ---------------------------------------------------------------------------------------------
struct FrontJob {            // Y[b][o] (+)= sum over a K range of X[b][i] * W[o][i] * scale
    const uint16_t* x; int K;                         // activations bf16 [B][K]
    const uint8_t* w; const float* scale; int N;      // weights e4m3 [N][K], block scales
    float* partial;                                   // f32 [k_splits][B][N]
    int n_tiles, k_splits, cta0;                      // tiles of 64 outputs, splits of the contraction, first CTA
};
struct FrontArgs { FrontJob job[3]; int B, block, n_cta; };

// CUDA-core split-K GEMM: CTA = (job, 64-output tile, K split), 256 threads = 64 outputs x 4 sequence
// groups; thread (o, g) folds its K range for sequences g, g + 4, ... (32 accumulators per pass of 128
// sequences). The weights of a 128-wide K chunk are staged dequantised in shared memory once per CTA;
// activations stream from L2. Works for any geometry.
constexpr int FT_N = 64, FT_KC = 128;
__global__ void __launch_bounds__(256)
front_gemm_simt_kernel(FrontArgs A) {
    __shared__ float ws[FT_KC][FT_N + 1];
    int jid = 0;
    while (jid < 2 && (int)blockIdx.x >= A.job[jid + 1].cta0) ++jid;
    const FrontJob& J = A.job[jid];
    const int local = blockIdx.x - J.cta0;
    const int tile = local % J.n_tiles, split = local / J.n_tiles;
    const int kper = ((J.K + J.k_splits - 1) / J.k_splits + FT_KC - 1) / FT_KC * FT_KC;
    const int k0 = split * kper, k1 = min(J.K, k0 + kper);
    const int o = tile * FT_N + (threadIdx.x & 63), bq = threadIdx.x >> 6;
    const int bsh = if_shift(A.block), sc_cols = (J.K + A.block - 1) / A.block;
    // sequences bq, bq + 4, ... ; at most 32 accumulators per thread per pass
    for (int b0 = 0; b0 < A.B; b0 += 128) {
        float acc[32];
#pragma unroll
        for (int r = 0; r < 32; ++r) acc[r] = 0.0f;
        for (int kc = k0; kc < k1; kc += FT_KC) {
            __syncthreads();
            for (int e = threadIdx.x; e < FT_KC * FT_N; e += 256) {
                const int kk = e % FT_KC, oo = e / FT_KC, i = kc + kk, og = tile * FT_N + oo;
                float v = 0.0f;
                if (i < k1 && og < J.N) v = __fmul_rn(rv_e4m3_to_f32(J.w[(size_t)og * J.K + i]), J.scale[(size_t)(og >> bsh) * sc_cols + (i >> bsh)]);
                ws[kk][oo] = v;
            }
            __syncthreads();
            const int kn = min(FT_KC, k1 - kc);
#pragma unroll
            for (int r = 0; r < 32; ++r) {
                const int b = b0 + bq + 4 * r;
                if (b < A.B) {
                    const uint16_t* xr = J.x + (size_t)b * J.K + kc;
                    float a = acc[r];
                    for (int kk = 0; kk < kn; ++kk) a = __fadd_rn(a, __fmul_rn(ws[kk][threadIdx.x & 63], rv_bf16_to_f32(xr[kk])));
                    acc[r] = a;
                }
            }
        }
        if (o < J.N)
#pragma unroll
            for (int r = 0; r < 32; ++r) {
                const int b = b0 + bq + 4 * r;
                if (b < A.B) J.partial[((size_t)split * A.B + b) * J.N + o] = acc[r];
            }
    }
}

struct EpiArgs {
    const float* pk; const float* pq; const float* pw;   // partials [splits][B][N]
    int sk, sq, sw;                                       // split counts
    const float* kn_w; const float* kn_b; const int32_t* pos;
    int B, nh, hd, rope_off, rope_seg; double theta; float eps;
    uint16_t* index_key; uint16_t* index_q; float* index_w;
};

// One CTA per sequence: reduce the split partials in split order, LayerNorm the key, rotate key and
// queries at the sequence's position, store bf16 (and the f32 head weights).
__global__ void __launch_bounds__(256)
front_epilogue_kernel(EpiArgs A) {
    extern __shared__ float fe_smem[];          // (nh + 1) * hd values: queries then key
    __shared__ double ss[256], sq[256];
    const int b = blockIdx.x, t = threadIdx.x, nh = A.nh, hd = A.hd;
    float* qv = fe_smem;
    float* kv = fe_smem + (size_t)nh * hd;
    for (int e = t; e < nh * hd; e += 256) {
        float a = 0.0f;
        for (int s = 0; s < A.sq; ++s) a = __fadd_rn(a, A.pq[((size_t)s * A.B + b) * nh * hd + e]);
        qv[e] = a;
    }
    double s1 = 0.0, s2 = 0.0;
    for (int e = t; e < hd; e += 256) {
        float a = 0.0f;
        for (int s = 0; s < A.sk; ++s) a = __fadd_rn(a, A.pk[((size_t)s * A.B + b) * hd + e]);
        kv[e] = a;
        s1 += (double)a; s2 += (double)a * (double)a;
    }
    if (t < nh) {
        float a = 0.0f;
        for (int s = 0; s < A.sw; ++s) a = __fadd_rn(a, A.pw[((size_t)s * A.B + b) * nh + t]);
        A.index_w[(size_t)b * nh + t] = a;
    }
    ss[t] = s1; sq[t] = s2;
    __syncthreads();
    for (int st = 128; st > 0; st >>= 1) {
        if (t < st) { ss[t] += ss[t + st]; sq[t] += sq[t + st]; }
        __syncthreads();
    }
    const float mean = (float)(ss[0] / (double)hd);
    const float var = __fsub_rn((float)(sq[0] / (double)hd), __fmul_rn(mean, mean));
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, A.eps)));
    for (int e = t; e < hd; e += 256)
        kv[e] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(kv[e], mean), inv), A.kn_w[e]), A.kn_b[e]);
    __syncthreads();
    // rotation: (nh + 1) segments of rope_seg at rope_off; pairs are read into registers first
    const int half = A.rope_seg / 2, pos = A.pos[b];
    const int npairs = (nh + 1) * half;
    float lo[8], hi[8];
    int cnt = 0;
    for (int p = t; p < npairs && cnt < 8; p += 256, ++cnt) {
        const int seg = p / half, j = p - seg * half;
        const float* v = fe_smem + (size_t)seg * hd + A.rope_off;
        rope_pair(v[2 * j], v[2 * j + 1], j, A.rope_seg, pos, A.theta, &lo[cnt], &hi[cnt]);
    }
    __syncthreads();
    cnt = 0;
    for (int p = t; p < npairs && cnt < 8; p += 256, ++cnt) {
        const int seg = p / half, j = p - seg * half;
        float* v = fe_smem + (size_t)seg * hd + A.rope_off;
        v[j] = lo[cnt]; v[half + j] = hi[cnt];
    }
    __syncthreads();
    for (int e = t; e < nh * hd; e += 256) A.index_q[(size_t)b * nh * hd + e] = rv_f32_to_bf16(qv[e]);
    for (int e = t; e < hd; e += 256) A.index_key[(size_t)b * hd + e] = rv_f32_to_bf16(kv[e]);
}

int ceil_div(int a, int b) { return (a + b - 1) / b; }

}  // namespace

RIVOLI_API int rivoli_gemv_fp8(const float* x, const unsigned char* packed, const float* scale, int o_dim, int i_dim,
                               int block, int nrow, float* y) {
    if (o_dim <= 0 || i_dim <= 0 || block <= 0) return 1001;
    if (block & (block - 1)) return 1003;
    if (nrow != 1 && nrow != 2) return 1004;
    rv_drain_error();
    if (nrow == 2) gemv_fp8_kernel<2><<<ceil_div(o_dim, 256), 256>>>(x, packed, scale, o_dim, i_dim, block, y);
    else gemv_fp8_kernel<1><<<ceil_div(o_dim, 256), 256>>>(x, packed, scale, o_dim, i_dim, block, y);
    return rv_launch_status();
}

// The reference switches to a split-K kernel for long rows (linalg.hip:296-321); here both names run the
// same fold, so their results are identical.
RIVOLI_API int rivoli_gemv_fp8_splitk(const float* x, const unsigned char* packed, const float* scale, int o_dim,
                                      int i_dim, int block, int nrow, float* y) {
    return rivoli_gemv_fp8(x, packed, scale, o_dim, i_dim, block, nrow, y);
}

RIVOLI_API int rivoli_layernorm(const float* x, const float* w, const float* b, int n, float eps, float* y) {
    if (n <= 0) return 1001;
    rv_drain_error();
    layernorm_kernel<<<1, 256>>>(x, w, b, n, eps, y);
    return rv_launch_status();
}

RIVOLI_API int rivoli_rope_interleave(float* base, int count, int stride, int seg, int pos, double theta) {
    if (count <= 0 || seg <= 0 || (seg & 1) || (seg / 2) > 1024) return 1001;
    if (count > 1 && stride < seg) return 1001;
    rv_drain_error();
    rope_interleave_kernel<<<count, seg / 2>>>(base, stride, seg, pos, theta);
    return rv_launch_status();
}

static void plan_jobs(const IndexFrontGeom* g, int B, FrontArgs* fa, size_t* floats) {
    const int N[3] = {g->index_dim, g->index_heads * g->index_dim, g->index_heads};
    const int K[3] = {g->hidden, g->q_lora, g->hidden};
    int cta = 0;
    size_t off = 0;
    for (int j = 0; j < 3; ++j) {
        FrontJob& J = fa->job[j];
        J.N = N[j]; J.K = K[j];
        J.n_tiles = ceil_div(N[j], FT_N);
        // enough CTAs to fill the machine, at least 256 contraction values per split, at most 32 splits
        int splits = ceil_div(296, J.n_tiles * 3);
        if (splits > K[j] / 256) splits = K[j] / 256;
        if (splits > 32) splits = 32;
        if (splits < 1) splits = 1;
        J.k_splits = splits;
        J.cta0 = cta;
        cta += J.n_tiles * splits;
        J.partial = reinterpret_cast<float*>(off);   // offset for now, rebased by the caller
        off += (size_t)splits * B * N[j];
    }
    fa->n_cta = cta; fa->B = B; fa->block = g->block;
    *floats = off;
}

RIVOLI_API size_t rivoli_index_frontend_scratch_bytes(const IndexFrontGeom* g, int B) {
    if (!g || B <= 0) return 0;
    FrontArgs fa;
    size_t floats = 0;
    plan_jobs(g, B, &fa, &floats);
    return floats * sizeof(float);
}

RIVOLI_API int rivoli_index_frontend_bf16(const IndexFrontGeom* g, const uint16_t* x, const uint16_t* q_resid,
                                          const int32_t* pos, int B, const unsigned char* wk, const float* wk_scale,
                                          const float* knorm_w, const float* knorm_b, const unsigned char* wq_b,
                                          const float* wq_b_scale, const unsigned char* wproj,
                                          const float* wproj_scale, uint16_t* index_key, uint16_t* index_q,
                                          float* index_w, void* scratch, void* stream) {
    if (!g || B <= 0 || !x || !q_resid || !pos || !wk || !wk_scale || !knorm_w || !knorm_b || !wq_b || !wq_b_scale ||
        !wproj || !wproj_scale || !index_key || !index_q || !index_w || !scratch)
        return 1001;
    if (g->hidden <= 0 || g->q_lora <= 0 || g->index_heads <= 0 || g->index_dim <= 0 || g->block <= 0) return 1001;
    if (g->block & (g->block - 1)) return 1003;
    if (g->rope_seg <= 0 || (g->rope_seg & 1) || g->rope_off < 0 || g->rope_off + g->rope_seg > g->index_dim) return 1002;
    if (g->index_heads > 256 || (size_t)(g->index_heads + 1) * g->index_dim * 4 > 200 * 1024) return 1002;
    if ((g->index_heads + 1) * (g->rope_seg / 2) > 8 * 256) return 1002;
    cudaStream_t st = (cudaStream_t)stream;
    FrontArgs fa;
    size_t floats = 0;
    plan_jobs(g, B, &fa, &floats);
    float* base = static_cast<float*>(scratch);
    const uint16_t* xs[3] = {x, q_resid, x};
    const unsigned char* ws[3] = {wk, wq_b, wproj};
    const float* ss[3] = {wk_scale, wq_b_scale, wproj_scale};
    for (int j = 0; j < 3; ++j) {
        fa.job[j].x = xs[j]; fa.job[j].w = ws[j]; fa.job[j].scale = ss[j];
        fa.job[j].partial = base + reinterpret_cast<size_t>(fa.job[j].partial);
    }
    rv_drain_error();
    front_gemm_simt_kernel<<<fa.n_cta, 256, 0, st>>>(fa);
    if (int e = rv_launch_status()) return e;
    EpiArgs ea{fa.job[0].partial, fa.job[1].partial, fa.job[2].partial, fa.job[0].k_splits, fa.job[1].k_splits,
               fa.job[2].k_splits, knorm_w, knorm_b, pos, B, g->index_heads, g->index_dim, g->rope_off, g->rope_seg,
               g->theta, g->eps, index_key, index_q, index_w};
    const size_t smem = (size_t)(g->index_heads + 1) * g->index_dim * sizeof(float);
    cudaFuncSetAttribute(front_epilogue_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    front_epilogue_kernel<<<B, 256, smem, st>>>(ea);
    return rv_launch_status();
}
