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
#include "tc_common.cuh"

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
    int n_tiles, k_splits, cta0, tile_n;              // output tiles of tile_n columns, splits of the contraction, first CTA
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
    const int o = tile * FT_N + (threadIdx.x & 63), bq = threadIdx.x >> 6;   // this kernel always plans tile_n == FT_N
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


// ---------------------------------------------------------------------------------------------
// The same split-K GEMM on the tensor cores (tcgen05 kind::f16). CTA = (job, output tile, K split);
// M = 128 sequences, N = the tile (128, or the whole of a narrower matrix), K fed in chunks of 64
// through three shared-memory stages: activations and raw weight codes arrive by cp.async (two chunks requested
// ahead), the codes of the current chunk are converted to bf16(code * block scale) (one rounding, 2^-9 relative; a 64-wide chunk of
// a 128-aligned tile lies inside ONE scale block). The accumulator leaves as the f32 split partial.
// ---------------------------------------------------------------------------------------------
constexpr int FM_THREADS = 256, FM_WARPS = 8;
constexpr int FM_NST = 3;                      // stages of (activations 16 KiB | raw weight codes 8 KiB) in flight
constexpr int FM_STAGE = 16384 + 8192;
constexpr int FM_BOFF = FM_NST * FM_STAGE;     // two converted weight tiles (bf16, 16 KiB each) follow the stages
constexpr int FM_SMEM = FM_BOFF + 2 * 16384;   // 104 KiB: two CTAs per SM

__device__ __forceinline__ uint64_t fm_desc(uint32_t saddr) {     // K-major, 128-byte swizzle, 8-row groups 1024 B apart
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void fm_mma(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ int g_front_err;

__global__ void __launch_bounds__(FM_THREADS)
front_gemm_mma_kernel(FrontArgs A) {
    extern __shared__ __align__(1024) uint8_t fm_smem[];
    __shared__ uint64_t bar[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_word;
    volatile int* abort_flag = &abort_word;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int jid = 0;
    while (jid < 2 && (int)blockIdx.x >= A.job[jid + 1].cta0) ++jid;
    const FrontJob& J = A.job[jid];
    const int local = blockIdx.x - J.cta0;
    const int tile = local % J.n_tiles, split = local / J.n_tiles;
    const int TN = J.tile_n;
    const int kper = ((J.K + J.k_splits - 1) / J.k_splits + 127) / 128 * 128;
    const int k0 = split * kper, k1 = min(J.K, k0 + kper);
    const int nch = k1 > k0 ? (k1 - k0) / 64 : 0;
    const int sc_cols = J.K / 128;
    const float* srow = J.scale + (size_t)((tile * TN) >> 7) * sc_cols;
    if (tid == 0) { tc::mbar_init(&bar[0], 1); tc::mbar_init(&bar[1], 1); tc::mbar_init_fence(); abort_word = 0; }
    if (warp == 0) tc::tmem_alloc<128>(&tmem_slot);
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = tmem_slot;
    // instruction descriptor: bf16 x bf16 -> f32, both K-major, M = 128, N = TN
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    const uint32_t lane_base = ((uint32_t)((warp & 3) * 32)) << 16;
    const int erow = (warp & 3) * 32 + lane, chalf = warp >> 2;
    bool ok = true;
    int done[2] = {0, 0};                                   // commits issued per weight buffer so far
    for (int b0 = 0; b0 < A.B && ok; b0 += 128) {
        // request chunk c: activations (128 sequences x 64 bf16, swizzled K-major; rows past B are zeros) and
        // the raw codes of TN weight rows x 64; one cp.async group per chunk, requested chunks or not
        // per-thread copy plan, fixed for the batch tile: 4 activation rows and up to 2 weight rows per thread
        const uint16_t* pa[4]; uint32_t da[4]; bool la[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = warp * 4 + i * FM_WARPS * 4 + (lane >> 3), j = lane & 7;
            la[i] = b0 + row < A.B;
            pa[i] = J.x + (size_t)(la[i] ? b0 + row : 0) * J.K + k0 + j * 8;
            da[i] = tc::sw128_chunk(row, j);
        }
        const uint8_t* pw[2]; uint32_t dw[2]; bool lw[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int row = warp * 8 + i * FM_WARPS * 8 + (lane >> 2), j = lane & 3;
            lw[i] = row < TN;
            pw[i] = J.w + (size_t)(tile * TN + (lw[i] ? row : 0)) * J.K + k0 + j * 16;
            dw[i] = 16384 + row * 64 + j * 16;
        }
        const uint32_t smem0 = tc::smem_u32(fm_smem);
        auto request = [&](int c) {
            if (c < nch) {
                const uint32_t st = smem0 + (c % FM_NST) * FM_STAGE;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (la[i]) tc::cp_async16(st + da[i], pa[i] + c * 64);
                    else *reinterpret_cast<uint4*>(fm_smem + (c % FM_NST) * FM_STAGE + da[i]) = make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int i = 0; i < 2; ++i)
                    if (lw[i]) tc::cp_async16(st + dw[i], pw[i] + c * 64);
            }
            tc::cp_async_commit();
        };
        request(0);
        request(1);
        for (int c = 0; c < nch && ok; ++c) {
            const int wb = c & 1;
            // stage (c + 2) % 3 was read by the MMAs of chunk c - 1, weight buffer wb by those of chunk c - 2
            if (c >= 1) ok = tc::mbar_wait_warp(&bar[(c - 1) & 1], (done[(c - 1) & 1] - 1) & 1, abort_flag, 81);
            if (!ok) break;
            request(c + 2);
            tc::cp_async_wait<2>();                          // chunk c has landed (two younger groups may be pending)
            __syncthreads();
            const uint8_t* sA = fm_smem + (c % FM_NST) * FM_STAGE;
            const uint8_t* sW = sA + 16384;
            uint8_t* sB = fm_smem + FM_BOFF + wb * 16384;
            const float sc = srow[(k0 + c * 64) >> 7];
            for (int r0 = warp * 4; r0 < TN; r0 += FM_WARPS * 4) {     // codes -> bf16(code * scale), swizzled K-major
                const int row = r0 + (lane >> 3), j = lane & 7;
                const uint2 cw = *reinterpret_cast<const uint2*>(sW + row * 64 + j * 8);
                uint32_t o[4];
                const uint32_t w2[2] = {cw.x, cw.y};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = rv_e4m3x2_to_f32x2((uint16_t)(w2[i >> 1] >> (16 * (i & 1))));
                    const __nv_bfloat162 h = __floats2bfloat162_rn(f.x * sc, f.y * sc);   // finite values: plain RNE
                    o[i] = *reinterpret_cast<const uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(sB + tc::sw128_chunk(row, j)) = make_uint4(o[0], o[1], o[2], o[3]);
            }
            tc::fence_proxy_async();
            __syncthreads();
            if (tid == 0) {
                tc::tc_fence_after();
                const uint64_t da0 = fm_desc(tc::smem_u32(sA)), db0 = fm_desc(tc::smem_u32(sB));
#pragma unroll
                for (int k = 0; k < 4; ++k) fm_mma(tmem, da0 + 2 * k, db0 + 2 * k, idesc, (c | k) ? 1u : 0u);   // +32 bytes = +2 in the address field
                tc::mma_commit(&bar[wb]);
            }
            ++done[wb];
        }
        tc::cp_async_wait<0>();
        // all MMAs of this batch tile: wait for the last commit of each weight buffer
        for (int st = 0; st < 2 && ok; ++st)
            if (done[st] > 0) ok = tc::mbar_wait_warp(&bar[st], (done[st] - 1) & 1, abort_flag, 83 + st);
        tc::tc_fence_after();
        if (ok && nch > 0) {
            const int ncol_chunks = TN / 32;                 // 32-column chunks; warps 0-3 take the even ones, 4-7 the odd
            for (int c = chalf; c < ncol_chunks; c += 2) {
                uint32_t r[32];
                tc::tmem_ld32(tmem + lane_base + c * 32, r);
                tc::tmem_ld_wait();
                if (b0 + erow < A.B) {
                    float4* dst = reinterpret_cast<float4*>(J.partial + ((size_t)split * A.B + b0 + erow) * J.N + tile * TN + c * 32);
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        dst[e] = make_float4(__uint_as_float(r[4 * e]), __uint_as_float(r[4 * e + 1]), __uint_as_float(r[4 * e + 2]),
                                             __uint_as_float(r[4 * e + 3]));
                }
            }
        } else if (ok) {                                     // an empty K range (more splits than 128-blocks): zeros
            for (int e = tid; e < 128 * TN; e += FM_THREADS) {
                const int row = e / TN, col = e - row * TN;
                if (b0 + row < A.B) J.partial[((size_t)split * A.B + b0 + row) * J.N + tile * TN + col] = 0.0f;
            }
        }
        tc::tc_fence_before();
        __syncthreads();
    }
    if (warp == 0) tc::tmem_dealloc<128>(tmem);
    if (tid == 0 && abort_word) atomicCAS(&g_front_err, 0, abort_word);
}

struct EpiArgs {
    const float* pk; const float* pq; const float* pw;   // partials [splits][B][N]
    int sk, sq, sw;                                       // split counts
    const float* kn_w; const float* kn_b; const int32_t* pos;
    int B, nh, hd, rope_off, rope_seg; double theta; float eps;
    uint16_t* index_key; uint16_t* index_q; float* index_w;
};

// One CTA per sequence: reduce the split partials in split order, LayerNorm the key, rotate key and
// queries at the sequence's position, store bf16 (and the f32 head weights). The rotation angles depend
// only on (position, pair index): rope_seg / 2 (cos, sin) pairs are computed once in f64 and shared by
// all index_heads + 1 vectors.
__global__ void __launch_bounds__(256)
front_epilogue_kernel(EpiArgs A) {
    extern __shared__ float fe_smem[];          // (nh + 1) * hd values: queries then key
    __shared__ double ss[256], sq[256];
    __shared__ float s_cs[512], s_sn[512];
    const int b = blockIdx.x, t = threadIdx.x, nh = A.nh, hd = A.hd;
    float* qv = fe_smem;
    float* kv = fe_smem + (size_t)nh * hd;
    const int half = A.rope_seg / 2, pos = A.pos[b];
    for (int j = t; j < half; j += 256) {
        const double ang = (double)pos * pow(A.theta, -2.0 * (double)j / (double)A.rope_seg);
        s_cs[j] = (float)cos(ang); s_sn[j] = (float)sin(ang);
    }
    const int nq4 = nh * hd / 4;                 // index_dim is a multiple of 4 (checked by the launcher)
    for (int e0 = t; e0 < nq4; e0 += 256 * 4) {      // four elements x up to eight splits of loads in flight per thread
        float4 a[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) a[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < A.sq; s0 += 8) {
            float4 p[4][8];
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    const int e = e0 + u * 256;
                    p[u][s] = (e < nq4 && s0 + s < A.sq)
                                  ? *reinterpret_cast<const float4*>(A.pq + ((size_t)(s0 + s) * A.B + b) * nh * hd + e * 4)
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int s = 0; s < 8; ++s)
                    if (s0 + s < A.sq) {            // split order; the guard keeps "+ 0" out of the fold
                        a[u].x = __fadd_rn(a[u].x, p[u][s].x); a[u].y = __fadd_rn(a[u].y, p[u][s].y);
                        a[u].z = __fadd_rn(a[u].z, p[u][s].z); a[u].w = __fadd_rn(a[u].w, p[u][s].w);
                    }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (e0 + u * 256 < nq4) *reinterpret_cast<float4*>(qv + (e0 + u * 256) * 4) = a[u];
    }
    double s1 = 0.0, s2 = 0.0;
    for (int e = t; e < hd; e += 256) {
        float a = 0.0f;
        for (int s0 = 0; s0 < A.sk; s0 += 8) {       // eight loads in flight, folded in split order
            float p[8];
#pragma unroll
            for (int s = 0; s < 8; ++s) p[s] = s0 + s < A.sk ? A.pk[((size_t)(s0 + s) * A.B + b) * hd + e] : 0.0f;
#pragma unroll
            for (int s = 0; s < 8; ++s)
                if (s0 + s < A.sk) a = __fadd_rn(a, p[s]);
        }
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
    // rotation: (nh + 1) segments of rope_seg at rope_off; every pair is read into registers before any write
    const int npairs = (nh + 1) * half;
    float lo[8], hi[8];
    int cnt = 0;
    for (int p = t; p < npairs && cnt < 8; p += 256, ++cnt) {
        const int seg = p / half, j = p - seg * half;
        const float* v = fe_smem + (size_t)seg * hd + A.rope_off;
        const float a = v[2 * j], c = v[2 * j + 1], cs = s_cs[j], sn = s_sn[j];
        lo[cnt] = __fsub_rn(__fmul_rn(a, cs), __fmul_rn(c, sn));
        hi[cnt] = __fadd_rn(__fmul_rn(c, cs), __fmul_rn(a, sn));
    }
    __syncthreads();
    cnt = 0;
    for (int p = t; p < npairs && cnt < 8; p += 256, ++cnt) {
        const int seg = p / half, j = p - seg * half;
        float* v = fe_smem + (size_t)seg * hd + A.rope_off;
        v[j] = lo[cnt]; v[half + j] = hi[cnt];
    }
    __syncthreads();
    for (int e = t; e < nh * hd / 2; e += 256) {   // two values per 32-bit store
        const uint32_t w2 = (uint32_t)rv_f32_to_bf16(qv[2 * e]) | ((uint32_t)rv_f32_to_bf16(qv[2 * e + 1]) << 16);
        reinterpret_cast<uint32_t*>(A.index_q + (size_t)b * nh * hd)[e] = w2;
    }
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

// The tensor-core GEMM covers: 128-blocks, contraction lengths that are multiples of 128, output counts that
// are multiples of 128 (tiled) or of 16 up to 128 (one tile), 16-byte aligned rows.
static bool front_mma_ok(const IndexFrontGeom* g) {
    const int N[3] = {g->index_dim, g->index_heads * g->index_dim, g->index_heads};
    const int K[3] = {g->hidden, g->q_lora, g->hidden};
    if (g->block != 128) return false;
    for (int j = 0; j < 3; ++j) {
        if (K[j] % 128) return false;
        if (N[j] % 16 || (N[j] > 128 && N[j] % 128)) return false;
    }
    return true;
}

static void plan_jobs(const IndexFrontGeom* g, int B, bool mma, FrontArgs* fa, size_t* floats) {
    const int N[3] = {g->index_dim, g->index_heads * g->index_dim, g->index_heads};
    const int K[3] = {g->hidden, g->q_lora, g->hidden};
    int cta = 0;
    size_t off = 0;
    for (int j = 0; j < 3; ++j) {
        FrontJob& J = fa->job[j];
        J.N = N[j]; J.K = K[j];
        J.tile_n = mma ? (N[j] < 128 ? N[j] : 128) : FT_N;
        J.n_tiles = ceil_div(N[j], J.tile_n);
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
    plan_jobs(g, B, front_mma_ok(g), &fa, &floats);   // the split count does not depend on the path
    return floats * sizeof(float);
}

RIVOLI_API int rivoli_index_frontend_bf16(const IndexFrontGeom* g, const uint16_t* x, const uint16_t* q_resid,
                                          const int32_t* pos, int B, const unsigned char* wk, const float* wk_scale,
                                          const float* knorm_w, const float* knorm_b, const unsigned char* wq_b,
                                          const float* wq_b_scale, const unsigned char* wproj,
                                          const float* wproj_scale, uint16_t* index_key, uint16_t* index_q,
                                          float* index_w, void* scratch, int force_simt, void* stream) {
    if (!g || B <= 0 || !x || !q_resid || !pos || !wk || !wk_scale || !knorm_w || !knorm_b || !wq_b || !wq_b_scale ||
        !wproj || !wproj_scale || !index_key || !index_q || !index_w || !scratch)
        return 1001;
    if (g->hidden <= 0 || g->q_lora <= 0 || g->index_heads <= 0 || g->index_dim <= 0 || g->block <= 0) return 1001;
    if (g->block & (g->block - 1)) return 1003;
    if (g->rope_seg <= 0 || (g->rope_seg & 1) || g->rope_off < 0 || g->rope_off + g->rope_seg > g->index_dim) return 1002;
    if (g->index_heads > 256 || (size_t)(g->index_heads + 1) * g->index_dim * 4 > 200 * 1024) return 1002;
    if ((g->index_heads + 1) * (g->rope_seg / 2) > 8 * 256 || g->rope_seg > 1024 || (g->index_dim & 3)) return 1002;
    cudaStream_t st = (cudaStream_t)stream;
    const bool mma = !force_simt && front_mma_ok(g) && (((uintptr_t)x | (uintptr_t)q_resid | (uintptr_t)wk | (uintptr_t)wq_b |
                                                         (uintptr_t)wproj | (uintptr_t)scratch) & 15) == 0;
    FrontArgs fa;
    size_t floats = 0;
    plan_jobs(g, B, mma, &fa, &floats);
    float* base = static_cast<float*>(scratch);
    const uint16_t* xs[3] = {x, q_resid, x};
    const unsigned char* ws[3] = {wk, wq_b, wproj};
    const float* ss[3] = {wk_scale, wq_b_scale, wproj_scale};
    for (int j = 0; j < 3; ++j) {
        fa.job[j].x = xs[j]; fa.job[j].w = ws[j]; fa.job[j].scale = ss[j];
        fa.job[j].partial = base + reinterpret_cast<size_t>(fa.job[j].partial);
    }
    rv_drain_error();
    if (mma) {
        cudaFuncSetAttribute(front_gemm_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FM_SMEM);
        front_gemm_mma_kernel<<<fa.n_cta, FM_THREADS, FM_SMEM, st>>>(fa);
    } else {
        front_gemm_simt_kernel<<<fa.n_cta, 256, 0, st>>>(fa);
    }
    if (int e = rv_launch_status()) return e;
    EpiArgs ea{fa.job[0].partial, fa.job[1].partial, fa.job[2].partial, fa.job[0].k_splits, fa.job[1].k_splits,
               fa.job[2].k_splits, knorm_w, knorm_b, pos, B, g->index_heads, g->index_dim, g->rope_off, g->rope_seg,
               g->theta, g->eps, index_key, index_q, index_w};
    const size_t smem = (size_t)(g->index_heads + 1) * g->index_dim * sizeof(float);
    cudaFuncSetAttribute(front_epilogue_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    front_epilogue_kernel<<<B, 256, smem, st>>>(ea);
    return rv_launch_status();
}

// Synchronises the stream; 1008 if a bounded wait of the tensor-core front end gave up since the last call.
RIVOLI_API int rivoli_index_frontend_status(void* stream) {
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return -(int)e;
    int h = 0;
    e = cudaMemcpyFromSymbol(&h, g_front_err, sizeof(int));
    if (e != cudaSuccess) return -(int)e;
    if (h) { const int z = 0; cudaMemcpyToSymbol(g_front_err, &z, sizeof(int)); }
    return h ? 1008 : 0;
}

