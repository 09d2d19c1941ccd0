// V4 cousin of the decode path, part 2: MQA sparse attention over one shared entry per position, gathered by an
// explicit index list, with a per-head sink in the softmax denominator.
// Reference behaviour: crates/backend/kernels/attn.hip:358-465.
#include "v4_common.cuh"

namespace {

// ---------------------------------------------------------------------------------------------------
// sparse attention, CUDA cores: any shape, f32 or bf16 storage. One CTA per (query row, head).
// ---------------------------------------------------------------------------------------------------
constexpr int GA_THREADS = 256;
constexpr int GA_ACC = 4;

__device__ __forceinline__ void v4_store_out(float* o, size_t i, float v) { o[i] = v4_rbf16(v); }
__device__ __forceinline__ void v4_store_out(uint16_t* o, size_t i, float v) { o[i] = rv_f32_to_bf16(v); }

template <class T>
__global__ void __launch_bounds__(GA_THREADS) v4_gather_attn_kernel(const T* __restrict__ q, const T* __restrict__ kv,
                                                                    size_t kv_row_stride_per_t,
                                                                    const float* __restrict__ sink,
                                                                    const int* __restrict__ idxs, int h, int d,
                                                                    int topk, float scale, T* __restrict__ o) {
    extern __shared__ __align__(16) float ga_smem[];
    float* qs = ga_smem;      // [d]
    float* lg = ga_smem + d;  // [topk] logits, then softmax weights
    __shared__ float red[GA_THREADS / 32];
    __shared__ float bc;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int head = blockIdx.x, t = blockIdx.y;
    const T* kvt = kv + (size_t)t * kv_row_stride_per_t;
    const int* ix = idxs + (size_t)t * topk;
    for (int i = tid; i < d; i += GA_THREADS) qs[i] = v4_load_f32(q, ((size_t)t * h + head) * d + i);
    __syncthreads();
    // logits: one warp per slot, lanes across the row
    float mx = -INFINITY;
    for (int j = warp; j < topk; j += GA_THREADS / 32) {
        const int p = ix[j];
        float l = -INFINITY;
        if (p >= 0) {
            float a = 0.0f;
            for (int i = lane; i < d; i += 32) a = fmaf(qs[i], v4_load_f32(kvt, (size_t)p * d + i), a);
            l = rv_warp_sum(a) * scale;
        }
        if (lane == 0) lg[j] = l;
        mx = fmaxf(mx, l);
    }
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int i = 1; i < GA_THREADS / 32; ++i) mx = fmaxf(mx, red[i]);
    __syncthreads();
    float ps = 0.0f;
    for (int j = tid; j < topk; j += GA_THREADS) {
        const float e = ix[j] >= 0 ? expf(lg[j] - mx) : 0.0f;
        lg[j] = e;
        ps += e;
    }
    ps = rv_warp_sum(ps);
    if (lane == 0) red[warp] = ps;
    __syncthreads();
    if (tid == 0) {
        float s = 0.0f;
        for (int i = 0; i < GA_THREADS / 32; ++i) s += red[i];
        // a query with every slot masked is made loud, not zero
        bc = isfinite(mx) ? s + expf(sink[head] - mx) : NAN;
    }
    __syncthreads();
    const float denom = bc;
    float acc[GA_ACC];
#pragma unroll
    for (int c = 0; c < GA_ACC; ++c) acc[c] = 0.0f;
    for (int j = 0; j < topk; ++j) {
        const int p = ix[j];
        if (p < 0) continue;
        const float e = lg[j];
#pragma unroll
        for (int c = 0; c < GA_ACC; ++c) {
            const int i = tid + c * GA_THREADS;
            if (i < d) acc[c] = fmaf(e, v4_load_f32(kvt, (size_t)p * d + i), acc[c]);
        }
    }
#pragma unroll
    for (int c = 0; c < GA_ACC; ++c) {
        const int i = tid + c * GA_THREADS;
        if (i < d) v4_store_out(o, ((size_t)t * h + head) * d + i, acc[c] / denom);
    }
}

// ---------------------------------------------------------------------------------------------------
// sparse attention, tensor cores: 64 heads x 512 dims, one CTA per sequence.
//
// The selected rows are gathered ONCE per sequence into shared memory (64-token tiles, two buffers,
// cp.async) and serve every head twice: as K of S = q K^T and as V of O += P V. 16 warps:
//   scores   warp (hg, tq, kh): heads 32hg..+31 x tokens 16tq..+15 over half of the 512 dims (16 k-steps of
//            m16n8k16); the two halves meet in shared memory through one add each (two addends: the sum does
//            not depend on their order);
//   softmax  8 threads per head over the tile's 64 tokens, running max / sum in registers;
//   values   warp (hg, dg): heads 32hg..+31 x dims 64dg..+63, 4 k-steps over the tile's tokens.
// Two m-tiles per warp halve the operand reloads from shared memory, which is what bounds this kernel.
// Rows are 1024 B; the 16-byte chunk c of row r sits at chunk (c ^ (r & 7)) so that the eight rows of an
// 8x8 ldmatrix tile fall in eight different bank groups.
// ---------------------------------------------------------------------------------------------------
constexpr int SA_H = 64, SA_D = 512, SA_TILE = 64, SA_THREADS = 512;
constexpr int SA_ROW_BYTES = SA_D * 2;
constexpr int SA_SQ = 0;                                   // [64 heads][1024 B]
constexpr int SA_SK = SA_SQ + SA_H * SA_ROW_BYTES;         // 2 x [64 tokens][1024 B]
constexpr int SA_SS = SA_SK + 2 * SA_TILE * SA_ROW_BYTES;  // f32 [64 heads][68]
constexpr int SA_SS_LD = 68;
constexpr int SA_SP = SA_SS + SA_H * SA_SS_LD * 4;         // bf16 [64 heads][64 tokens], chunk-swizzled
constexpr int SA_FAC = SA_SP + SA_H * SA_TILE * 2;         // f32 [64] rescale of the running output
constexpr int SA_INV = SA_FAC + SA_H * 4;                  // f32 [64] 1 / denominator
constexpr int SA_IDX = SA_INV + SA_H * 4;                  // i32 [2][64] the tile's slots
constexpr int SA_SEL = SA_IDX + 2 * SA_TILE * 4;            // i32 [SA_SEL_MAX] the sequence's selection row
constexpr int SA_SEL_MAX = 2048;
constexpr int SA_TOTAL = SA_SEL + SA_SEL_MAX * 4;


__device__ __forceinline__ uint32_t v4_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void v4_cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void v4_ldsm4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void v4_ldsm4_t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ float v4_ex2(float x) {   // 2^x, -inf -> 0; relative error 2^-22
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two f32 -> packed bf16x2 (lo = a), round to nearest even, and the two rounded values' sum.
__device__ __forceinline__ uint32_t v4_pack_bf16x2(float a, float b, float& sum) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    sum += __uint_as_float(r << 16) + __uint_as_float(r & 0xffff0000u);
    return r;
}
__device__ __forceinline__ void v4_mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(SA_THREADS, 1) v4_sparse_attend_mma_kernel(const uint16_t* __restrict__ q,
                                                                             const uint16_t* __restrict__ kv_cache,
                                                                             size_t kv_rows,
                                                                             const float* __restrict__ sink,
                                                                             const int32_t* __restrict__ sel, int cols,
                                                                             float scale_log2,
                                                                             uint16_t* __restrict__ out) {
    extern __shared__ __align__(1024) unsigned char sa_smem[];
    const int b = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t sbase = v4_smem_u32(sa_smem);
    float* sS = reinterpret_cast<float*>(sa_smem + SA_SS);
    float* sFac = reinterpret_cast<float*>(sa_smem + SA_FAC);
    float* sInv = reinterpret_cast<float*>(sa_smem + SA_INV);
    int32_t* sIdx = reinterpret_cast<int32_t*>(sa_smem + SA_IDX);
    const uint16_t* kvb = kv_cache + (size_t)b * kv_rows * SA_D;
    const int32_t* ix = sel + (size_t)b * cols;
    const int n_tiles = (cols + SA_TILE - 1) / SA_TILE;
    // chunk (row, c) -> byte offset inside a [rows][1024 B] operand
    auto swz = [](int row, int c) { return row * SA_ROW_BYTES + ((c ^ (row & 7)) << 4); };

    // chunk `it` (0..7) of this thread's share of tile t: one 16-byte piece of one row
    auto gather_piece = [&](int t, int buf, int it) {
        const int ch = tid + it * SA_THREADS, row = ch >> 6, c = ch & 63;
        const int j = t * SA_TILE + row;
        const int p = j < cols ? ix[j] : -1;
        if (c == 0) sIdx[buf * SA_TILE + row] = p;
        const int off = SA_SK + buf * SA_TILE * SA_ROW_BYTES + swz(row, c);
        if (p >= 0) v4_cp_async16(sbase + off, kvb + (size_t)p * SA_D + c * 8);
        else *reinterpret_cast<uint4*>(sa_smem + off) = make_uint4(0, 0, 0, 0);   // masked slot: a row of zeros
    };

    // Under a programmatic dependent launch the kernel before this one may still be running, and the caller
    // may have produced q with it: nothing is read before the dependency wait. Then q of this sequence, the
    // selection row and the first tile.
    rv_grid_dep_wait();
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int ch = tid + it * SA_THREADS, row = ch >> 6, c = ch & 63;
        v4_cp_async16(sbase + SA_SQ + swz(row, c), q + ((size_t)b * SA_H + row) * SA_D + c * 8);
    }
    if (cols <= SA_SEL_MAX) {   // read the row once; the per-tile gathers then take their slots from shared memory
        int32_t* sSel = reinterpret_cast<int32_t*>(sa_smem + SA_SEL);
        for (int i = tid; i < cols; i += SA_THREADS) sSel[i] = ix[i];
        ix = sSel;
        __syncthreads();
    }
#pragma unroll
    for (int it = 0; it < 8; ++it) gather_piece(0, 0, it);
    asm volatile("cp.async.commit_group;" ::: "memory");

    // softmax state of head (tid >> 3), replicated in its 8 threads
    float m_run = -INFINITY, l_run = 0.0f;
    // output accumulators of warp (hg, dg): 2 m-tiles x 8 n-tiles of 8 dims
    float acc[2][8][4];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int n = 0; n < 8; ++n) acc[m][n][0] = acc[m][n][1] = acc[m][n][2] = acc[m][n][3] = 0.0f;

    const int hg = warp & 1;                        // heads 32 hg .. +31
    const int tq = (warp >> 1) & 3, kh = warp >> 3; // scores: token quarter, half of the dims
    const int dg = warp >> 1;                       // values: dims 64 dg .. +63
    const int mi = lane >> 3, l7 = lane & 7;

    for (int t = 0; t < n_tiles; ++t) {
        const int buf = t & 1;
        if (t + 1 < n_tiles) {
#pragma unroll
            for (int it = 0; it < 8; ++it) gather_piece(t + 1, buf ^ 1, it);
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const uint32_t sK = sbase + SA_SK + buf * SA_TILE * SA_ROW_BYTES;

        // ---- scores: S[32 heads][16 tokens] over this warp's half of the dims
        {
            float sc[2][2][4];
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
                for (int n = 0; n < 2; ++n) sc[m][n][0] = sc[m][n][1] = sc[m][n][2] = sc[m][n][3] = 0.0f;
            const int arow = 32 * hg + ((mi & 1) << 3) + l7;
            const int brow = 16 * tq + ((mi >> 1) << 3) + l7;
            const int ks0 = kh * (SA_D / 32);
            uint32_t a0[2][4], a1[2][4], bb[2][4];
            v4_ldsm4(sbase + SA_SQ + swz(arow, 2 * ks0 + (mi >> 1)), a0[0]);
            v4_ldsm4(sbase + SA_SQ + swz(arow + 16, 2 * ks0 + (mi >> 1)), a1[0]);
            v4_ldsm4(sK + swz(brow, 2 * ks0 + (mi & 1)), bb[0]);
#pragma unroll
            for (int i = 0; i < SA_D / 32; ++i) {
                const int cur = i & 1, nxt = cur ^ 1, ks = ks0 + i + 1;
                if (i + 1 < SA_D / 32) {
                    v4_ldsm4(sbase + SA_SQ + swz(arow, 2 * ks + (mi >> 1)), a0[nxt]);
                    v4_ldsm4(sbase + SA_SQ + swz(arow + 16, 2 * ks + (mi >> 1)), a1[nxt]);
                    v4_ldsm4(sK + swz(brow, 2 * ks + (mi & 1)), bb[nxt]);
                }
                v4_mma_bf16(sc[0][0], a0[cur], bb[cur][0], bb[cur][1]);
                v4_mma_bf16(sc[0][1], a0[cur], bb[cur][2], bb[cur][3]);
                v4_mma_bf16(sc[1][0], a1[cur], bb[cur][0], bb[cur][1]);
                v4_mma_bf16(sc[1][1], a1[cur], bb[cur][2], bb[cur][3]);
            }
            // the two halves meet in shared memory: the lower half stores, the upper half adds (a + b: no order to pick)
            if (kh == 1) __syncthreads();
#pragma unroll
            for (int m = 0; m < 2; ++m)
#pragma unroll
                for (int n = 0; n < 2; ++n) {
                    float2* p0 = reinterpret_cast<float2*>(sS + (32 * hg + 16 * m + (lane >> 2)) * SA_SS_LD + 16 * tq + 8 * n + (lane & 3) * 2);
                    float2* p1 = p0 + 4 * SA_SS_LD;   // 8 rows down
                    if (kh == 0) {
                        *p0 = make_float2(sc[m][n][0], sc[m][n][1]);
                        *p1 = make_float2(sc[m][n][2], sc[m][n][3]);
                    } else {
                        const float2 u = *p0, v = *p1;
                        *p0 = make_float2(u.x + sc[m][n][0], u.y + sc[m][n][1]);
                        *p1 = make_float2(v.x + sc[m][n][2], v.y + sc[m][n][3]);
                    }
                }
            if (kh == 0) __syncthreads();
        }
        __syncthreads();

        // ---- softmax over the tile: head = tid / 8, tokens 8 * (tid % 8) .. +7
        {
            const int head = tid >> 3, part = tid & 7;
            float sv[8];
            const float4* srow = reinterpret_cast<const float4*>(sS + head * SA_SS_LD + part * 8);
            const float4 x0 = srow[0], x1 = srow[1];
            sv[0] = x0.x; sv[1] = x0.y; sv[2] = x0.z; sv[3] = x0.w; sv[4] = x1.x; sv[5] = x1.y; sv[6] = x1.z; sv[7] = x1.w;
#pragma unroll
            for (int j = 0; j < 8; ++j) sv[j] *= scale_log2;
            float tmax = -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (sIdx[buf * SA_TILE + part * 8 + j] < 0) sv[j] = -INFINITY;
                tmax = fmaxf(tmax, sv[j]);
            }
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
            const float m_new = fmaxf(m_run, tmax);
            const float fac = m_new == -INFINITY ? 1.0f : v4_ex2(m_run - m_new);
            const float m_use = m_new == -INFINITY ? 0.0f : m_new;    // every slot masked so far: all p are 2^-inf = 0
            uint32_t pk[4];
            float psum = 0.0f;                                         // the sum of what the value product sees
#pragma unroll
            for (int j = 0; j < 8; j += 2) pk[j >> 1] = v4_pack_bf16x2(v4_ex2(sv[j] - m_use), v4_ex2(sv[j + 1] - m_use), psum);
            psum += __shfl_xor_sync(0xffffffffu, psum, 1);
            psum += __shfl_xor_sync(0xffffffffu, psum, 2);
            psum += __shfl_xor_sync(0xffffffffu, psum, 4);
            l_run = l_run * fac + psum;
            m_run = m_new;
            *reinterpret_cast<uint4*>(sa_smem + SA_SP + head * (SA_TILE * 2) + ((part ^ (head & 7)) << 4)) =
                make_uint4(pk[0], pk[1], pk[2], pk[3]);
            if (part == 0) sFac[head] = fac;
        }
        __syncthreads();

        // ---- values: O[32 heads][64 dims] += P[32 heads][64 tokens] V[64 tokens][64 dims]
        {
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                const float f0 = sFac[32 * hg + 16 * m + (lane >> 2)], f1 = sFac[32 * hg + 16 * m + (lane >> 2) + 8];
                if (f0 != 1.0f || f1 != 1.0f) {
#pragma unroll
                    for (int n = 0; n < 8; ++n) { acc[m][n][0] *= f0; acc[m][n][1] *= f0; acc[m][n][2] *= f1; acc[m][n][3] *= f1; }
                }
            }
            const int prow = 32 * hg + ((mi & 1) << 3) + l7;
#pragma unroll
            for (int ks = 0; ks < SA_TILE / 16; ++ks) {
                uint32_t a0[4], a1[4];
                v4_ldsm4(sbase + SA_SP + prow * (SA_TILE * 2) + (((2 * ks + (mi >> 1)) ^ (prow & 7)) << 4), a0);
                v4_ldsm4(sbase + SA_SP + (prow + 16) * (SA_TILE * 2) + (((2 * ks + (mi >> 1)) ^ (prow & 7)) << 4), a1);
                const int vrow = 16 * ks + ((mi & 1) << 3) + l7;
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t bb[4];
                    v4_ldsm4_t(sK + swz(vrow, 8 * dg + 2 * np + (mi >> 1)), bb);
                    v4_mma_bf16(acc[0][2 * np], a0, bb[0], bb[1]);
                    v4_mma_bf16(acc[0][2 * np + 1], a0, bb[2], bb[3]);
                    v4_mma_bf16(acc[1][2 * np], a1, bb[0], bb[1]);
                    v4_mma_bf16(acc[1][2 * np + 1], a1, bb[2], bb[3]);
                }
            }
        }
        __syncthreads();
    }

    // the sink joins the denominator only, shifted by the same running max
    {
        const int head = tid >> 3;
        if ((tid & 7) == 0) {
            const float l = l_run + v4_ex2(sink[head] * 1.4426950408889634f - m_run);
            sInv[head] = m_run == -INFINITY ? NAN : 1.0f / l;
        }
    }
    __syncthreads();
    // bf16 output staged in the q region (q is dead after the last score pass), then whole rows go out in
    // 16-byte pieces
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        const int r0 = 32 * hg + 16 * m + (lane >> 2);
        const float i0 = sInv[r0], i1 = sInv[r0 + 8];
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            float unused = 0.0f;
            const int c = 8 * dg + n;                         // 16-byte chunk of the row: dims 8c .. 8c+7
            const int off = ((lane & 3) << 2);
            *reinterpret_cast<uint32_t*>(sa_smem + SA_SQ + swz(r0, c) + off) =
                v4_pack_bf16x2(acc[m][n][0] * i0, acc[m][n][1] * i0, unused);
            *reinterpret_cast<uint32_t*>(sa_smem + SA_SQ + swz(r0 + 8, c) + off) =
                v4_pack_bf16x2(acc[m][n][2] * i1, acc[m][n][3] * i1, unused);
        }
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int ch = tid + it * SA_THREADS, row = ch >> 6, c = ch & 63;
        *reinterpret_cast<uint4*>(out + ((size_t)b * SA_H + row) * SA_D + c * 8) =
            *reinterpret_cast<const uint4*>(sa_smem + SA_SQ + swz(row, c));
    }
}

}  // namespace


RIVOLI_API int rivoli_gather_attn_shared_kv(const float* q, const float* kv, const float* sink, const int* idxs, int m,
                                            int h, int d, int topk, float scale, float* o, void* stream) {
    if (m <= 0 || h <= 0 || d <= 0 || topk <= 0) return 1001;
    if (d > GA_THREADS * GA_ACC) return 1002;   // dims past the per-thread accumulators would never be written
    const size_t smem = ((size_t)d + (size_t)topk) * sizeof(float);
    if (smem + sizeof(float) * (GA_THREADS + 2) > 65536) return 1006;
    rv_drain_error();
    cudaFuncSetAttribute(v4_gather_attn_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    v4_gather_attn_kernel<float><<<dim3((unsigned)h, (unsigned)m), GA_THREADS, smem, (cudaStream_t)stream>>>(
        q, kv, 0, sink, idxs, h, d, topk, scale, o);
    return rv_launch_status();
}

RIVOLI_API int rivoli_v4_sparse_attend_bf16(const V4Geom* g, int n_seqs, const uint16_t* q, const uint16_t* kv_cache,
                                            const float* sink, const int32_t* sel, int cols, uint16_t* out,
                                            int force_simt, void* stream) {
    if (int rc = v4_check_geom(g, n_seqs)) return rc;
    if (cols <= 0) return 1001;
    if (g->head_dim > GA_THREADS * GA_ACC) return 1002;
    const size_t kv_rows = (size_t)g->window + (size_t)g->max_comp;
    rv_drain_error();
    cudaStream_t st = (cudaStream_t)stream;
    if (!force_simt && g->n_heads == SA_H && g->head_dim == SA_D) {
        cudaFuncSetAttribute(v4_sparse_attend_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SA_TOTAL);
        rv_launch_dependent(v4_sparse_attend_mma_kernel, dim3((unsigned)n_seqs), dim3(SA_THREADS), (size_t)SA_TOTAL, st, q,
                            kv_cache, kv_rows, sink, sel, cols, g->softmax_scale * 1.4426950408889634f, out);
        return rv_launch_status();
    }
    const size_t smem = ((size_t)g->head_dim + (size_t)cols) * sizeof(float);
    if (smem > 200 * 1024) return 1006;
    if (n_seqs > 65535) return 1002;
    cudaFuncSetAttribute(v4_gather_attn_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    v4_gather_attn_kernel<uint16_t><<<dim3((unsigned)g->n_heads, (unsigned)n_seqs), GA_THREADS, smem, st>>>(
        q, kv_cache, kv_rows * (size_t)g->head_dim, sink, sel, g->n_heads, g->head_dim, cols, g->softmax_scale, out);
    return rv_launch_status();
}
