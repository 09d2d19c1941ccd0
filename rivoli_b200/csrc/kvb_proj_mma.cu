// Batched kv_b projections on the tensor cores (tcgen05, kind::f16: bf16 x bf16 -> f32).
//
// kv_b holds e4m3 codes with one f32 scale per 128 x 128 block. An e4m3 code is exactly a bf16
// number, so the codes go to shared memory as bf16 (converted on the way in) and the activations
// stay bf16: every product in the MMA is exact. The block scale cannot ride inside the MMA, so each
// run of the contraction with ONE scale gets its own TMEM accumulator and the epilogue adds the
// runs in f32: out = sum_run scale_run * D_run.
//
//   absorb: q_abs[b][h][i] = sum_d q[b][h][d] * kvb[448 h + d][i]         M = 128 sequences, N = 128 of the
//           512 latent columns (one scale column), K = nope = 192 = two runs (the head's rows straddle one
//           block boundary); CTA = (column block, head); weights are the MN-major B operand.
//   value:  ctx[b][h][j]  = sum_i o[b][h][i] * kvb[448 h + 192 + j][i]     M = 128 sequences, N = 64 of the 256
//           value rows (one scale row), K = kvl = 512 = four runs (one per scale column); CTA = (row block,
//           head); weights are the K-major B operand.
// Geometry outside these shapes takes the CUDA-core kernels of kvb_proj.cu.
// All waits are bounded (tc_common.cuh); a wait that gives up sets g_kp_err (rivoli_kvb_proj_status).
#include "codec.cuh"
#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int KP_THREADS = 128;
__device__ int g_kp_err;

__device__ __forceinline__ uint64_t kp_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;   // 128-byte swizzle
    return d;
}
// Instruction descriptor, kind::f16: bf16 x bf16 -> f32.
__device__ __forceinline__ uint32_t kp_idesc(int M, int N, int b_mn_major) {
    uint32_t d = 0;
    d |= 1u << 4;                      // accumulator f32
    d |= 1u << 7;                      // A = bf16
    d |= 1u << 10;                     // B = bf16
    d |= (uint32_t)b_mn_major << 16;   // A is always K-major here
    d |= (uint32_t)(N >> 3) << 17;
    d |= (uint32_t)(M >> 4) << 24;
    return d;
}
__device__ __forceinline__ void kp_mma(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// 8 e4m3 codes -> 8 bf16 (exact), as one 16-byte chunk.
__device__ __forceinline__ uint4 kp_codes_to_bf16(uint2 c) {
    uint32_t o[4];
    const uint32_t w[2] = {c.x, c.y};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint16_t pair = (uint16_t)(w[i >> 1] >> (16 * (i & 1)));
        const float2 f = rv_e4m3x2_to_f32x2(pair);
        o[i] = (__float_as_uint(f.x) >> 16) | (__float_as_uint(f.y) & 0xffff0000u);   // exact: 3 mantissa bits
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

struct KpArgs {
    const uint16_t* x;      // activations [B][H][xs] bf16 (xs = row pitch per head)
    const uint8_t* kvb; const float* scale;
    int H, xs, nope, vh, kvl, rope, block, B;
    uint16_t* out;
};

// ---------------------------------------------------------------------------------------------
// absorb: grid (kvl / 128, H), 128 threads. Shared: A [nope/64][128 rows][128 B] | B [2][nope][128 B].
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(KP_THREADS)
kvb_absorb_mma_kernel(KpArgs A) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_word;
    volatile int* abort_flag = &abort_word;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int iblk = blockIdx.x, h = blockIdx.y;
    const int nope = A.nope, kvl = A.kvl, W = A.kvl + A.rope;
    const int a_bytes = (nope / 64) * 16384;
    uint8_t* sA = smem;
    uint8_t* sB = smem + a_bytes;
    const size_t rbase = (size_t)h * (nope + A.vh);
    const int sc_cols = kvl / 128;
    // runs of d with one scale: [0, cut) and [cut, nope); cut = distance to the next block boundary
    const int cut = min(nope, (int)(128 - (rbase & 127)));
    const float s0 = A.scale[(rbase >> 7) * sc_cols + iblk];
    const bool two_runs = cut < nope;
    const float s1 = two_runs ? A.scale[((rbase + cut) >> 7) * sc_cols + iblk] : 0.0f;

    if (tid == 0) { tc::mbar_init(&bar, 1); tc::mbar_init_fence(); abort_word = 0; }
    if (warp == 0) tc::tmem_alloc<256>(&tmem_slot);
    // weights: row d, this CTA's 128 columns = 16 pieces of 8 codes -> bf16 chunks, MN-major tile
    for (int p = tid; p < nope * 16; p += KP_THREADS) {
        const int d = p >> 4, pc = p & 15;
        const uint2 c = *reinterpret_cast<const uint2*>(A.kvb + (rbase + d) * kvl + iblk * 128 + pc * 8);
        *reinterpret_cast<uint4*>(sB + (pc >> 3) * (nope * 128) + tc::sw128_chunk(d, pc & 7)) = kp_codes_to_bf16(c);
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t idesc = kp_idesc(128, 128, 1);
    const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
    bool ok = true;
    int phase = 0;
    for (int b0 = 0; b0 < A.B && ok; b0 += 128, phase ^= 1) {
        // activations: 128 sequences x nope bf16, K-major swizzled tile; rows past B are zeros
        const int chunks = nope / 8;   // 16-byte chunks per row
        for (int c = tid; c < 128 * chunks; c += KP_THREADS) {
            const int row = c / chunks, j = c - row * chunks;
            uint8_t* dst = sA + (j >> 3) * 16384 + tc::sw128_chunk(row, j & 7);
            if (b0 + row < A.B) tc::cp_async16(tc::smem_u32(dst), A.x + ((size_t)(b0 + row) * A.H + h) * A.xs + j * 8);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
        tc::cp_async_commit();
        tc::cp_async_wait<0>();
        tc::fence_proxy_async();
        __syncthreads();
        if (tid == 0) {
            tc::tc_fence_after();
            const uint32_t a0 = tc::smem_u32(sA), b0a = tc::smem_u32(sB);
            for (int k = 0; k < nope / 16; ++k) {     // 16 bf16 per MMA; a run boundary is a multiple of 64
                const int run = (k * 16 >= cut) ? 1 : 0;
                const bool first = (k * 16 == 0) || (k * 16 == cut);
                kp_mma(tmem + run * 128, kp_desc(a0 + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                       kp_desc(b0a + k * 2048, (uint32_t)nope * 128, 1024), idesc, first ? 0u : 1u);
            }
            tc::mma_commit(&bar);
        }
        // the rope segment of q rides along (column block 0 only): 16-byte copies, row = sequence
        if (iblk == 0 && b0 + tid < A.B) {
            const uint4* src = reinterpret_cast<const uint4*>(A.x + ((size_t)(b0 + tid) * A.H + h) * A.xs + nope);
            uint4* dst = reinterpret_cast<uint4*>(A.out + ((size_t)(b0 + tid) * A.H + h) * W + kvl);
            for (int e = 0; e < A.rope / 8; ++e) dst[e] = src[e];
        }
        ok = tc::mbar_wait(&bar, phase, abort_flag, 71);
        tc::tc_fence_after();
        if (ok) {
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t r0[32], r1[32];
                tc::tmem_ld32(tmem + lane_base + c * 32, r0);
                tc::tmem_ld32(tmem + lane_base + 128 + c * 32, r1);
                tc::tmem_ld_wait();
                if (!two_runs) {   // the second accumulator was never written
#pragma unroll
                    for (int e = 0; e < 32; ++e) r1[e] = 0u;
                }
                if (b0 + tid < A.B) {
                    uint32_t o[16];
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const float v0 = fmaf(__uint_as_float(r1[e]), s1, __uint_as_float(r0[e]) * s0);
                        const float v1 = fmaf(__uint_as_float(r1[e + 1]), s1, __uint_as_float(r0[e + 1]) * s0);
                        o[e >> 1] = (uint32_t)rv_f32_to_bf16(v0) | ((uint32_t)rv_f32_to_bf16(v1) << 16);
                    }
                    uint4* dst = reinterpret_cast<uint4*>(A.out + ((size_t)(b0 + tid) * A.H + h) * W + iblk * 128 + c * 32);
#pragma unroll
                    for (int e = 0; e < 4; ++e) dst[e] = make_uint4(o[4 * e], o[4 * e + 1], o[4 * e + 2], o[4 * e + 3]);
                }
            }
        }
        tc::tc_fence_before();
        __syncthreads();   // TMEM and the A tile are free for the next batch tile
    }
    if (warp == 0) tc::tmem_dealloc<256>(tmem);
    if (tid == 0 && abort_word) atomicCAS(&g_kp_err, 0, abort_word);
}

// ---------------------------------------------------------------------------------------------
// value: grid (vh / 64, H), 128 threads. Shared: A [kvl/64][128 rows][128 B] | B [kvl/64][64 rows][128 B].
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(KP_THREADS)
kvb_value_mma_kernel(KpArgs A) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_word;
    __shared__ float s_sc[8];
    volatile int* abort_flag = &abort_word;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int jblk = blockIdx.x, h = blockIdx.y;
    const int kvl = A.kvl, vh = A.vh;
    const int kch = kvl / 64;                 // 128-byte K chunks
    uint8_t* sA = smem;
    uint8_t* sB = smem + kch * 16384;
    const size_t row0 = (size_t)h * (A.nope + vh) + A.nope + (size_t)jblk * 64;   // 64 value rows in ONE scale row
    const int sc_cols = kvl / 128;
    if (tid < sc_cols) s_sc[tid] = A.scale[(row0 >> 7) * sc_cols + tid];
    if (tid == 0) { tc::mbar_init(&bar, 1); tc::mbar_init_fence(); abort_word = 0; }
    if (warp == 0) tc::tmem_alloc<256>(&tmem_slot);
    // weights: 64 rows x kvl codes -> bf16, K-major swizzled tile
    const int pieces = kvl / 8;
    for (int p = tid; p < 64 * pieces; p += KP_THREADS) {
        const int j = p / pieces, pc = p - j * pieces;
        const uint2 c = *reinterpret_cast<const uint2*>(A.kvb + (row0 + j) * kvl + pc * 8);
        *reinterpret_cast<uint4*>(sB + (pc >> 3) * 8192 + tc::sw128_chunk(j, pc & 7)) = kp_codes_to_bf16(c);
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t idesc = kp_idesc(128, 64, 0);
    const uint32_t lane_base = ((uint32_t)(warp * 32)) << 16;
    bool ok = true;
    int phase = 0;
    for (int b0 = 0; b0 < A.B && ok; b0 += 128, phase ^= 1) {
        const int chunks = kvl / 8;
        for (int c = tid; c < 128 * chunks; c += KP_THREADS) {
            const int row = c / chunks, j = c - row * chunks;
            uint8_t* dst = sA + (j >> 3) * 16384 + tc::sw128_chunk(row, j & 7);
            if (b0 + row < A.B) tc::cp_async16(tc::smem_u32(dst), A.x + ((size_t)(b0 + row) * A.H + h) * A.xs + j * 8);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
        tc::cp_async_commit();
        tc::cp_async_wait<0>();
        tc::fence_proxy_async();
        __syncthreads();
        if (tid == 0) {
            tc::tc_fence_after();
            const uint32_t a0 = tc::smem_u32(sA), b0a = tc::smem_u32(sB);
            for (int k = 0; k < kvl / 16; ++k) {      // 8 MMAs per scale column (128 latent dims)
                const int run = k >> 3;
                kp_mma(tmem + run * 64, kp_desc(a0 + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                       kp_desc(b0a + (k >> 2) * 8192 + (k & 3) * 32, 16, 1024), idesc, (k & 7) ? 1u : 0u);
            }
            tc::mma_commit(&bar);
        }
        ok = tc::mbar_wait(&bar, phase, abort_flag, 72);
        tc::tc_fence_after();
        if (ok) {
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
                float acc[32];
#pragma unroll
                for (int e = 0; e < 32; ++e) acc[e] = 0.0f;
                for (int run = 0; run < sc_cols; ++run) {
                    uint32_t r[32];
                    tc::tmem_ld32(tmem + lane_base + run * 64 + c * 32, r);
                    tc::tmem_ld_wait();
                    const float s = s_sc[run];
#pragma unroll
                    for (int e = 0; e < 32; ++e) acc[e] = fmaf(__uint_as_float(r[e]), s, acc[e]);
                }
                if (b0 + tid < A.B) {
                    uint32_t o[16];
#pragma unroll
                    for (int e = 0; e < 32; e += 2)
                        o[e >> 1] = (uint32_t)rv_f32_to_bf16(acc[e]) | ((uint32_t)rv_f32_to_bf16(acc[e + 1]) << 16);
                    uint4* dst = reinterpret_cast<uint4*>(A.out + ((size_t)(b0 + tid) * A.H + h) * vh + jblk * 64 + c * 32);
#pragma unroll
                    for (int e = 0; e < 4; ++e) dst[e] = make_uint4(o[4 * e], o[4 * e + 1], o[4 * e + 2], o[4 * e + 3]);
                }
            }
        }
        tc::tc_fence_before();
        __syncthreads();
    }
    if (warp == 0) tc::tmem_dealloc<256>(tmem);
    if (tid == 0 && abort_word) atomicCAS(&g_kp_err, 0, abort_word);
}

}  // namespace

// The tensor-core kernels cover: 128 x 128 scale blocks; kvl a multiple of 128 up to 512; nope a multiple
// of 64 up to 256 whose rows straddle at most one block boundary; vh and the head's row count multiples
// of 64; 16-byte aligned activation rows.
extern "C" int rivoli_kvb_mma_supported(int H, int qh, int nope, int vh, int kvl, int rope, int block) {
    if (block != 128 || kvl % 128 || kvl > 512 || nope % 64 || nope > 256 || vh % 64 || (nope + vh) % 64) return 0;
    if (qh % 8 || rope % 8 || H <= 0) return 0;
    for (int h = 0; h < 2 && h < H; ++h) {          // the straddle pattern repeats with period <= 2 heads
        const int off = (h * (nope + vh)) & 127;
        if (nope > (128 - off) + 128) return 0;       // would need a third run
    }
    return 1;
}

extern "C" int rivoli_kvb_absorb_mma(const uint16_t* q, const uint8_t* kvb, const float* scale, int H, int qh, int nope,
                                     int vh, int kvl, int rope, int block, int B, uint16_t* q_abs, cudaStream_t st) {
    const KpArgs a{q, kvb, scale, H, qh, nope, vh, kvl, rope, block, B, q_abs};
    const size_t smem = (size_t)(nope / 64) * 16384 + (size_t)2 * nope * 128;
    cudaFuncSetAttribute(kvb_absorb_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rv_drain_error();
    kvb_absorb_mma_kernel<<<dim3(kvl / 128, H), KP_THREADS, smem, st>>>(a);
    return rv_launch_status();
}

extern "C" int rivoli_kvb_value_mma(const uint16_t* clat, const uint8_t* kvb, const float* scale, int H, int nope, int vh,
                                    int kvl, int block, int B, uint16_t* ctx, cudaStream_t st) {
    const KpArgs a{clat, kvb, scale, H, kvl, nope, vh, kvl, 0, block, B, ctx};
    const size_t smem = (size_t)(kvl / 64) * 16384 + (size_t)(kvl / 64) * 8192;
    cudaFuncSetAttribute(kvb_value_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rv_drain_error();
    kvb_value_mma_kernel<<<dim3(vh / 64, H), KP_THREADS, smem, st>>>(a);
    return rv_launch_status();
}

// Synchronises the stream; 1008 if a bounded wait of a tensor-core projection gave up since the last call.
RIVOLI_API int rivoli_kvb_proj_status(void* stream) {
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return -(int)e;
    int h = 0;
    e = cudaMemcpyFromSymbol(&h, g_kp_err, sizeof(int));
    if (e != cudaSuccess) return -(int)e;
    if (h) { const int z = 0; cudaMemcpyToSymbol(g_kp_err, &z, sizeof(int)); }
    return h ? 1008 : 0;
}
