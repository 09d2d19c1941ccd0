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
//   value:  ctx[b][h][j]  = sum_i o[b][h][i] * kvb[448 h + 192 + j][i]     M = 128 sequences, N = 128 of the 256
//           value rows (two scale rows, one per 64 columns), K = kvl = 512 = four runs (one per scale
//           column); CTA = (row block, head) - 128 CTAs, one wave; weights are the K-major B operand.
// Geometry outside these shapes takes the CUDA-core kernels of kvb_proj.cu.
// All waits are bounded (tc_common.cuh); a wait that gives up sets g_kp_err (rivoli_kvb_proj_status).
#include "codec.cuh"
#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int KP_THREADS = 256;   // 8 warps: loaders by (warp = row, lane = chunk); epilogue by (lane quadrant, column half)
constexpr int KP_WARPS = KP_THREADS / 32;
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
    // activations of a batch tile: 128 sequences x nope bf16, K-major swizzled; warp = row, lane = 16-byte chunk;
    // rows past B are zeros. Asynchronous: requested BEFORE the weights are fetched and converted.
    auto load_acts = [&](int b0) {
        const int chunks = nope / 8;
        for (int row = warp; row < 128; row += KP_WARPS) {
            const bool live = b0 + row < A.B;
            const uint16_t* src = A.x + ((size_t)(live ? b0 + row : 0) * A.H + h) * A.xs;
            for (int j = lane; j < chunks; j += 32) {
                uint8_t* dst = sA + (j >> 3) * 16384 + tc::sw128_chunk(row, j & 7);
                if (live) tc::cp_async16(tc::smem_u32(dst), src + j * 8);
                else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            }
        }
        tc::cp_async_commit();
    };
    load_acts(0);
    // weights: row d, this CTA's 128 columns = 16 pieces of 8 codes -> bf16 chunks, MN-major tile.
    // Two rows per warp pass (lane = row half x piece); ALL passes (nope <= 256: at most 16) are in flight
    // before the first conversion, so the tile costs one memory round trip.
    {
        uint2 c[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const int d = warp * 2 + u * KP_WARPS * 2 + (lane >> 4);
            c[u] = d < nope ? *reinterpret_cast<const uint2*>(A.kvb + (rbase + d) * kvl + iblk * 128 + (lane & 15) * 8) : make_uint2(0, 0);
        }
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const int d = warp * 2 + u * KP_WARPS * 2 + (lane >> 4), pc = lane & 15;
            if (d < nope)
                *reinterpret_cast<uint4*>(sB + (pc >> 3) * (nope * 128) + tc::sw128_chunk(d, pc & 7)) = kp_codes_to_bf16(c[u]);
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t idesc = kp_idesc(128, 128, 1);
    const uint32_t lane_base = ((uint32_t)((warp & 3) * 32)) << 16;   // TMEM lane quadrant of this warp
    const int erow = (warp & 3) * 32 + lane, chalf = warp >> 2;      // epilogue: sequence row, column half
    bool ok = true;
    int phase = 0;
    for (int b0 = 0; b0 < A.B && ok; b0 += 128, phase ^= 1) {
        if (b0 > 0) load_acts(b0);     // the first tile was requested before the weights
        // the rope segment of q rides along (column block 0 only; thread = sequence row): its loads go out
        // now and are stored after the MMAs were issued, off every wait's critical path
        uint4 rope_v[8];
        const bool rope_mine = iblk == 0 && tid < 128 && b0 + tid < A.B;
        if (rope_mine) {
            const uint4* src = reinterpret_cast<const uint4*>(A.x + ((size_t)(b0 + tid) * A.H + h) * A.xs + nope);
#pragma unroll
            for (int e = 0; e < 8; ++e) rope_v[e] = e < A.rope / 8 ? src[e] : make_uint4(0, 0, 0, 0);
        }
        tc::cp_async_wait<0>();
        tc::fence_proxy_async();
        __syncthreads();
        if (tid == 0) {
            tc::tc_fence_after();
            const uint32_t a0 = tc::smem_u32(sA), b0a = tc::smem_u32(sB);
            for (int k = 0; k < nope / 16; ++k) {     // 16 bf16 per MMA; a run boundary is a multiple of 64
                const int run = (k * 16 >= cut) ? 1 : 0;
                const bool first = (k * 16 == 0) || (k * 16 == cut);
#ifdef KP_TEST_KMAJOR   // timing experiment only (wrong numbers): the same tile described as K-major
                kp_mma(tmem + run * 128, kp_desc(a0 + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                       kp_desc(b0a + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024), kp_idesc(128, 128, 0), first ? 0u : 1u);
#else
                kp_mma(tmem + run * 128, kp_desc(a0 + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                       kp_desc(b0a + k * 2048, (uint32_t)nope * 128, 1024), idesc, first ? 0u : 1u);
#endif
            }
            tc::mma_commit(&bar);
        }
        if (rope_mine) {
            uint4* dst = reinterpret_cast<uint4*>(A.out + ((size_t)(b0 + tid) * A.H + h) * W + kvl);
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (e < A.rope / 8) dst[e] = rope_v[e];
        }
        ok = tc::mbar_wait_warp(&bar, phase, abort_flag, 71);
        tc::tc_fence_after();
        if (ok) {
#pragma unroll 1
            for (int c = chalf * 2; c < chalf * 2 + 2; ++c) {
                uint32_t r0[32], r1[32];
                tc::tmem_ld32(tmem + lane_base + c * 32, r0);
                tc::tmem_ld32(tmem + lane_base + 128 + c * 32, r1);
                tc::tmem_ld_wait();
                if (!two_runs) {   // the second accumulator was never written
#pragma unroll
                    for (int e = 0; e < 32; ++e) r1[e] = 0u;
                }
                if (b0 + erow < A.B) {
                    uint32_t o[16];
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const float v0 = fmaf(__uint_as_float(r1[e]), s1, __uint_as_float(r0[e]) * s0);
                        const float v1 = fmaf(__uint_as_float(r1[e + 1]), s1, __uint_as_float(r0[e + 1]) * s0);
                        o[e >> 1] = (uint32_t)rv_f32_to_bf16(v0) | ((uint32_t)rv_f32_to_bf16(v1) << 16);
                    }
                    uint4* dst = reinterpret_cast<uint4*>(A.out + ((size_t)(b0 + erow) * A.H + h) * W + iblk * 128 + c * 32);
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
// value: grid (vh / 128, H), 256 threads; N = 128 value rows = two 64-row scale rows.
// Shared: A half [kvl/128][128 rows][128 B] (the contraction is fed in two halves) | B [kvl/64][128 rows][128 B].
// TMEM: one 128-column accumulator per scale column (kvl / 128 <= 4 runs).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(KP_THREADS)
kvb_value_mma_kernel(KpArgs A) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t bar[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_word;
    __shared__ float s_sc[2][4];
    volatile int* abort_flag = &abort_word;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int jblk = blockIdx.x, h = blockIdx.y;
    const int kvl = A.kvl, vh = A.vh;
    const int kch = kvl / 64;                 // 128-byte K chunks in all
    const int hch = kch / 2;                  // per half
    uint8_t* sA = smem;
    uint8_t* sB = smem + hch * 16384;
    const size_t row0 = (size_t)h * (A.nope + vh) + A.nope + (size_t)jblk * 128;   // 128 value rows = 2 scale rows
    const int sc_cols = kvl / 128;
    if (tid < 2 * sc_cols) s_sc[tid / sc_cols][tid % sc_cols] = A.scale[((row0 + (tid / sc_cols) * 64) >> 7) * sc_cols + tid % sc_cols];
    if (tid == 0) { tc::mbar_init(&bar[0], 1); tc::mbar_init(&bar[1], 1); tc::mbar_init_fence(); abort_word = 0; }
    if (warp == 0) tc::tmem_alloc<512>(&tmem_slot);
    // activations of one half of the contraction for a batch tile: 128 sequences x kvl/2 bf16, K-major
    // swizzled; warp = row, lane = 16-byte chunk; rows past B are zeros. Asynchronous.
    auto load_acts = [&](int b0, int half) {
        const int chunks = kvl / 16;
        for (int row = warp; row < 128; row += KP_WARPS) {
            const bool live = b0 + row < A.B;
            const uint16_t* src = A.x + ((size_t)(live ? b0 + row : 0) * A.H + h) * A.xs + half * (kvl / 2);
            for (int j = lane; j < chunks; j += 32) {
                uint8_t* dst = sA + (j >> 3) * 16384 + tc::sw128_chunk(row, j & 7);
                if (live) tc::cp_async16(tc::smem_u32(dst), src + j * 8);
                else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
            }
        }
        tc::cp_async_commit();
    };
    load_acts(0, 0);
    // weights: 128 rows x kvl codes -> bf16, K-major swizzled tile; warp = row, lane = piece of 8 codes;
    // all sixteen rows of a warp (32 loads per lane) in flight before the first conversion
    const int pieces = kvl / 8;
    {
        uint2 c[16][2];
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            const uint8_t* wrow = A.kvb + (row0 + warp + r * KP_WARPS) * kvl;
#pragma unroll
            for (int u = 0; u < 2; ++u)
                c[r][u] = lane + 32 * u < pieces ? *reinterpret_cast<const uint2*>(wrow + (lane + 32 * u) * 8) : make_uint2(0, 0);
        }
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            const int j = warp + r * KP_WARPS;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int pc = lane + 32 * u;
                if (pc < pieces) *reinterpret_cast<uint4*>(sB + (pc >> 3) * 16384 + tc::sw128_chunk(j, pc & 7)) = kp_codes_to_bf16(c[r][u]);
            }
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t idesc = kp_idesc(128, 128, 0);
    const uint32_t lane_base = ((uint32_t)((warp & 3) * 32)) << 16;   // TMEM lane quadrant of this warp
    const int erow = (warp & 3) * 32 + lane, chalf = warp >> 2;      // epilogue: sequence row, 64-column half
    bool ok = true;
    int phase = 0;
    for (int b0 = 0; b0 < A.B && ok; b0 += 128, phase ^= 1) {
        for (int half = 0; half < 2 && ok; ++half) {
            if (b0 > 0 || half > 0) load_acts(b0, half);   // the very first request went out before the weights
            tc::cp_async_wait<0>();
            tc::fence_proxy_async();
            __syncthreads();
            if (tid == 0) {
                tc::tc_fence_after();
                const uint32_t a0 = tc::smem_u32(sA), b0a = tc::smem_u32(sB);
                const int ks = kvl / 32;                  // MMAs per half; 8 per scale column (128 latent dims)
                for (int kk = 0; kk < ks; ++kk) {
                    const int k = half * ks + kk;
                    kp_mma(tmem + (k >> 3) * 128, kp_desc(a0 + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                           kp_desc(b0a + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024), idesc, (k & 7) ? 1u : 0u);
                }
                tc::mma_commit(&bar[half]);
            }
            // the A half may be overwritten (and the accumulators read) only once these MMAs are done
            ok = tc::mbar_wait_warp(&bar[half], phase, abort_flag, 72 + half);
        }
        tc::tc_fence_after();
        if (ok) {
#pragma unroll 1
            for (int c = chalf * 2; c < chalf * 2 + 2; ++c) {
                float acc[32];
#pragma unroll
                for (int e = 0; e < 32; ++e) acc[e] = 0.0f;
                for (int run = 0; run < sc_cols; ++run) {
                    uint32_t r[32];
                    tc::tmem_ld32(tmem + lane_base + run * 128 + c * 32, r);
                    tc::tmem_ld_wait();
                    const float sc = s_sc[chalf][run];
#pragma unroll
                    for (int e = 0; e < 32; ++e) acc[e] = fmaf(__uint_as_float(r[e]), sc, acc[e]);
                }
                if (b0 + erow < A.B) {
                    uint32_t o[16];
#pragma unroll
                    for (int e = 0; e < 32; e += 2)
                        o[e >> 1] = (uint32_t)rv_f32_to_bf16(acc[e]) | ((uint32_t)rv_f32_to_bf16(acc[e + 1]) << 16);
                    uint4* dst = reinterpret_cast<uint4*>(A.out + ((size_t)(b0 + erow) * A.H + h) * vh + jblk * 128 + c * 32);
#pragma unroll
                    for (int e = 0; e < 4; ++e) dst[e] = make_uint4(o[4 * e], o[4 * e + 1], o[4 * e + 2], o[4 * e + 3]);
                }
            }
        }
        tc::tc_fence_before();
        __syncthreads();
    }
    if (warp == 0) tc::tmem_dealloc<512>(tmem);
    if (tid == 0 && abort_word) atomicCAS(&g_kp_err, 0, abort_word);
}

}  // namespace

// The tensor-core kernels cover: 128 x 128 scale blocks; kvl 256 or 512; nope a multiple of 64 up to 256
// whose rows straddle at most one block boundary; vh a multiple of 128; the head's row count a multiple
// of 64; 16-byte aligned activation rows; rope <= 64.
extern "C" int rivoli_kvb_mma_supported(int H, int qh, int nope, int vh, int kvl, int rope, int block) {
    if (block != 128 || kvl % 256 || kvl > 512 || nope % 64 || nope > 256 || vh % 128 || (nope + vh) % 64) return 0;
    if (qh % 8 || rope % 8 || rope > 64 || H <= 0) return 0;
    for (int h = 0; h < 2 && h < H; ++h) {          // the straddle pattern repeats with period <= 2 heads
        const int off = (h * (nope + vh)) & 127;
        if (nope > (128 - off) + 128) return 0;       // would need a third run
    }
    return 1;
}

extern "C" int rivoli_kvb_absorb_mma(const uint16_t* q, const uint8_t* kvb, const float* scale, int H, int qh, int nope,
                                     int vh, int kvl, int rope, int block, int B, uint16_t* q_abs, cudaStream_t st) {
    const KpArgs a{q, kvb, scale, H, qh, nope, vh, kvl, rope, block, B, q_abs};
    size_t smem = (size_t)(nope / 64) * 16384 + (size_t)2 * nope * 128;
#ifdef KP_TEST_ONE_CTA   // timing experiment: one CTA per SM
    if (smem < 120 * 1024) smem = 120 * 1024;
#endif
    cudaFuncSetAttribute(kvb_absorb_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rv_drain_error();
    kvb_absorb_mma_kernel<<<dim3(kvl / 128, H), KP_THREADS, smem, st>>>(a);
    return rv_launch_status();
}

extern "C" int rivoli_kvb_value_mma(const uint16_t* clat, const uint8_t* kvb, const float* scale, int H, int nope, int vh,
                                    int kvl, int block, int B, uint16_t* ctx, cudaStream_t st) {
    const KpArgs a{clat, kvb, scale, H, kvl, nope, vh, kvl, 0, block, B, ctx};
    const size_t smem = (size_t)(kvl / 128) * 16384 + (size_t)(kvl / 64) * 16384;
    cudaFuncSetAttribute(kvb_value_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rv_drain_error();
    kvb_value_mma_kernel<<<dim3(vh / 128, H), KP_THREADS, smem, st>>>(a);
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

