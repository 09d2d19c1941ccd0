// Gather roofline probe: how fast can CTAs pull 576-byte latent rows, picked at random from the
// paged pool, into shared memory - the access pattern that bounds the attention kernel - by
// each of the copy methods a kernel could use. Diagnostic only (bench.py --profile gather);
// nothing on the product path calls it.
//   method 0: cp.async 16 B, row by row, the 32 lanes of a warp on consecutive chunks
//   method 1: cp.async.bulk, one 576-byte row per thread (lands unswizzled)
//   method 2: TMA tile::gather4, box 128 B x 1 row with the 128-byte swizzle (+ 64 B x 1 row with
//             the 64-byte swizzle for the rope part): lands in the UMMA K-major operand layout
//   method 3: method 0 with the rows of the tile `GP_AHEAD` tiles on prefetched into L2
//             (cp.async.bulk.prefetch.L2, one 576-byte request per row)
// All waits are bounded; a wait that gives up sets the error word and the probe returns 1008.
#include "common.cuh"
#include "tmap.hpp"

namespace {

constexpr int GP_ROWB = 576, GP_TILE = 128;
constexpr int GP_AHEAD = 3;
constexpr int GP_LATB = 65536, GP_ROPEB = 8192, GP_TILEB = GP_LATB + GP_ROPEB;   // = 128 * 576

__device__ int g_gp_err;      // a bounded wait gave up
__device__ float g_gp_sink;   // keeps the copied bytes observable

__device__ __forceinline__ uint32_t gp_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void gp_mbar_init(uint64_t* b, int n) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(gp_smem(b)), "r"(n));
}
__device__ __forceinline__ void gp_mbar_expect(uint64_t* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(gp_smem(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool gp_mbar_wait(uint64_t* b, uint32_t parity, int* err) {
    for (int i = 0; i < 4000000; ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(gp_smem(b)), "r"(parity) : "memory");
        if (ok) return true;
    }
    *err = 1;
    return false;
}

template <int METHOD, int DEPTH>
__global__ void __launch_bounds__(128)
gather_probe_kernel(const __grid_constant__ CUtensorMap tm_lat, const __grid_constant__ CUtensorMap tm_rope,
                    const uint8_t* __restrict__ pool, const float* __restrict__ scales,
                    const uint32_t* __restrict__ rows, int ntiles) {
    int* err = &g_gp_err;
    extern __shared__ __align__(1024) uint8_t gp_buf[];
    __shared__ uint64_t full[DEPTH];
    __shared__ float s_scale[DEPTH][GP_TILE];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t* myrows = rows + (size_t)blockIdx.x * ntiles * GP_TILE;
    if (tid == 0) {
        for (int d = 0; d < DEPTH; ++d) gp_mbar_init(&full[d], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    float acc = 0.f;
    auto issue = [&](int j) {
        const int d = j % DEPTH;
        uint8_t* dst = gp_buf + (size_t)d * GP_TILEB;
        const uint32_t r = myrows[j * GP_TILE + tid];
        s_scale[d][tid] = scales[r];
        if (METHOD == 3 && j + GP_AHEAD < ntiles) {
            const uint32_t rp = myrows[(j + GP_AHEAD) * GP_TILE + tid];
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(pool + (size_t)rp * GP_ROWB), "r"(GP_ROWB) : "memory");
        }
        if (METHOD == 0 || METHOD == 3) {
            const unsigned long long sp = (unsigned long long)(pool + (size_t)r * GP_ROWB);
            for (int it = 0; it < 32; ++it) {
                const uint8_t* rs = (const uint8_t*)__shfl_sync(0xffffffffu, sp, it);
                uint8_t* rd = dst + (warp * 32 + it) * GP_ROWB;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(gp_smem(rd + lane * 16)), "l"(rs + lane * 16) : "memory");
                if (lane < 4)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(gp_smem(rd + 512 + lane * 16)), "l"(rs + 512 + lane * 16) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        } else if (METHOD == 1) {
            if (tid == 0) gp_mbar_expect(&full[d], GP_TILEB);
            __syncthreads();
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(gp_smem(dst + tid * GP_ROWB)), "l"(pool + (size_t)r * GP_ROWB), "r"(GP_ROWB), "r"(gp_smem(&full[d])) : "memory");
        } else if (warp == 0) {
            const uint4 q = *reinterpret_cast<const uint4*>(myrows + j * GP_TILE + lane * 4);
            if (lane == 0) gp_mbar_expect(&full[d], GP_TILEB);
            __syncwarp();
#pragma unroll
            for (int c = 0; c < 4; ++c)
                asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
                             ::"r"(gp_smem(dst + c * 16384 + lane * 512)), "l"(&tm_lat), "r"(c * 128), "r"((int)q.x), "r"((int)q.y),
                               "r"((int)q.z), "r"((int)q.w), "r"(gp_smem(&full[d])) : "memory");
            asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
                         ::"r"(gp_smem(dst + GP_LATB + lane * 256)), "l"(&tm_rope), "r"(512), "r"((int)q.x), "r"((int)q.y),
                           "r"((int)q.z), "r"((int)q.w), "r"(gp_smem(&full[d])) : "memory");
        }
    };
    if (METHOD == 3)
        for (int j = 0; j < GP_AHEAD && j < ntiles; ++j) {
            const uint32_t rp = myrows[j * GP_TILE + tid];
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(pool + (size_t)rp * GP_ROWB), "r"(GP_ROWB) : "memory");
        }
    for (int j = 0; j < DEPTH - 1 && j < ntiles; ++j) issue(j);
    for (int j = 0; j < ntiles; ++j) {
        if (j + DEPTH - 1 < ntiles) issue(j + DEPTH - 1);
        const int d = j % DEPTH;
        if (METHOD == 0 || METHOD == 3) {
            const int pend = min(DEPTH - 1, ntiles - 1 - j);
            if (pend >= 2) asm volatile("cp.async.wait_group 2;" ::: "memory");
            else if (pend == 1) asm volatile("cp.async.wait_group 1;" ::: "memory");
            else asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();
        } else if (!gp_mbar_wait(&full[d], (j / DEPTH) & 1, err)) {
            break;
        }
        acc += (float)gp_buf[(size_t)d * GP_TILEB + tid * 128 + (j & 63)] + s_scale[d][tid];
        __syncthreads();   // the buffer may be refilled
    }
    if (acc == 12345.678f) g_gp_sink = acc;
}

template <int METHOD, int DEPTH>
int run_probe(const CUtensorMap& tl, const CUtensorMap& tr, const uint8_t* pool, const float* scales, const uint32_t* rows,
              int n_ctas, int n_tiles, float* ms_out, cudaStream_t st) {
    const size_t smem = (size_t)DEPTH * GP_TILEB;
    if (cudaFuncSetAttribute(gather_probe_kernel<METHOD, DEPTH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return 1002;
    const int zero = 0;
    cudaMemcpyToSymbolAsync(g_gp_err, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, st);
    cudaEvent_t a, b;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    const int warm = 3, reps = 10;
    for (int i = 0; i < warm + reps; ++i) {
        if (i == warm) cudaEventRecord(a, st);
        gather_probe_kernel<METHOD, DEPTH><<<n_ctas, 128, smem, st>>>(tl, tr, pool, scales, rows, n_tiles);
    }
    cudaEventRecord(b, st);
    cudaError_t e = cudaStreamSynchronize(st);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, a, b);
    int h = 0;
    cudaMemcpyFromSymbol(&h, g_gp_err, sizeof(int));
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    if (e != cudaSuccess) return -(int)e;
    *ms_out = ms / reps;
    return h ? 1008 : 0;
}

}  // namespace

// Average time (ms) of one launch in which each of n_ctas CTAs gathers n_tiles tiles of 128 rows
// (rows[cta][tile][128], pool row numbers < n_pool_rows) with `depth` tiles in flight.
RIVOLI_API int rivoli_probe_gather(int method, int depth, int n_ctas, int n_tiles, const uint8_t* pool,
                                   unsigned long long n_pool_rows, const float* scales, const uint32_t* rows,
                                   float* ms_out, void* stream) {
    if (!pool || !scales || !rows || !ms_out || n_ctas <= 0 || n_tiles <= 0 || depth < 1 || depth > 3) return 1001;
    if (((uintptr_t)pool | (uintptr_t)rows) & 15) return 1005;
    CUtensorMap tl, tr;
    {
        rivoli::EncodeTiledFn fn = rivoli::encode_tiled_fn();
        if (!fn) return 1008;
        const cuuint64_t dims[2] = {GP_ROWB, n_pool_rows};
        const cuuint64_t strides[1] = {GP_ROWB};
        const cuuint32_t estr[2] = {1, 1}, box_l[2] = {128, 1}, box_r[2] = {64, 1};
        if (fn(&tl, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(pool), dims, strides, box_l, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS ||
            fn(&tr, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(pool), dims, strides, box_r, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return 1008;
    }
    cudaStream_t st = (cudaStream_t)stream;
    rv_drain_error();
#define GP_CASE(M, D) if (method == M && depth == D) return run_probe<M, D>(tl, tr, pool, scales, rows, n_ctas, n_tiles, ms_out, st)
    GP_CASE(0, 1); GP_CASE(0, 2); GP_CASE(0, 3);
    GP_CASE(1, 1); GP_CASE(1, 2); GP_CASE(1, 3);
    GP_CASE(2, 1); GP_CASE(2, 2); GP_CASE(2, 3);
    GP_CASE(3, 1); GP_CASE(3, 2); GP_CASE(3, 3);
#undef GP_CASE
    return 1001;
}
