// The two contractions through kv_b either side of MLA attention.
//
//   rivoli_mla_absorb_fp8 / rivoli_mla_value_fp8 : the reference's single-token f32 operators
//       (crates/backend/kernels/mla.hip:12-231): same symbols, arguments, guard codes. One thread
//       per output, the reference's fold order (d, resp. i, ascending; q * (e4m3 * scale)), no
//       contraction - bit-identical to the host references of its tests
//       (crates/engine/tests/kernel_attend.rs:361-390).
//   rivoli_mla_absorb_batched_bf16 / rivoli_mla_value_batched_bf16 : the batched decode form
//       (bf16 activations [B][H][..]); CUDA-core kernels here for any geometry, tensor-core
//       kernels in kvb_proj_mma.cu for the model geometry.
//
// kv_b: e4m3 codes [H*(nope+vh) rows][kvl cols], scale[(row / block) * ceil(kvl/block) + col / block].
#include "codec.cuh"
#include "common.cuh"

namespace {

__device__ __forceinline__ int kp_shift(int block) { return 31 - __clz(block); }

template <int R>
__global__ void __launch_bounds__(256)
absorb_f32_kernel(const float* __restrict__ q, const uint8_t* __restrict__ kvb, const float* __restrict__ scale, int H,
                  int qh, int nope, int vh, int kvl, int block, float* __restrict__ qabs) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)H * kvl) return;
    const int head = (int)(idx / kvl), i = (int)(idx % kvl);
    const int bsh = kp_shift(block), sc_cols = (kvl + block - 1) / block;
    const size_t rbase = (size_t)head * (nope + vh);
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;
    for (int d = 0; d < nope; ++d) {
        const size_t row = rbase + d;
        const float ws = __fmul_rn(rv_e4m3_to_f32(kvb[row * kvl + i]), scale[(row >> bsh) * sc_cols + (i >> bsh)]);
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = __fadd_rn(acc[r], __fmul_rn(q[(size_t)r * H * qh + (size_t)head * qh + d], ws));
    }
#pragma unroll
    for (int r = 0; r < R; ++r) qabs[(size_t)r * H * kvl + idx] = acc[r];
}

template <int R>
__global__ void __launch_bounds__(256)
value_f32_kernel(const float* __restrict__ clat, const uint8_t* __restrict__ kvb, const float* __restrict__ scale, int H,
                 int nope, int vh, int kvl, int block, float* __restrict__ ctx) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)H * vh) return;
    const int head = (int)(idx / vh), j = (int)(idx % vh);
    const int bsh = kp_shift(block), sc_cols = (kvl + block - 1) / block;
    const size_t row = (size_t)head * (nope + vh) + nope + j;
    const uint8_t* w = kvb + row * kvl;
    const float* srow = scale + (row >> bsh) * sc_cols;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;
    for (int i = 0; i < kvl; ++i) {
        const float ws = __fmul_rn(rv_e4m3_to_f32(w[i]), srow[i >> bsh]);
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = __fadd_rn(acc[r], __fmul_rn(clat[(size_t)r * H * kvl + (size_t)head * kvl + i], ws));
    }
#pragma unroll
    for (int r = 0; r < R; ++r) ctx[(size_t)r * H * vh + idx] = acc[r];
}

// Batched bf16, any geometry: one thread per (sequence, head, output), the same folds.
__global__ void __launch_bounds__(256)
absorb_batched_simt_kernel(const uint16_t* __restrict__ q, const uint8_t* __restrict__ kvb,
                           const float* __restrict__ scale, int H, int qh, int nope, int vh, int kvl, int rope,
                           int block, int B, uint16_t* __restrict__ q_abs) {
    const int W = kvl + rope;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)B * H * W) return;
    const int i = (int)(idx % W);
    const size_t bh = idx / W;
    const int head = (int)(bh % H);
    const uint16_t* qr = q + bh * qh;
    if (i >= kvl) { q_abs[idx] = qr[nope + (i - kvl)]; return; }   // the rope segment rides along, bit for bit
    const int bsh = kp_shift(block), sc_cols = (kvl + block - 1) / block;
    const size_t rbase = (size_t)head * (nope + vh);
    float acc = 0.0f;
    for (int d = 0; d < nope; ++d) {
        const size_t row = rbase + d;
        const float ws = __fmul_rn(rv_e4m3_to_f32(kvb[row * kvl + i]), scale[(row >> bsh) * sc_cols + (i >> bsh)]);
        acc = __fadd_rn(acc, __fmul_rn(rv_bf16_to_f32(qr[d]), ws));
    }
    q_abs[idx] = rv_f32_to_bf16(acc);
}

__global__ void __launch_bounds__(256)
value_batched_simt_kernel(const uint16_t* __restrict__ clat, const uint8_t* __restrict__ kvb,
                          const float* __restrict__ scale, int H, int nope, int vh, int kvl, int block, int B,
                          uint16_t* __restrict__ ctx) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)B * H * vh) return;
    const int j = (int)(idx % vh);
    const size_t bh = idx / vh;
    const int head = (int)(bh % H);
    const int bsh = kp_shift(block), sc_cols = (kvl + block - 1) / block;
    const size_t row = (size_t)head * (nope + vh) + nope + j;
    const uint8_t* w = kvb + row * kvl;
    const float* srow = scale + (row >> bsh) * sc_cols;
    const uint16_t* cr = clat + bh * kvl;
    float acc = 0.0f;
    for (int i = 0; i < kvl; ++i)
        acc = __fadd_rn(acc, __fmul_rn(rv_bf16_to_f32(cr[i]), __fmul_rn(rv_e4m3_to_f32(w[i]), srow[i >> bsh])));
    ctx[idx] = rv_f32_to_bf16(acc);
}

int guard_dims(int H, int qh, int nope, int vh, int kvl, int block) {
    if (H <= 0 || qh <= 0 || nope <= 0 || vh <= 0 || kvl <= 0 || block <= 0) return 1001;
    if (block & (block - 1)) return 1003;   // the block index is a shift
    return 0;
}

}  // namespace

RIVOLI_API int rivoli_mla_absorb_fp8(const float* q, const unsigned char* kvb, const float* kvb_scale, int H, int qh,
                                     int nope, int vh, int kvl, int block, int nrow, float* qabs) {
    if (int e = guard_dims(H, qh, nope, vh, kvl, block)) return e;
    if (nrow != 1 && nrow != 2) return 1004;
    const unsigned grid = (unsigned)(((size_t)H * kvl + 255) / 256);
    rv_drain_error();
    if (nrow == 2) absorb_f32_kernel<2><<<grid, 256>>>(q, kvb, kvb_scale, H, qh, nope, vh, kvl, block, qabs);
    else absorb_f32_kernel<1><<<grid, 256>>>(q, kvb, kvb_scale, H, qh, nope, vh, kvl, block, qabs);
    return rv_launch_status();
}

RIVOLI_API int rivoli_mla_value_fp8(const float* clat, const unsigned char* kvb, const float* kvb_scale, int H,
                                    int nope, int vh, int kvl, int block, int nrow, float* ctx) {
    if (int e = guard_dims(H, 1, nope, vh, kvl, block)) return e;
    if (nrow != 1 && nrow != 2) return 1004;
    if (kvl & 3) return 1002;   // the reference's value kernel loads weights as words (mla.hip:216-225)
    const unsigned grid = (unsigned)(((size_t)H * vh + 255) / 256);
    rv_drain_error();
    if (nrow == 2) value_f32_kernel<2><<<grid, 256>>>(clat, kvb, kvb_scale, H, nope, vh, kvl, block, ctx);
    else value_f32_kernel<1><<<grid, 256>>>(clat, kvb, kvb_scale, H, nope, vh, kvl, block, ctx);
    return rv_launch_status();
}

// Defined in kvb_proj_mma.cu: 0 if the geometry is outside the tensor-core kernels.
extern "C" int rivoli_kvb_mma_supported(int H, int qh, int nope, int vh, int kvl, int rope, int block);
extern "C" int rivoli_kvb_absorb_mma(const uint16_t* q, const uint8_t* kvb, const float* scale, int H, int qh, int nope,
                                     int vh, int kvl, int rope, int block, int B, uint16_t* q_abs, cudaStream_t st);
extern "C" int rivoli_kvb_value_mma(const uint16_t* clat, const uint8_t* kvb, const float* scale, int H, int nope, int vh,
                                    int kvl, int block, int B, uint16_t* ctx, cudaStream_t st);

RIVOLI_API int rivoli_mla_absorb_batched_bf16(const uint16_t* q, const unsigned char* kvb, const float* kvb_scale, int H,
                                              int qh, int nope, int vh, int kvl, int rope, int block, int B,
                                              uint16_t* q_abs, int force_simt, void* stream) {
    if (int e = guard_dims(H, qh, nope, vh, kvl, block)) return e;
    if (B <= 0 || rope < 0 || !q || !kvb || !kvb_scale || !q_abs) return 1001;
    if (nope + rope > qh) return 1002;
    cudaStream_t st = (cudaStream_t)stream;
    if (!force_simt && rivoli_kvb_mma_supported(H, qh, nope, vh, kvl, rope, block)) {
        if (((uintptr_t)q | (uintptr_t)kvb | (uintptr_t)q_abs) & 15) return 1005;
        return rivoli_kvb_absorb_mma(q, kvb, kvb_scale, H, qh, nope, vh, kvl, rope, block, B, q_abs, st);
    }
    const size_t total = (size_t)B * H * (kvl + rope);
    rv_drain_error();
    absorb_batched_simt_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(q, kvb, kvb_scale, H, qh, nope, vh, kvl,
                                                                                rope, block, B, q_abs);
    return rv_launch_status();
}

RIVOLI_API int rivoli_mla_value_batched_bf16(const uint16_t* clat, const unsigned char* kvb, const float* kvb_scale,
                                             int H, int nope, int vh, int kvl, int block, int B, uint16_t* ctx,
                                             int force_simt, void* stream) {
    if (int e = guard_dims(H, 1, nope, vh, kvl, block)) return e;
    if (B <= 0 || !clat || !kvb || !kvb_scale || !ctx) return 1001;
    cudaStream_t st = (cudaStream_t)stream;
    if (!force_simt && rivoli_kvb_mma_supported(H, nope, nope, vh, kvl, 0, block)) {
        if (((uintptr_t)clat | (uintptr_t)kvb | (uintptr_t)ctx) & 15) return 1005;
        return rivoli_kvb_value_mma(clat, kvb, kvb_scale, H, nope, vh, kvl, block, B, ctx, st);
    }
    const size_t total = (size_t)B * H * vh;
    rv_drain_error();
    value_batched_simt_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(clat, kvb, kvb_scale, H, nope, vh, kvl,
                                                                               block, B, ctx);
    return rv_launch_status();
}
