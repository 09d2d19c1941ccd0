// V4 cousin of the decode path, part 3: the KV compressor (deposit, pooling, finish) and the fp8 prefix quantiser.
#include "v4_common.cuh"

namespace {

// ---------------------------------------------------------------------------------------------------
// KV compressor, decode arm: deposit one token into the pooling state; when a block closes, pool it
// (softmax over the ENTRY axis per feature), bf16 store, RMSNorm, rotate the last rd dims at the block's
// first position, then the finishing quantisation (spread for the indexer's compressor, fp8 block-64
// on the un-rotated dims for the attention compressor).
// Reference: crates/backend/kernels/kvcompress.hip (deposit / decode / pool_row / finish_row),
// crates/oracles/src/v4oracle/compress.rs:131-200.
// ---------------------------------------------------------------------------------------------------
constexpr int CP_THREADS = 256;
constexpr int CP_ENTS_MAX = 128;
constexpr float CP_FP8_MAX = 448.0f;

__device__ __forceinline__ float cp_block_sum(float v, float* red) {   // red: CP_THREADS / 32 floats
    v = rv_warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < CP_THREADS / 32; ++i) t += red[i];
    __syncthreads();
    return t;
}

// e4m3 round trip with round-to-nearest-even everywhere and saturation at 448: the hardware converter's rule.
__device__ __forceinline__ float cp_e4m3_roundtrip(float q) {
    uint16_t c;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(c) : "f"(q), "f"(0.0f));
    return rv_e4m3x2_to_f32x2(c).x;
}

// fp8 quantise-dequantise of one block of `block` values starting at seg (one warp; power-of-two scale,
// amax floor 1e-4): crates/backend/kernels/mla.hip:319-338. Exact: the maximum is associative, the rest is
// per element.
__device__ __forceinline__ void cp_act_quant_block(const float* seg, float* out, int block) {
    const int lane = threadIdx.x & 31;
    float amax = 1e-4f;
    for (int i = lane; i < block; i += 32) amax = fmaxf(amax, fabsf(seg[i]));
    amax = rv_warp_max(amax);
    const uint32_t bits = __float_as_uint(__fmul_rn(amax, __fdiv_rn(1.0f, CP_FP8_MAX)));
    const int e = (int)((bits >> 23) & 0xffu) - 127 + ((bits & 0x7fffffu) ? 1 : 0);
    const float s = __uint_as_float((uint32_t)(e + 127) << 23);
    for (int i = lane; i < block; i += 32) {
        float q = __fdiv_rn(seg[i], s);
        q = q < -CP_FP8_MAX ? -CP_FP8_MAX : (q > CP_FP8_MAX ? CP_FP8_MAX : q);
        out[i] = __fmul_rn(cp_e4m3_roundtrip(q), s);
    }
}

__global__ void cp_act_quant_f8_prefix_kernel(const float* src, float* dst, int rows, int row_stride, int n, int block) {
    const int nb = n / block;
    const size_t id = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);   // one warp per block
    if (id >= (size_t)rows * (size_t)nb) return;
    const size_t off = (size_t)(id / nb) * row_stride + (size_t)(id % nb) * block;
    cp_act_quant_block(src + off, dst + off, block);
}

struct CpState {
    float* kv;      // [ents][cd]
    float* score;   // [ents][cd]
};

// bf16 row -> RMSNorm (bf16 store) -> rotation of the last rd dims at `pos` (bf16 store), in place, by one CTA.
// red: CP_THREADS / 32 floats of shared memory.
__device__ __forceinline__ void cp_finish_row(float* row, const float* __restrict__ norm, const float* __restrict__ freqs,
                                              CompGeom p, int pos, float* red) {
    const int tid = threadIdx.x, d = p.d;
    float part = 0.0f;
    for (int e = tid; e < d; e += CP_THREADS) part += row[e] * row[e];
    const float rs = 1.0f / sqrtf(cp_block_sum(part, red) / (float)d + p.eps);
    for (int e = tid; e < d; e += CP_THREADS) row[e] = v4_rbf16(norm[e] * (row[e] * rs));
    __syncthreads();
    float* seg = row + (d - p.rd);
    for (int i = tid; i < p.rd / 2; i += CP_THREADS) {
        const float c = freqs[(size_t)pos * p.rd + 2 * i], sn = freqs[(size_t)pos * p.rd + 2 * i + 1];
        const float a = seg[2 * i], b = seg[2 * i + 1];
        seg[2 * i] = v4_rbf16(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn)));
        seg[2 * i + 1] = v4_rbf16(__fadd_rn(__fmul_rn(a, sn), __fmul_rn(b, c)));
    }
    __syncthreads();
}

// Pool + bf16 + RMSNorm + rotation of one sequence's state into row[d] (shared or global), by one CTA;
// then the overlap half of the state moves down.
__device__ __forceinline__ void cp_pool_finish(CpState st, const float* __restrict__ norm,
                                               const float* __restrict__ freqs, float* row, CompGeom p,
                                               int start_pos, float* red) {
    const int tid = threadIdx.x, d = p.d, cd = p.cd, overlap = p.coff == 2;
    for (int e = tid; e < d; e += CP_THREADS) {
        float mx = -INFINITY;
        for (int j = 0; j < p.ents; ++j) mx = fmaxf(mx, st.score[(size_t)j * cd + ((overlap && j >= p.ratio) ? d : 0) + e]);
        float o = 0.0f;
        if (isfinite(mx)) {
            float sum = 0.0f;
            for (int j = 0; j < p.ents; ++j)
                sum += expf(st.score[(size_t)j * cd + ((overlap && j >= p.ratio) ? d : 0) + e] - mx);
            for (int j = 0; j < p.ents; ++j) {
                const size_t a = (size_t)j * cd + ((overlap && j >= p.ratio) ? d : 0) + e;
                o += st.kv[a] * (expf(st.score[a] - mx) / sum);
            }
        }
        row[e] = v4_rbf16(o);
    }
    __syncthreads();
    cp_finish_row(row, norm, freqs, p, (start_pos / p.ratio) * p.ratio, red);
    if (overlap) {   // every pooling read is done (barriers above): the overlap half moves down
        const size_t n = (size_t)p.ratio * cd;
        for (size_t i = tid; i < n; i += CP_THREADS) {
            st.kv[i] = st.kv[n + i];
            st.score[i] = st.score[n + i];
        }
    }
    __syncthreads();
}

// Prefill arm: block b of a prompt that starts at position 0. Entry j of its window is row j - ratio of block b
// (second half of the projected row) or, with overlap, row j of block b - 1 (first half; absent for block 0);
// scores get the positional bias of the row's place in ITS block.
__global__ void __launch_bounds__(CP_THREADS) cp_prefill_kernel(const float* __restrict__ kv,
                                                                const float* __restrict__ score,
                                                                const float* __restrict__ ape, CompFinish f, CompGeom p) {
    __shared__ float red[CP_THREADS / 32];
    const int b = blockIdx.x, tid = threadIdx.x, d = p.d, cd = p.cd, overlap = p.coff == 2;
    float* row = f.out + (size_t)b * d;
    for (int e = tid; e < d; e += CP_THREADS) {
        float mx = -INFINITY;
        float sum = 0.0f, o = 0.0f;
        for (int pass = 0; pass < 3; ++pass) {   // 0: maximum, 1: sum of exponentials, 2: weighted values
            for (int j = 0; j < p.ents; ++j) {
                int sblk, src_j, half;
                if (!overlap) { sblk = b; src_j = j; half = 0; }
                else if (j >= p.ratio) { sblk = b; src_j = j - p.ratio; half = d; }
                else if (b > 0) { sblk = b - 1; src_j = j; half = 0; }
                else continue;
                const size_t src = (size_t)(sblk * p.ratio + src_j) * cd + half + e;
                const float sc = score[src] + ape[(size_t)src_j * cd + half + e];
                if (pass == 0) mx = fmaxf(mx, sc);
                else if (pass == 1) sum += expf(sc - mx);
                else o += kv[src] * (expf(sc - mx) / sum);
            }
            if (pass == 0 && !isfinite(mx)) break;
        }
        row[e] = v4_rbf16(isfinite(mx) ? o : 0.0f);
    }
    __syncthreads();
    cp_finish_row(row, f.norm, f.freqs, p, b * p.ratio, red);
}

__global__ void __launch_bounds__(CP_THREADS) cp_deposit_kernel(const float* __restrict__ kv,
                                                                const float* __restrict__ score,
                                                                const float* __restrict__ ape, float* kv_state,
                                                                float* score_state, CompGeom p, int s, int slot0) {
    const int remainder = s % p.ratio, cutoff = s - remainder, overlap = p.coff == 2;
    const int state_off = overlap ? p.ratio : 0;
    const size_t stride = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (overlap && cutoff >= p.ratio) {   // the last full block's rows become the overlap half
        const size_t n = (size_t)p.ratio * p.cd;
        for (size_t i = tid; i < n; i += stride) {
            const size_t src = (size_t)(cutoff - p.ratio) * p.cd + i;
            kv_state[i] = kv[src];
            score_state[i] = score[src] + ape[i];
        }
    }
    if (remainder > 0) {                  // the open block's rows, from slot0 on
        const size_t n = (size_t)remainder * p.cd, dst0 = (size_t)(state_off + slot0) * p.cd;
        for (size_t i = tid; i < n; i += stride) {
            const size_t src = (size_t)cutoff * p.cd + i;
            kv_state[dst0 + i] = kv[src];
            score_state[dst0 + i] = score[src] + ape[(size_t)slot0 * p.cd + i];
        }
    }
}

__global__ void __launch_bounds__(CP_THREADS) cp_decode_kernel(float* kv_state, float* score_state, CompFinish f,
                                                               CompGeom p, int start_pos) {
    __shared__ float red[CP_THREADS / 32];
    cp_pool_finish(CpState{kv_state, score_state}, f.norm, f.freqs, f.out, p, start_pos, red);
}

// Batched decode step: one CTA per sequence. cache row = cache + (b * cache_rows + cache_row0 + block) * d (bf16).
__global__ void __launch_bounds__(CP_THREADS) cp_step_kernel(CompGeom p, const int32_t* __restrict__ pos,
                                                             const float* __restrict__ kv_proj,
                                                             const float* __restrict__ score_proj,
                                                             const float* __restrict__ ape, float* kv_state,
                                                             float* score_state, const float* __restrict__ norm,
                                                             const float* __restrict__ freqs, int rotate,
                                                             uint16_t* __restrict__ cache, int cache_rows,
                                                             int cache_row0, float* __restrict__ prequant,
                                                             uint8_t* __restrict__ packed,
                                                             uint32_t* __restrict__ packed_exp) {
    extern __shared__ __align__(16) float cp_row[];   // [d]
    __shared__ float red[CP_THREADS / 32];
    __shared__ uint32_t exp_word;
    __shared__ int row_lo, row_hi;
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sp = pos[b], slot = sp % p.ratio, d = p.d;
    const size_t st_n = (size_t)p.ents * p.cd;
    CpState st{kv_state + (size_t)b * st_n, score_state + (size_t)b * st_n};
    const size_t dst = (size_t)((p.coff == 2 ? p.ratio : 0) + slot) * p.cd;
    for (int e = tid; e < p.cd; e += CP_THREADS) {
        st.kv[dst + e] = kv_proj[(size_t)b * p.cd + e];
        st.score[dst + e] = score_proj[(size_t)b * p.cd + e] + ape[(size_t)slot * p.cd + e];
    }
    if ((sp + 1) % p.ratio != 0) return;   // the block is still open
    __syncthreads();
    cp_pool_finish(st, norm, freqs, cp_row, p, sp, red);
    if (prequant) for (int e = tid; e < d; e += CP_THREADS) prequant[(size_t)b * d + e] = cp_row[e];
    if (rotate) {
        // the spread of blockindex.hip:97-138 on the row in shared memory
        for (int h = 1; h < d; h <<= 1) {
            for (int t = tid; t < (d >> 1); t += CP_THREADS) {
                const int j = 2 * t - (t & (h - 1));
                const float a = cp_row[j], c = cp_row[j + h];
                cp_row[j] = __fadd_rn(a, c);
                cp_row[j + h] = __fsub_rn(a, c);
            }
            __syncthreads();
        }
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)d));
        for (int i = tid; i < d; i += CP_THREADS) cp_row[i] = v4_rbf16(__fmul_rn(cp_row[i], scale));
        __syncthreads();
        const float floor_ = __fmul_rn(V4_FP4_MAX, __uint_as_float(1u << 23));
        for (int blk = warp; blk < d / 32; blk += CP_THREADS / 32) {
            const float v = cp_row[blk * 32 + lane];
            const float s = v4_round_scale(fmaxf(rv_warp_max(fabsf(v)), floor_));
            float q = __fdiv_rn(v, s);
            q = q < -V4_FP4_MAX ? -V4_FP4_MAX : (q > V4_FP4_MAX ? V4_FP4_MAX : q);
            cp_row[blk * 32 + lane] = __fmul_rn(v4_e2m1_roundtrip(q), s);
        }
    } else {
        // fp8 block-64 on the dims that were not rotated (crates/oracles/src/v4oracle/compress.rs:235-247)
        for (int blk = warp; blk < (d - p.rd) / 64; blk += CP_THREADS / 32) cp_act_quant_block(cp_row + blk * 64, cp_row + blk * 64, 64);
    }
    if (tid == 0) { exp_word = 0u; row_lo = 1000; row_hi = -1000; }
    __syncthreads();
    uint16_t* out = cache + ((size_t)b * cache_rows + cache_row0 + sp / p.ratio) * d;
    for (int e = tid; e < d; e += CP_THREADS) out[e] = rv_f32_to_bf16(cp_row[e]);
    if (packed) {
        // the scorer's second form of the same row (d == 128, cache_rows rows per sequence): int8 multiples of the row's
        // unit 2^(pmin - 130), pmin = the smallest biased exponent any non-empty block's largest magnitude has; the
        // row's word holds pmin, 0 for an all-zero row, 0xff when the row is not of that form (blocks more than 3
        // binades apart, magnitudes outside 2^-40 .. 2^40)
        const size_t prow = (size_t)b * cache_rows + cache_row0 + sp / p.ratio;
        float v = 0.0f;
        if (warp < 4) {
            v = rv_bf16_to_f32(rv_f32_to_bf16(cp_row[warp * 32 + lane]));
            int pb = (int)((__float_as_uint(v) >> 23) & 0xffu);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) pb = max(pb, __shfl_xor_sync(0xffffffffu, pb, o));
            if (lane == 0 && pb > 0) { atomicMin(&row_lo, pb); atomicMax(&row_hi, pb); }
        }
        __syncthreads();
        const int lo = row_lo, hi = row_hi;
        const bool form = hi < lo || (lo >= 87 && hi <= 167 && hi - lo <= 3);
        if (warp < 4) {
            const float x = (form && hi >= lo) ? v * __int_as_float((257 - lo) << 23) : 0.0f;
            const int m = __float2int_rn(x);
            bool ok = form && (float)m == x && (hi >= lo || (__float_as_uint(v) & 0x7fffffffu) == 0);
            ok = __all_sync(0xffffffffu, ok);
            packed[prow * 128 + warp * 32 + lane] = (uint8_t)(m & 0xff);
            if (lane == 0 && !ok) atomicOr(&exp_word, 1u);
        }
        __syncthreads();
        if (tid == 0) packed_exp[prow] = exp_word ? 0xffu : (hi >= lo ? (uint32_t)lo : 0u);
    }
}

static int cp_guard(const CompGeom& p) {
    if (p.ratio <= 1 || p.d <= 0 || p.rd <= 0 || p.coff < 1 || p.coff > 2) return 1001;
    if (p.rd > p.d || (p.rd & 1)) return 1002;
    if (p.cd != p.coff * p.d || p.ents != p.coff * p.ratio) return 1003;
    if (p.ents > CP_ENTS_MAX) return 1004;
    if ((p.coff == 2) != (p.ratio == 4)) return 1010;
    return 0;
}
}  // namespace

RIVOLI_API int rivoli_act_quant_f8_prefix(const float* src, float* dst, int rows, int row_stride, int n, int block,
                                          void* stream) {
    if (rows <= 0 || n <= 0 || block <= 0 || row_stride < n) return 1001;
    if (src != dst && n != row_stride) return 1002;   // the untouched tail of a row only survives in place
    if (n % block) return 1004;
    const size_t total = (size_t)rows * (size_t)(n / block);
    rv_drain_error();
    cp_act_quant_f8_prefix_kernel<<<(unsigned)((total + 7) / 8), 256, 0, (cudaStream_t)stream>>>(src, dst, rows, row_stride,
                                                                                                n, block);
    return rv_launch_status();
}

RIVOLI_API int rivoli_kv_compress_deposit(const float* kv, const float* score, const float* ape, float* kv_state,
                                          float* score_state, const CompGeom* pp, int s, int slot0, void* stream) {
    if (!pp) return 1000;
    const CompGeom p = *pp;
    if (int g = cp_guard(p)) return g;
    if (s <= 0) return 1005;
    if (slot0 < 0 || slot0 + s % p.ratio > p.ratio) return 1008;
    const int rem = s % p.ratio;
    const size_t n = (size_t)(p.ratio > rem ? p.ratio : rem) * p.cd;
    rv_drain_error();
    cp_deposit_kernel<<<(unsigned)((n + CP_THREADS - 1) / CP_THREADS), CP_THREADS, 0, (cudaStream_t)stream>>>(
        kv, score, ape, kv_state, score_state, p, s, slot0);
    return rv_launch_status();
}

RIVOLI_API int rivoli_kv_compress_prefill(const float* kv, const float* score, const float* ape, const CompFinish* ff,
                                          const CompGeom* pp, int nblk, void* stream) {
    if (!pp || !ff) return 1000;
    const CompGeom p = *pp;
    if (int g = cp_guard(p)) return g;
    if (nblk <= 0) return 1006;
    rv_drain_error();
    cp_prefill_kernel<<<(unsigned)nblk, CP_THREADS, 0, (cudaStream_t)stream>>>(kv, score, ape, *ff, p);
    return rv_launch_status();
}

RIVOLI_API int rivoli_kv_compress_decode(float* kv_state, float* score_state, const CompFinish* ff, const CompGeom* pp,
                                         int start_pos, void* stream) {
    if (!pp || !ff) return 1000;
    const CompGeom p = *pp;
    if (int g = cp_guard(p)) return g;
    if (start_pos <= 0) return 1007;                 // position 0 belongs to the prefill arm
    if ((start_pos + 1) % p.ratio != 0) return 1009; // the block has not closed
    rv_drain_error();
    cp_decode_kernel<<<1, CP_THREADS, 0, (cudaStream_t)stream>>>(kv_state, score_state, *ff, p, start_pos);
    return rv_launch_status();
}

RIVOLI_API int rivoli_v4_compress_step_bf16(const CompGeom* pp, int n_seqs, const int32_t* pos, const float* kv_proj,
                                            const float* score_proj, const float* ape, float* kv_state,
                                            float* score_state, const float* norm, const float* freqs, int rotate,
                                            uint16_t* cache, int cache_rows, int cache_row0, float* prequant,
                                            unsigned char* packed, uint32_t* packed_exp, void* stream) {
    if (!pp) return 1000;
    const CompGeom p = *pp;
    if (int g = cp_guard(p)) return g;
    if (n_seqs <= 0 || cache_rows <= 0 || cache_row0 < 0) return 1001;
    if (rotate && (p.d > V4_ROT_MAX || (p.d & (p.d - 1)) || p.d % 32)) return 1002;
    if (!rotate && (p.d - p.rd) % 64) return 1004;
    if ((packed != nullptr) != (packed_exp != nullptr)) return 1001;
    if (packed && (!rotate || p.d != 128)) return 1002;   // the packed form is the indexer's: spread rows of width 128
    if ((size_t)p.d * 4 > 48 * 1024) return 1002;
    rv_drain_error();
    cp_step_kernel<<<(unsigned)n_seqs, CP_THREADS, (size_t)p.d * 4, (cudaStream_t)stream>>>(
        p, pos, kv_proj, score_proj, ape, kv_state, score_state, norm, freqs, rotate, cache, cache_rows, cache_row0, prequant,
        packed, packed_exp);
    return rv_launch_status();
}
