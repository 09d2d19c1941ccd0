// V4 cousin of the decode path: Hadamard + fp4 spread, block scorer, scored block selection and MQA
// sparse attention with a per-head sink.
//
// Reference behaviour: crates/backend/kernels/blockindex.hip:97-138,234-306 (spread, block scorer),
// crates/backend/kernels/attn.hip:358-465 (gather attention), crates/engine/src/v4/select.rs:153-232
// (selection rows). The spread, the scores and the selected indices are bit-exact against the host
// rules: every add and multiply on those paths is an explicit round-to-nearest intrinsic, so nothing
// is contracted into a fused multiply-add, and every fold runs in the host's order.
//
// Storage on this side is bf16 (the reference keeps bf16 VALUES in f32 arrays: every producer on the
// path ends in a bf16 store), which halves the gathered bytes and feeds the tensor cores directly.
#include "codec.cuh"
#include "common.cuh"
#include "topk_core.cuh"

namespace {

__device__ __forceinline__ float v4_rbf16(float x) { return rv_bf16_to_f32(rv_f32_to_bf16(x)); }

// ---------------------------------------------------------------------------------------------------
// spread
// ---------------------------------------------------------------------------------------------------
constexpr int V4_ROT_MAX = 256;
constexpr float V4_FP4_MAX = 6.0f;

// e2m1 round trip of q (already clamped to [-6, 6]): nearest grid point, midpoints to the even code.
__device__ __forceinline__ float v4_e2m1_roundtrip(float q) {
    const float a = fabsf(q);
    int code = 0;
    code += a > 0.25f;
    code += a >= 0.75f;
    code += a > 1.25f;
    code += a >= 1.75f;
    code += a > 2.5f;
    code += a >= 3.5f;
    code += a > 5.0f;
    const float mag = code < 4 ? 0.5f * (float)code : (code == 4 ? 2.0f : (code == 5 ? 3.0f : (code == 6 ? 4.0f : 6.0f)));
    return signbit(q) ? -mag : mag;
}

// Smallest power of two >= amax / 6, from the exponent field of the product.
__device__ __forceinline__ float v4_round_scale(float amax) {
    const uint32_t b = __float_as_uint(__fmul_rn(amax, __fdiv_rn(1.0f, V4_FP4_MAX)));
    const int e = (int)((b >> 23) & 0xffu) - 127 + ((b & 0x7fffffu) ? 1 : 0);
    return __uint_as_float((uint32_t)(e + 127) << 23);
}

// One CTA per row. The butterfly visits the operand pairs (j, j + h) stage by stage exactly as the host
// loop does; which thread evaluates a pair does not change the value.
__global__ void __launch_bounds__(128) v4_spread_kernel(float* __restrict__ x, int d) {
    __shared__ float sh[V4_ROT_MAX];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float* row = x + (size_t)blockIdx.x * d;
    for (int i = tid; i < d; i += 128) sh[i] = row[i];
    __syncthreads();
    for (int h = 1; h < d; h <<= 1) {
        for (int t = tid; t < (d >> 1); t += 128) {
            const int j = 2 * t - (t & (h - 1));
            const float a = sh[j], b = sh[j + h];
            sh[j] = __fadd_rn(a, b);
            sh[j + h] = __fsub_rn(a, b);
        }
        __syncthreads();
    }
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)d));
    for (int i = tid; i < d; i += 128) sh[i] = v4_rbf16(__fmul_rn(sh[i], scale));
    __syncthreads();
    // one warp per block of 32: the maximum is exact under any association
    const float floor_ = __fmul_rn(V4_FP4_MAX, __uint_as_float(1u << 23));
    for (int b = warp; b < d / 32; b += 4) {
        const float v = sh[b * 32 + lane];
        const float amax = fmaxf(rv_warp_max(fabsf(v)), floor_);
        const float s = v4_round_scale(amax);
        float q = __fdiv_rn(v, s);
        q = q < -V4_FP4_MAX ? -V4_FP4_MAX : (q > V4_FP4_MAX ? V4_FP4_MAX : q);
        sh[b * 32 + lane] = v4_rbf16(__fmul_rn(v4_e2m1_roundtrip(q), s));
    }
    __syncthreads();
    for (int i = tid; i < d; i += 128) row[i] = sh[i];
}

// ---------------------------------------------------------------------------------------------------
// block scorer
// ---------------------------------------------------------------------------------------------------
constexpr int SC_CB = 4;          // blocks a warp scores per iteration
constexpr int SC_MAX_HEADS = 64;  // two lanes-worth of heads
constexpr int SC_MAX_HD = 128;

__device__ __forceinline__ float v4_load_f32(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float v4_load_f32(const uint16_t* p, size_t i) { return rv_bf16_to_f32(p[i]); }

// Scores of blocks [c0, c0 + SC_CB) for one query row, by one warp. Lane l owns heads l and l + 32: each
// dot is an ascending fold over the hd terms (separate multiply and add), exactly the host's; the head
// sum is then an ascending f32 fold over the bf16 terms, evaluated redundantly by every lane.
// qT: shared [hd][64] f32 (transposed: lanes read consecutive words); wsh: shared [64] f32;
// stage: this warp's shared [SC_CB][hd] f32. Returns through out[SC_CB] (same value in every lane).
template <class T>
__device__ __forceinline__ void v4_score_blocks_warp(const float* __restrict__ qT, const float* __restrict__ wsh,
                                                     float* __restrict__ stage, const T* __restrict__ kv, int c0,
                                                     int n_comp, int heads, int hd, float (&out)[SC_CB]) {
    const int lane = threadIdx.x & 31;
    __syncwarp();
    for (int i = lane; i < SC_CB * hd; i += 32) {
        const int cb = i / hd, e = i - cb * hd;
        stage[i] = c0 + cb < n_comp ? v4_load_f32(kv, (size_t)(c0 + cb) * hd + e) : 0.0f;
    }
    __syncwarp();
    float dot[SC_CB][2];
#pragma unroll
    for (int cb = 0; cb < SC_CB; ++cb) dot[cb][0] = dot[cb][1] = 0.0f;
    for (int i = 0; i < hd; i += 4) {
        float4 kvv[SC_CB];
#pragma unroll
        for (int cb = 0; cb < SC_CB; ++cb) kvv[cb] = *reinterpret_cast<const float4*>(stage + cb * hd + i);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float q0 = qT[(i + e) * SC_MAX_HEADS + lane], q1 = qT[(i + e) * SC_MAX_HEADS + 32 + lane];
#pragma unroll
            for (int cb = 0; cb < SC_CB; ++cb) {
                const float kvx = e == 0 ? kvv[cb].x : (e == 1 ? kvv[cb].y : (e == 2 ? kvv[cb].z : kvv[cb].w));
                dot[cb][0] = __fadd_rn(dot[cb][0], __fmul_rn(q0, kvx));
                dot[cb][1] = __fadd_rn(dot[cb][1], __fmul_rn(q1, kvx));
            }
        }
    }
    const float w0 = wsh[lane], w1 = wsh[32 + lane];
#pragma unroll
    for (int cb = 0; cb < SC_CB; ++cb) {
        // bf16 store, relu, times the (signed) head weight, bf16 store
        const float t0 = v4_rbf16(__fmul_rn(fmaxf(v4_rbf16(dot[cb][0]), 0.0f), w0));
        const float t1 = v4_rbf16(__fmul_rn(fmaxf(v4_rbf16(dot[cb][1]), 0.0f), w1));
        float acc = 0.0f;
        const int n0 = heads < 32 ? heads : 32;
        for (int hh = 0; hh < n0; ++hh) acc = __fadd_rn(acc, __shfl_sync(0xffffffffu, t0, hh));
        for (int hh = 32; hh < heads; ++hh) acc = __fadd_rn(acc, __shfl_sync(0xffffffffu, t1, hh - 32));
        out[cb] = v4_rbf16(acc);
    }
}

// Stage one query row's index q transposed ([hd][64], zero beyond `heads`) and its head weights.
template <class T>
__device__ __forceinline__ void v4_stage_q(const T* __restrict__ q, const float* __restrict__ w, int heads, int hd,
                                           float* __restrict__ qT, float* __restrict__ wsh) {
    for (int i = threadIdx.x; i < hd * SC_MAX_HEADS; i += blockDim.x) {
        const int e = i / SC_MAX_HEADS, hh = i - e * SC_MAX_HEADS;
        qT[i] = hh < heads ? v4_load_f32(q, (size_t)hh * hd + e) : 0.0f;
    }
    for (int i = threadIdx.x; i < SC_MAX_HEADS; i += blockDim.x) wsh[i] = i < heads ? w[i] : 0.0f;
}

constexpr int SCK_THREADS = 256;
constexpr int SCK_BLOCKS_PER_CTA = 256;   // blocks one CTA of the one-sequence scorer covers

// Reference-layout scorer: f32 arrays, s query rows against one shared block array.
__global__ void __launch_bounds__(SCK_THREADS) v4_score_blocks_kernel(const float* __restrict__ q,
                                                                      const float* __restrict__ kv,
                                                                      const float* __restrict__ w,
                                                                      float* __restrict__ score, int n_comp, int heads,
                                                                      int hd) {
    extern __shared__ __align__(16) float sc_smem[];
    float* qT = sc_smem;
    float* wsh = qT + hd * SC_MAX_HEADS;
    float* stage = wsh + SC_MAX_HEADS;
    const int t = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    v4_stage_q(q + (size_t)t * heads * hd, w + (size_t)t * heads, heads, hd, qT, wsh);
    __syncthreads();
    const int c_begin = blockIdx.x * SCK_BLOCKS_PER_CTA;
    const int c_end = min(n_comp, c_begin + SCK_BLOCKS_PER_CTA);
    for (int c0 = c_begin + warp * SC_CB; c0 < c_end; c0 += (SCK_THREADS / 32) * SC_CB) {
        float out[SC_CB];
        v4_score_blocks_warp(qT, wsh, stage + warp * SC_CB * hd, kv, c0, n_comp, heads, hd, out);
        if (lane < SC_CB && c0 + lane < c_end) {
            float v = out[0];
#pragma unroll
            for (int cb = 1; cb < SC_CB; ++cb) v = lane == cb ? out[cb] : v;
            score[(size_t)t * n_comp + c0 + lane] = v;
        }
    }
}

// Any shape: one thread per (t, c), everything sequential.
__global__ void v4_score_blocks_serial_kernel(const float* __restrict__ q, const float* __restrict__ kv,
                                              const float* __restrict__ w, float* __restrict__ score, int s,
                                              int n_comp, int heads, int hd) {
    const size_t id = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= (size_t)s * (size_t)n_comp) return;
    const int t = (int)(id / (size_t)n_comp), c = (int)(id % (size_t)n_comp);
    float acc = 0.0f;
    for (int hh = 0; hh < heads; ++hh) {
        const float* qh = q + ((size_t)t * heads + hh) * hd;
        float dot = 0.0f;
        for (int i = 0; i < hd; ++i) dot = __fadd_rn(dot, __fmul_rn(qh[i], kv[(size_t)c * hd + i]));
        dot = fmaxf(v4_rbf16(dot), 0.0f);
        acc = __fadd_rn(acc, v4_rbf16(__fmul_rn(dot, w[(size_t)t * heads + hh])));
    }
    score[id] = v4_rbf16(acc);
}

// ---------------------------------------------------------------------------------------------------
// block scorer on the integer tensor cores, exact
//
// Rows that came through the spread are, block of 32 by block of 32, small integers times one power of
// two: v = m * 2^e with |m| < 16 once e = (exponent of the block's largest magnitude) - 3. A block's share of
// a dot product is then I_j * 2^(eq_j + ek_j) with I_j = sum of 32 integer products, which
// mma.m16n8k32.s8 returns exactly (K = 32 is one block). The host's ascending f32 fold over the 128
// products never rounds as long as every partial sum is representable: all of them are multiples of
// 2^Emin and smaller than 2^(Emax + 15) (4 blocks x 32 terms x 15 x 15 < 2^15), so Emax - Emin <= 9
// suffices, and then the fold equals the exact sum, which is what sum_j float(I_j) * 2^E_j gives here.
// Everything after the dot (bf16 store, relu, head weight, bf16 store, ascending head sum) is evaluated
// in the host's order on CUDA cores. A pair that misses the condition, or a row that is not of that form
// (a value that is not an integer multiple of its block's unit, a subnormal, an exponent near the range
// ends), raises the sequence's flag and the selection kernel re-scores that sequence with the ordered
// CUDA-core fold: the result is exact either way.
// ---------------------------------------------------------------------------------------------------
constexpr int SI_THREADS = 256;
constexpr int SI_CHUNK = 256;       // blocks (columns) per CTA
constexpr int SI_SPAN = 9;

__device__ __forceinline__ void v4_mma_s8(int (&d)[4], const uint4& a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ float v4_rbf16_hw(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }  // finite inputs

// Largest biased exponent among the bf16 values packed in w0, w1.
__device__ __forceinline__ int v4_max_exp4(uint32_t w0, uint32_t w1) {
    const uint32_t a = max(w0 & 0x7f800000u, w1 & 0x7f800000u), b = max((w0 << 16) & 0x7f800000u, (w1 << 16) & 0x7f800000u);
    return (int)(max(a, b) >> 23);
}
// Four bf16 values (two words) times `scale` (a power of two) -> four int8. ok is cleared when a product is
// not an integer (the value is not a multiple of the block's unit).
__device__ __forceinline__ uint32_t v4_pack4(uint32_t w0, uint32_t w1, float scale, bool& ok) {
    const float x0 = __uint_as_float(w0 << 16) * scale, x1 = __uint_as_float(w0 & 0xffff0000u) * scale;
    const float x2 = __uint_as_float(w1 << 16) * scale, x3 = __uint_as_float(w1 & 0xffff0000u) * scale;
    const int m0 = __float2int_rn(x0), m1 = __float2int_rn(x1), m2 = __float2int_rn(x2), m3 = __float2int_rn(x3);
    ok = ok && (float)m0 == x0 && (float)m1 == x1 && (float)m2 == x2 && (float)m3 == x3;
    if (scale == 0.0f) ok = ok && ((w0 | w1) & 0x7fff7fffu) == 0;   // an "empty" block must really be zeros
    // cvt.pack d, a, b, c: d[7:0] = sat(b), d[15:8] = sat(a), d[31:16] = c[15:0]
    uint32_t hi, out;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(m3), "r"(m2), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(m1), "r"(m0), "r"(hi));
    return out;
}
// 2^(130 - pb): turns values of a block whose largest exponent is pb into integers below 16. Blocks whose
// exponent sits at the very bottom of the range are left to the ordered fold.
__device__ __forceinline__ float v4_unit_inv(int pb, bool& ok) {
    if (pb < 4) { ok = ok && pb == 0; return 0.0f; }
    return __int_as_float((257 - pb) << 23);
}
// 2^(pb - 130), or 0 for an empty block.
__device__ __forceinline__ float v4_unit(int pb) { return pb < 4 ? 0.0f : __int_as_float((pb - 3) << 23); }

// PACKED: the rows come as int8 + block exponents (rivoli_v4_index_pack_bf16), written once when a row enters
// the cache; otherwise every row is converted from bf16 on every step.
template <bool PACKED>
__global__ void __launch_bounds__(SI_THREADS) v4_score_int8_kernel(V4Geom g, const int32_t* __restrict__ pos,
                                                                   const uint16_t* __restrict__ index_q,
                                                                   const float* __restrict__ index_w,
                                                                   const uint16_t* __restrict__ index_kv,
                                                                   const uint8_t* __restrict__ packed,
                                                                   const uint32_t* __restrict__ packed_exp,
                                                                   float* __restrict__ scores,
                                                                   int32_t* __restrict__ flags) {
    __shared__ __align__(16) uint32_t qfrag[4 * 4 * 32 * 4];   // [m-tile][block][lane][4 regs]: A fragments, 8 KB
    __shared__ __align__(16) float qunit[64][4];               // per head: 2^(e - 130) of its four blocks (0 = empty)
    __shared__ float wsh[64];
    __shared__ int qstat[3];                                   // over the heads: min / max block exponent, widest span
    __shared__ __align__(16) float terms[SI_THREADS / 32][64][8];   // written as float2: needs the alignment
    const int b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_comp = min((pos[b] + 1) / g.ratio, g.max_comp);
    const int c_begin = blockIdx.x * SI_CHUNK;
    if (n_comp <= g.index_topk || c_begin >= n_comp) return;   // positional sequences are not scored
    const int heads = g.index_heads;
    bool ok = true;
    if (tid == 0) { qstat[0] = 1000; qstat[1] = -1000; qstat[2] = 0; }
    __syncthreads();
    // ---- q of this sequence: one thread per (head, block of 32)
    {
        const int hh = tid >> 2, j = tid & 3;
        uint32_t wv[16];
        int pb = 0;
        if (hh < heads) {
            const uint4* src = reinterpret_cast<const uint4*>(index_q + ((size_t)b * heads + hh) * 128 + j * 32);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 v = src[i];
                wv[4 * i] = v.x; wv[4 * i + 1] = v.y; wv[4 * i + 2] = v.z; wv[4 * i + 3] = v.w;
            }
#pragma unroll
            for (int i = 0; i < 16; i += 2) pb = max(pb, v4_max_exp4(wv[i], wv[i + 1]));
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) wv[i] = 0;
        }
        const float inv = v4_unit_inv(pb, ok);
        const int mt = hh >> 4, r = hh & 15;
#pragma unroll
        for (int k4 = 0; k4 < 8; ++k4) {                       // values 4 k4 .. 4 k4 + 3 of the block
            const uint32_t packed = v4_pack4(wv[2 * k4], wv[2 * k4 + 1], inv, ok);
            const int kk = 4 * k4, fl = (r & 7) * 4 + ((kk & 15) >> 2), reg = (r >> 3) + 2 * (kk >> 4);
            qfrag[((mt * 4 + j) * 32 + fl) * 4 + reg] = packed;
        }
        qunit[hh][j] = v4_unit(pb);
        // exponent range of the head's non-empty blocks (its four threads are neighbours)
        int lo = pb >= 4 ? pb : 1000, hi = pb >= 4 ? pb : -1000;
        lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, 1)); hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, 1));
        lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, 2)); hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, 2));
        if (j == 0 && hi >= lo) { atomicMin(&qstat[0], lo); atomicMax(&qstat[1], hi); atomicMax(&qstat[2], hi - lo); }
        if (tid < 64) wsh[tid] = tid < heads ? index_w[(size_t)b * heads + tid] : 0.0f;
    }
    __syncthreads();
    const int q_lo = qstat[0], q_hi = qstat[1], q_span = qstat[2];
    const uint16_t* kv = index_kv + (size_t)b * g.max_comp * 128;
    const int grp = lane >> 2, quad = lane & 3;
    const int c_end = min(n_comp, c_begin + SI_CHUNK);
    for (int c0 = c_begin + warp * 8; c0 < c_end; c0 += (SI_THREADS / 32) * 8) {
        // ---- B fragments: row c0 + grp, this thread's 8 values of each block
        const int c = c0 + grp;
        uint32_t b0[4], b1[4];
        float ku[4];
        int k_lo = 1000, k_hi = -1000;
        if (PACKED) {
            const uint8_t* prow = packed + ((size_t)b * g.max_comp + c) * 128;
            const uint32_t e4 = c < n_comp ? packed_exp[(size_t)b * g.max_comp + c] : 0u;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                b0[j] = b1[j] = 0u;
                if (c < n_comp) {
                    b0[j] = *reinterpret_cast<const uint32_t*>(prow + j * 32 + quad * 4);
                    b1[j] = *reinterpret_cast<const uint32_t*>(prow + j * 32 + 16 + quad * 4);
                }
                const int pb = (e4 >> (8 * j)) & 0xff;
                if (pb == 0xff) ok = false;                 // the packer could not take this block
                ku[j] = pb == 0xff ? 0.0f : v4_unit(pb);
                if (pb >= 4 && pb != 0xff) { k_lo = min(k_lo, pb); k_hi = max(k_hi, pb); }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint2 lo = make_uint2(0, 0), hi = make_uint2(0, 0);
                if (c < n_comp) {
                    lo = *reinterpret_cast<const uint2*>(kv + (size_t)c * 128 + j * 32 + quad * 4);
                    hi = *reinterpret_cast<const uint2*>(kv + (size_t)c * 128 + j * 32 + 16 + quad * 4);
                }
                int pb = max(v4_max_exp4(lo.x, lo.y), v4_max_exp4(hi.x, hi.y));
                pb = max(pb, __shfl_xor_sync(0xffffffffu, pb, 1));
                pb = max(pb, __shfl_xor_sync(0xffffffffu, pb, 2));
                const float inv = v4_unit_inv(pb, ok);
                b0[j] = v4_pack4(lo.x, lo.y, inv, ok);
                b1[j] = v4_pack4(hi.x, hi.y, inv, ok);
                ku[j] = v4_unit(pb);
                if (pb >= 4) { k_lo = min(k_lo, pb); k_hi = max(k_hi, pb); }
            }
        }
        // Every (head, this row) pair: block exponents E_j = eq_j + ek_j - 260 span at most span_q + span_k, and lie
        // inside [q_lo + k_lo, q_hi + k_hi] - 260. Inside the limits the ordered f32 fold is exact.
        if (k_hi >= k_lo && q_hi >= q_lo &&
            (q_span + (k_hi - k_lo) > SI_SPAN || q_lo + k_lo - 260 < -120 || q_hi + k_hi - 260 > 100))
            ok = false;
        // units of the two columns this thread's accumulators belong to
        float kuA[4], kuB[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            kuA[j] = __shfl_sync(0xffffffffu, ku[j], (quad * 2) * 4);
            kuB[j] = __shfl_sync(0xffffffffu, ku[j], (quad * 2 + 1) * 4);
        }
#pragma unroll 1
        for (int mt = 0; mt < 4; ++mt) {
            int acc[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 a = *reinterpret_cast<const uint4*>(&qfrag[((mt * 4 + j) * 32 + lane) * 4]);
                v4_mma_s8(acc[j], a, b0[j], b1[j]);
            }
#pragma unroll
            for (int rh = 0; rh < 2; ++rh) {                   // row half of the accumulator
                const int hh = 16 * mt + grp + 8 * rh;
                const float4 qu = *reinterpret_cast<const float4*>(qunit[hh]);
                const float wv = wsh[hh];
                float dA = 0.0f, dB = 0.0f;
                dA = fmaf((float)acc[0][2 * rh], qu.x * kuA[0], dA); dB = fmaf((float)acc[0][2 * rh + 1], qu.x * kuB[0], dB);
                dA = fmaf((float)acc[1][2 * rh], qu.y * kuA[1], dA); dB = fmaf((float)acc[1][2 * rh + 1], qu.y * kuB[1], dB);
                dA = fmaf((float)acc[2][2 * rh], qu.z * kuA[2], dA); dB = fmaf((float)acc[2][2 * rh + 1], qu.z * kuB[2], dB);
                dA = fmaf((float)acc[3][2 * rh], qu.w * kuA[3], dA); dB = fmaf((float)acc[3][2 * rh + 1], qu.w * kuB[3], dB);
                // bf16 store, relu, times the (signed) head weight, bf16 store
                const float tA = v4_rbf16_hw(__fmul_rn(fmaxf(v4_rbf16_hw(dA), 0.0f), wv));
                const float tB = v4_rbf16_hw(__fmul_rn(fmaxf(v4_rbf16_hw(dB), 0.0f), wv));
                *reinterpret_cast<float2*>(&terms[warp][hh][quad * 2]) = make_float2(tA, tB);
            }
        }
        __syncwarp();
        if (lane < 8 && c0 + lane < c_end) {
            float acc = 0.0f;
#pragma unroll 8
            for (int hh = 0; hh < heads; ++hh) acc = __fadd_rn(acc, terms[warp][hh][lane]);
            scores[(size_t)b * g.max_comp + c0 + lane] = v4_rbf16_hw(acc);
        }
        __syncwarp();
    }
    if (!ok) atomicOr(&flags[b], 1);
}

// One thread per (row, block of 32): the block's values as int8 multiples of 2^(pb - 130), pb = biased exponent of the
// block's largest magnitude, stored in the row's exponent word (0 = empty block, 0xff = not of the integer form: the
// scorer then hands the sequence to the ordered fold, which reads the bf16 rows).
__global__ void v4_index_pack_kernel(V4Geom g, const int32_t* __restrict__ row_begin, const int32_t* __restrict__ row_end,
                                     const uint16_t* __restrict__ index_kv, uint8_t* __restrict__ packed,
                                     uint32_t* __restrict__ packed_exp) {
    const int b = blockIdx.y;
    const int r0 = row_begin ? row_begin[b] : 0, r1 = min(row_end[b], g.max_comp);
    const int id = blockIdx.x * blockDim.x + threadIdx.x, row = r0 + (id >> 2), j = id & 3;
    uint32_t e = 0;
    if (row < r1) {
        const size_t off = ((size_t)b * g.max_comp + row) * 128 + j * 32;
        const uint4* src = reinterpret_cast<const uint4*>(index_kv + off);
        uint32_t wv[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 v = src[i];
            wv[4 * i] = v.x; wv[4 * i + 1] = v.y; wv[4 * i + 2] = v.z; wv[4 * i + 3] = v.w;
        }
        int pb = 0;
#pragma unroll
        for (int i = 0; i < 16; i += 2) pb = max(pb, v4_max_exp4(wv[i], wv[i + 1]));
        bool ok = pb < 0xff;
        const float inv = v4_unit_inv(pb, ok);
        uint32_t out[8];
#pragma unroll
        for (int k4 = 0; k4 < 8; ++k4) out[k4] = v4_pack4(wv[2 * k4], wv[2 * k4 + 1], inv, ok);
        uint4* dst = reinterpret_cast<uint4*>(packed + off);
        dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
        dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
        e = (uint32_t)(ok ? pb : 0xff) << (8 * j);
    }
    // the four blocks of a row sit in four neighbouring threads
    e |= __shfl_xor_sync(0xffffffffu, e, 1);
    e |= __shfl_xor_sync(0xffffffffu, e, 2);
    if (row < r1 && j == 0) packed_exp[(size_t)b * g.max_comp + row] = e;
}

// ---------------------------------------------------------------------------------------------------
// batched selection: window row + positional or scored compressed columns, one CTA per sequence
// ---------------------------------------------------------------------------------------------------
constexpr int SEL_MAX_COMP = 16384;

// f32 total order (sign-magnitude), the order the reference ranks by: -0.0 below +0.0.
__device__ __forceinline__ uint32_t v4_total_key(float v) {
    const uint32_t b = __float_as_uint(v);
    return b ^ ((uint32_t)((int32_t)b >> 31) | 0x80000000u);
}

struct SelSmem {
    TkShared tk;
    float wsh[SC_MAX_HEADS];
};

__global__ void __launch_bounds__(TK_THREADS) v4_select_kernel(V4Geom g, const int32_t* __restrict__ pos,
                                                               const uint16_t* __restrict__ index_q,
                                                               const float* __restrict__ index_w,
                                                               const uint16_t* __restrict__ index_kv,
                                                               int32_t* __restrict__ sel,
                                                               float* __restrict__ scores,
                                                               const int32_t* __restrict__ flags, int force_fold) {
    extern __shared__ __align__(16) unsigned char sel_smem_raw[];
    SelSmem& sh = *reinterpret_cast<SelSmem*>(sel_smem_raw);
    float* qT = reinterpret_cast<float*>(sel_smem_raw + ((sizeof(SelSmem) + 15) & ~(size_t)15));
    float* stage = qT + g.index_dim * SC_MAX_HEADS;
    float* sc = stage + TK_WARPS * SC_CB * g.index_dim;
    uint32_t* picked = reinterpret_cast<uint32_t*>(sc + g.max_comp);

    const int b = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    rv_grid_dep_trigger();   // the attention kernel may start staging its queries
    const int W = g.window, K = g.index_topk, p = pos[b];
    int32_t* row = sel + (size_t)b * (W + K);
    // the ring: oldest first once full, live slots then -1 before that
    if (p >= W - 1) {
        const int cut = p % W;
        for (int j = tid; j < W; j += TK_THREADS) row[j] = j < W - 1 - cut ? cut + 1 + j : j - (W - 1 - cut);
    } else {
        for (int j = tid; j < W; j += TK_THREADS) row[j] = j <= p ? j : -1;
    }
    int n_comp = (p + 1) / g.ratio;
    n_comp = n_comp < g.max_comp ? n_comp : g.max_comp;
    if (n_comp <= K) {   // every closed block, in order
        for (int c = tid; c < K; c += TK_THREADS) row[W + c] = c < n_comp ? W + c : -1;
        return;
    }
    float* srow = scores + (size_t)b * g.max_comp;
    rv_grid_dep_wait();      // the scorer's rows and flags
    if (force_fold || flags[b]) {
        // the ordered CUDA-core fold: rows the integer scorer could not take, or every row on request
        v4_stage_q(index_q + (size_t)b * g.index_heads * g.index_dim, index_w + (size_t)b * g.index_heads, g.index_heads,
                   g.index_dim, qT, sh.wsh);
        __syncthreads();
        const uint16_t* kv = index_kv + (size_t)b * g.max_comp * g.index_dim;
        for (int c0 = warp * SC_CB; c0 < n_comp; c0 += TK_WARPS * SC_CB) {
            float out[SC_CB];
            v4_score_blocks_warp(qT, sh.wsh, stage + warp * SC_CB * g.index_dim, kv, c0, n_comp, g.index_heads,
                                 g.index_dim, out);
            if (lane < SC_CB && c0 + lane < n_comp) {
                float v = out[0];
#pragma unroll
                for (int cb = 1; cb < SC_CB; ++cb) v = lane == cb ? out[cb] : v;
                sc[c0 + lane] = v;
                srow[c0 + lane] = v;
            }
        }
    } else {
        for (int c = tid; c < n_comp; c += TK_THREADS) sc[c] = srow[c];
    }
    __syncthreads();
    auto key_at = [&](int i) { return v4_total_key(sc[i]); };
    uint32_t pivot, need;
    tk_radix_select(key_at, n_comp, (uint32_t)K, sh.tk, pivot, need);
    tk_compact(key_at, n_comp, (uint32_t)K, pivot, need, sh.tk, picked);
    __syncthreads();
    for (int j = tid; j < K; j += TK_THREADS) row[W + j] = W + (int32_t)picked[j];
}

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

// Optional per-tile timeline of CTA 0, thread 0 for tuning builds (-DRIVOLI_DEBUG_TIMES); compiled out otherwise.
#ifdef RIVOLI_DEBUG_TIMES
__device__ long long g_v4_times[32 * 8];
#define V4_STAMP(tile, slot) do { if (blockIdx.x == 0 && threadIdx.x == 0 && (tile) < 32) g_v4_times[(tile) * 8 + (slot)] = clock64(); } while (0)
#else
#define V4_STAMP(tile, slot) do { } while (0)
#endif

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
    V4_STAMP(30, 0);
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

    // q of this sequence (not produced by the kernel before this one), then that kernel's selection row, then
    // the first tile
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int ch = tid + it * SA_THREADS, row = ch >> 6, c = ch & 63;
        v4_cp_async16(sbase + SA_SQ + swz(row, c), q + ((size_t)b * SA_H + row) * SA_D + c * 8);
    }
    rv_grid_dep_wait();
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
        V4_STAMP(t, 0);
        if (t + 1 < n_tiles) {
#pragma unroll
            for (int it = 0; it < 8; ++it) gather_piece(t + 1, buf ^ 1, it);
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        V4_STAMP(t, 1);
        __syncthreads();
        V4_STAMP(t, 2);
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
        V4_STAMP(t, 3);
        __syncthreads();
        V4_STAMP(t, 4);

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
        V4_STAMP(t, 5);

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
        V4_STAMP(t, 6);
        __syncthreads();
        V4_STAMP(t, 7);
    }

    V4_STAMP(30, 1);
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
    V4_STAMP(30, 2);
}

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
                                                             int cache_row0, float* __restrict__ prequant) {
    extern __shared__ __align__(16) float cp_row[];   // [d]
    __shared__ float red[CP_THREADS / 32];
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
    __syncthreads();
    uint16_t* out = cache + ((size_t)b * cache_rows + cache_row0 + sp / p.ratio) * d;
    for (int e = tid; e < d; e += CP_THREADS) out[e] = rv_f32_to_bf16(cp_row[e]);
}

static int cp_guard(const CompGeom& p) {
    if (p.ratio <= 1 || p.d <= 0 || p.rd <= 0 || p.coff < 1 || p.coff > 2) return 1001;
    if (p.rd > p.d || (p.rd & 1)) return 1002;
    if (p.cd != p.coff * p.d || p.ents != p.coff * p.ratio) return 1003;
    if (p.ents > CP_ENTS_MAX) return 1004;
    if ((p.coff == 2) != (p.ratio == 4)) return 1010;
    return 0;
}

static int v4_check_geom(const V4Geom* g, int n_seqs) {
    if (!g || n_seqs <= 0) return 1001;
    if (g->n_heads <= 0 || g->head_dim <= 0 || g->window <= 0 || g->index_heads <= 0 || g->index_dim <= 0 ||
        g->index_topk <= 0 || g->ratio <= 1 || g->max_comp <= 0)
        return 1001;
    return 0;
}

}  // namespace

#ifdef RIVOLI_DEBUG_TIMES
RIVOLI_API int rivoli_v4_debug_times(long long* host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, g_v4_times, sizeof(long long) * 32 * 8);
}
#endif

RIVOLI_API int rivoli_act_quant_f4_rotated(float* x, int rows, int d, void* stream) {
    if (rows <= 0 || d <= 0) return 1001;
    if (d > V4_ROT_MAX) return 1002;
    if (d & (d - 1)) return 1003;
    if (d % 32) return 1004;
    rv_drain_error();
    v4_spread_kernel<<<(unsigned)rows, 128, 0, (cudaStream_t)stream>>>(x, d);
    return rv_launch_status();
}

RIVOLI_API int rivoli_index_score_blocks(const float* q, const float* kv, const float* w, float* score, int s,
                                         int n_comp, int heads, int hd, void* stream) {
    if (s <= 0 || heads <= 0 || hd <= 0) return 1001;
    if (n_comp <= 0) return 1005;   // an empty compressed region has no score row to write
    rv_drain_error();
    cudaStream_t st = (cudaStream_t)stream;
    if (heads <= SC_MAX_HEADS && hd <= SC_MAX_HD && hd % 4 == 0 && s <= 65535) {
        const size_t smem = ((size_t)hd * SC_MAX_HEADS + SC_MAX_HEADS + (size_t)(SCK_THREADS / 32) * SC_CB * hd) * sizeof(float);
        cudaFuncSetAttribute(v4_score_blocks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        dim3 grid((unsigned)((n_comp + SCK_BLOCKS_PER_CTA - 1) / SCK_BLOCKS_PER_CTA), (unsigned)s);
        v4_score_blocks_kernel<<<grid, SCK_THREADS, smem, st>>>(q, kv, w, score, n_comp, heads, hd);
    } else {
        const size_t total = (size_t)s * (size_t)n_comp;
        v4_score_blocks_serial_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(q, kv, w, score, s, n_comp, heads, hd);
    }
    return rv_launch_status();
}

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
                                            void* stream) {
    if (!pp) return 1000;
    const CompGeom p = *pp;
    if (int g = cp_guard(p)) return g;
    if (n_seqs <= 0 || cache_rows <= 0 || cache_row0 < 0) return 1001;
    if (rotate && (p.d > V4_ROT_MAX || (p.d & (p.d - 1)) || p.d % 32)) return 1002;
    if (!rotate && (p.d - p.rd) % 64) return 1004;
    if ((size_t)p.d * 4 > 48 * 1024) return 1002;
    rv_drain_error();
    cp_step_kernel<<<(unsigned)n_seqs, CP_THREADS, (size_t)p.d * 4, (cudaStream_t)stream>>>(
        p, pos, kv_proj, score_proj, ape, kv_state, score_state, norm, freqs, rotate, cache, cache_rows, cache_row0, prequant);
    return rv_launch_status();
}

RIVOLI_API size_t rivoli_v4_select_scratch_bytes(const V4Geom* g, int n_seqs) {
    if (!g || n_seqs <= 0 || g->max_comp <= 0) return 0;
    return ((size_t)n_seqs * (size_t)g->max_comp + (size_t)n_seqs) * 4;   // score rows, then one flag per sequence
}

RIVOLI_API int rivoli_v4_index_pack_bf16(const V4Geom* g, int n_seqs, const int32_t* row_begin, const int32_t* row_end,
                                         int max_rows, const uint16_t* index_kv, unsigned char* packed,
                                         uint32_t* packed_exp, void* stream) {
    if (int rc = v4_check_geom(g, n_seqs)) return rc;
    if (!row_end || !packed || !packed_exp || max_rows <= 0) return 1001;
    if (g->index_dim != 128 || n_seqs > 65535) return 1002;
    rv_drain_error();
    dim3 grid((unsigned)((max_rows * 4 + 255) / 256), (unsigned)n_seqs);
    v4_index_pack_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(*g, row_begin, row_end, index_kv, packed, packed_exp);
    return rv_launch_status();
}

RIVOLI_API int rivoli_v4_select_blocks_bf16(const V4Geom* g, int n_seqs, const int32_t* pos, const uint16_t* index_q,
                                            const float* index_w, const uint16_t* index_kv, const unsigned char* packed,
                                            const uint32_t* packed_exp, int32_t* sel, void* scratch, int force_fold,
                                            void* stream) {
    if (int rc = v4_check_geom(g, n_seqs)) return rc;
    if (!scratch || ((packed != nullptr) != (packed_exp != nullptr))) return 1001;
    if (g->index_heads > SC_MAX_HEADS || g->index_dim > SC_MAX_HD || g->max_comp > SEL_MAX_COMP || g->index_topk > 4096)
        return 1002;
    if (g->index_dim % 32) return 1004;
    const size_t smem = ((sizeof(SelSmem) + 15) & ~(size_t)15) +
                        ((size_t)g->index_dim * SC_MAX_HEADS + (size_t)TK_WARPS * SC_CB * g->index_dim + (size_t)g->max_comp +
                         (size_t)g->index_topk) * 4;
    if (smem > 227 * 1024) return 1002;
    rv_drain_error();
    cudaStream_t st = (cudaStream_t)stream;
    float* scores = static_cast<float*>(scratch);
    int32_t* flags = reinterpret_cast<int32_t*>(scores + (size_t)n_seqs * g->max_comp);
    const bool tensor = !force_fold && g->index_dim == 128 && n_seqs <= 65535;
    if (tensor) {
        cudaMemsetAsync(flags, 0, (size_t)n_seqs * 4, st);
        dim3 grid((unsigned)((g->max_comp + SI_CHUNK - 1) / SI_CHUNK), (unsigned)n_seqs);
        if (packed)
            v4_score_int8_kernel<true><<<grid, SI_THREADS, 0, st>>>(*g, pos, index_q, index_w, index_kv, packed, packed_exp,
                                                                    scores, flags);
        else
            v4_score_int8_kernel<false><<<grid, SI_THREADS, 0, st>>>(*g, pos, index_q, index_w, index_kv, packed, packed_exp,
                                                                     scores, flags);
    }
    cudaFuncSetAttribute(v4_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rv_launch_dependent(v4_select_kernel, dim3((unsigned)n_seqs), dim3(TK_THREADS), smem, st, *g, pos, index_q, index_w,
                        index_kv, sel, scores, (const int32_t*)flags, tensor ? 0 : 1);
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
