// V4 cousin of the decode path, part 1: Hadamard + fp4 spread, block scorer, scored block selection.
//
// Reference behaviour: crates/backend/kernels/blockindex.hip:97-138,234-306 (spread, block scorer),
// crates/engine/src/v4/select.rs:153-232 (selection rows). The spread, the scores and the selected indices are
// bit-exact against the host rules: every add and multiply on those paths is an explicit round-to-nearest
// intrinsic, so nothing is contracted into a fused multiply-add, and every fold runs in the host's order.
//
// Storage on this side is bf16 (the reference keeps bf16 VALUES in f32 arrays: every producer on the
// path ends in a bf16 store), which halves the bytes and feeds the tensor cores directly.
#include "topk_core.cuh"
#include "v4_common.cuh"

namespace {

// ---------------------------------------------------------------------------------------------------
// spread
// ---------------------------------------------------------------------------------------------------
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

// Scores of blocks [c0, c0 + SC_CB) for one query row, by one warp. Lane l owns heads l and l + 32: each
// dot is an ascending fold over the hd terms (separate multiply and add), exactly the host's; the head
// sum is then an ascending f32 fold over the bf16 terms, evaluated redundantly by every lane.
// qT: shared [hd][64] f32 (transposed: lanes read consecutive words); wsh: shared [64] f32;
// stage: this warp's shared [SC_CB][hd] f32. Returns through out[SC_CB] (same value in every lane).
template <class T>
__device__ __forceinline__ void v4_score_blocks_warp(const float* __restrict__ qT, const float* __restrict__ wsh,
                                                     float* __restrict__ stage, const T* __restrict__ kv, int c0,
                                                     int n_comp, int heads, int hd, float (&out)[SC_CB],
                                                     const uint32_t* cols = nullptr) {
    const int lane = threadIdx.x & 31;
    __syncwarp();
    for (int i = lane; i < SC_CB * hd; i += 32) {
        const int cb = i / hd, e = i - cb * hd;
        // blocks c0 .. c0 + SC_CB - 1, or the listed ones (cols[c0 + cb], c0 + cb < n_comp = the list's length)
        const bool live = c0 + cb < n_comp;
        const size_t c = live ? (cols ? cols[c0 + cb] : (uint32_t)(c0 + cb)) : 0;
        stage[i] = live ? v4_load_f32(kv, c * hd + e) : 0.0f;
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
// two, and the block scales of one row lie within a few binades of each other (that is what the Hadamard
// rotation is for). Take as a ROW's unit u = 2^(pmin - 130), pmin the smallest biased exponent any
// non-empty block's largest magnitude has: every value of the row is an integer multiple of u, below
// 16 * 2^span in magnitude (span = pmax - pmin). With span <= 3 on both sides the integers fit int8 and
// the whole 128-term dot product is ONE integer,
//     q_h . kv_c = I * u_q * u_k,   I = sum of 128 integer products,  |I| < 2^21,
// which four chained mma.m16n8k32.s8 return exactly. The host's ascending f32 fold over the 128 products
// never rounds here: every partial sum is a multiple of u_q u_k below 2^21 u_q u_k, inside f32's 24 bits,
// so it ends on the same value, float(I) * u_q * u_k. Everything after the dot (bf16 store, relu, head
// weight, bf16 store, ascending head sum) runs in the host's order on CUDA cores.
// A CACHED row that is not of that form (a value that is not a multiple of the unit, block scales more
// than 3 binades apart, a subnormal, magnitudes outside 2^-40 .. 2^40) gets a marker instead of a score
// and the selection kernel re-scores that column with the ordered CUDA-core fold; a QUERY row outside the
// form raises the sequence's flag and the whole sequence takes the ordered fold. Exact either way.
// ---------------------------------------------------------------------------------------------------
constexpr int SI_THREADS = 256;
constexpr int SI_CHUNK = 256;       // blocks (columns) per CTA
constexpr int SI_SPAN = 3;          // binades between the block scales of one row
constexpr int SI_NT = 2;            // column tiles of 8 a warp scores per iteration
constexpr int SI_PMIN = 87, SI_PMAX = 167;     // biased exponents 2^-40 .. 2^40
constexpr uint32_t SI_REFOLD = 0xffc0deadu;   // score word of a column left to the ordered fold (a NaN no fold produces)

__device__ __forceinline__ void v4_mma_s8(int (&d)[4], const uint4& a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float v4_rbf16_hw(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }  // finite inputs

// Largest biased exponent among the bf16 values packed in w0, w1.
__device__ __forceinline__ int v4_max_exp4(uint32_t w0, uint32_t w1) {
    const uint32_t a = max(w0 & 0x7f800000u, w1 & 0x7f800000u), b = max((w0 << 16) & 0x7f800000u, (w1 << 16) & 0x7f800000u);
    return (int)(max(a, b) >> 23);
}
// Four bf16 values (two words) times `scale` (a power of two) -> four int8. ok is cleared when a product is
// not an integer (the value is not a multiple of the row's unit).
__device__ __forceinline__ uint32_t v4_pack4(uint32_t w0, uint32_t w1, float scale, bool& ok) {
    const float x0 = __uint_as_float(w0 << 16) * scale, x1 = __uint_as_float(w0 & 0xffff0000u) * scale;
    const float x2 = __uint_as_float(w1 << 16) * scale, x3 = __uint_as_float(w1 & 0xffff0000u) * scale;
    const int m0 = __float2int_rn(x0), m1 = __float2int_rn(x1), m2 = __float2int_rn(x2), m3 = __float2int_rn(x3);
    ok = ok && (float)m0 == x0 && (float)m1 == x1 && (float)m2 == x2 && (float)m3 == x3;
    if (scale == 0.0f) ok = ok && ((w0 | w1) & 0x7fff7fffu) == 0;   // an "empty" row must really be zeros
    // cvt.pack d, a, b, c: d[7:0] = sat(b), d[15:8] = sat(a), d[31:16] = c[15:0]
    uint32_t hi, out;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(m3), "r"(m2), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(m1), "r"(m0), "r"(hi));
    return out;
}
// Row unit from the smallest / largest block exponent of a row (pmin > pmax when every block is empty):
// inv = 2^(130 - pmin) turns the row into integers, unit = 2^(pmin - 130) turns them back; both 0 for an empty
// row. Rows outside the limits clear ok.
__device__ __forceinline__ void v4_row_unit(int pmin, int pmax, float& inv, float& unit, bool& ok) {
    inv = 0.0f;
    unit = 0.0f;
    if (pmax < pmin) return;
    if (pmin < SI_PMIN || pmax > SI_PMAX || pmax - pmin > SI_SPAN) { ok = false; return; }
    inv = __int_as_float((257 - pmin) << 23);
    unit = __int_as_float((pmin - 3) << 23);
}

// PACKED: the rows come as int8 + row exponent (rivoli_v4_index_pack_bf16), written once when a row enters
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
    __shared__ float qunit[64];                                // per head: its row unit (0 = empty row)
    __shared__ float wsh[64];
    // written as float2 (needs the alignment); rows padded by two words so the eight heads of a store spread over banks
    __shared__ __align__(16) float terms[SI_THREADS / 32][64][8 * SI_NT + 2];
    const int b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_comp = min((pos[b] + 1) / g.ratio, g.max_comp);
    const int c_begin = blockIdx.x * SI_CHUNK;
    if (n_comp <= g.index_topk || c_begin >= n_comp) return;   // positional sequences are not scored
    const int heads = g.index_heads;
    bool ok = true;
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
        // exponent range of the head's non-empty blocks (its four threads are neighbours)
        int lo = pb > 0 ? pb : 1000, hi = pb > 0 ? pb : -1000;
        lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, 1)); hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, 1));
        lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, 2)); hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, 2));
        float inv, unit;
        v4_row_unit(lo, hi, inv, unit, ok);
        const int mt = hh >> 4, r = hh & 15;
#pragma unroll
        for (int k4 = 0; k4 < 8; ++k4) {                       // values 4 k4 .. 4 k4 + 3 of the block
            const uint32_t packed4 = v4_pack4(wv[2 * k4], wv[2 * k4 + 1], inv, ok);
            const int kk = 4 * k4, fl = (r & 7) * 4 + ((kk & 15) >> 2), reg = (r >> 3) + 2 * (kk >> 4);
            qfrag[((mt * 4 + j) * 32 + fl) * 4 + reg] = packed4;
        }
        if (j == 0) qunit[hh] = unit;
        if (tid < 64) wsh[tid] = tid < heads ? index_w[(size_t)b * heads + tid] : 0.0f;
    }
    __syncthreads();
    const uint16_t* kv = index_kv + (size_t)b * g.max_comp * 128;
    const int grp = lane >> 2, quad = lane & 3;
    const int c_end = min(n_comp, c_begin + SI_CHUNK);
    // units and weights of the eight heads this thread's accumulators belong to
    float qu[8], qw[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int hh = 16 * (i >> 1) + grp + 8 * (i & 1);
        qu[i] = qunit[hh];
        qw[i] = wsh[hh];
    }
    // SI_NT column tiles of 8 per iteration: every A fragment read from shared memory serves SI_NT MMAs
    for (int c0 = c_begin + warp * (8 * SI_NT); c0 < c_end; c0 += (SI_THREADS / 32) * (8 * SI_NT)) {
        uint32_t b0[SI_NT][4], b1[SI_NT][4];
        float kuA[SI_NT], kuB[SI_NT];
        uint32_t bad_rows[SI_NT];
#pragma unroll
        for (int t = 0; t < SI_NT; ++t) {
            // ---- B fragments: row c0 + 8 t + grp, this thread's 8 values of each block
            const int c = c0 + 8 * t + grp;
            float ku = 0.0f;
            bool okk = true;                                    // this row (column of the score matrix)
            if (PACKED) {
                const uint8_t* prow = packed + ((size_t)b * g.max_comp + c) * 128;
                const uint32_t e = c < n_comp ? packed_exp[(size_t)b * g.max_comp + c] : 0u;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    b0[t][j] = b1[t][j] = 0u;
                    if (c < n_comp) {
                        b0[t][j] = *reinterpret_cast<const uint32_t*>(prow + j * 32 + quad * 4);
                        b1[t][j] = *reinterpret_cast<const uint32_t*>(prow + j * 32 + 16 + quad * 4);
                    }
                }
                if (e == 0xffu) okk = false;                    // the packer could not take this row
                else if (e != 0u) ku = __int_as_float(((int)e - 3) << 23);
            } else {
                uint2 lo[4], hi[4];
                int k_lo = 1000, k_hi = -1000;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    lo[j] = hi[j] = make_uint2(0, 0);
                    if (c < n_comp) {
                        lo[j] = *reinterpret_cast<const uint2*>(kv + (size_t)c * 128 + j * 32 + quad * 4);
                        hi[j] = *reinterpret_cast<const uint2*>(kv + (size_t)c * 128 + j * 32 + 16 + quad * 4);
                    }
                    // the block's largest exponent over the quad that holds the row, then the row's extremes
                    int pb = max(v4_max_exp4(lo[j].x, lo[j].y), v4_max_exp4(hi[j].x, hi[j].y));
                    pb = max(pb, __shfl_xor_sync(0xffffffffu, pb, 1));
                    pb = max(pb, __shfl_xor_sync(0xffffffffu, pb, 2));
                    if (pb > 0) { k_lo = min(k_lo, pb); k_hi = max(k_hi, pb); }
                }
                float inv;
                v4_row_unit(k_lo, k_hi, inv, ku, okk);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    b0[t][j] = v4_pack4(lo[j].x, lo[j].y, inv, okk);
                    b1[t][j] = v4_pack4(hi[j].x, hi[j].y, inv, okk);
                }
            }
            // a row's verdict sits in the four lanes of its quad
            bad_rows[t] = __ballot_sync(0xffffffffu, !okk);
            // units of the two columns this thread's accumulators belong to
            kuA[t] = __shfl_sync(0xffffffffu, ku, (quad * 2) * 4);
            kuB[t] = __shfl_sync(0xffffffffu, ku, (quad * 2 + 1) * 4);
        }
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
            int acc[SI_NT][4];
#pragma unroll
            for (int t = 0; t < SI_NT; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 a = *reinterpret_cast<const uint4*>(&qfrag[((mt * 4 + j) * 32 + lane) * 4]);
#pragma unroll
                for (int t = 0; t < SI_NT; ++t) v4_mma_s8(acc[t], a, b0[t][j], b1[t][j]);
            }
#pragma unroll
            for (int rh = 0; rh < 2; ++rh) {                   // row half of the accumulator
                const int hh = 16 * mt + grp + 8 * rh;
                const float u = qu[2 * mt + rh], wv = qw[2 * mt + rh];
#pragma unroll
                for (int t = 0; t < SI_NT; ++t) {
                    const float dA = (float)acc[t][2 * rh] * (u * kuA[t]), dB = (float)acc[t][2 * rh + 1] * (u * kuB[t]);
                    // bf16 store, relu, times the (signed) head weight, bf16 store
                    const float tA = v4_rbf16_hw(__fmul_rn(fmaxf(v4_rbf16_hw(dA), 0.0f), wv));
                    const float tB = v4_rbf16_hw(__fmul_rn(fmaxf(v4_rbf16_hw(dB), 0.0f), wv));
                    *reinterpret_cast<float2*>(&terms[warp][hh][8 * t + quad * 2]) = make_float2(tA, tB);
                }
            }
        }
        __syncwarp();
        if (lane < 8 * SI_NT && c0 + lane < c_end) {           // lane j carries column j's ordered head sum
            float acc = 0.0f;
#pragma unroll 8
            for (int hh = 0; hh < heads; ++hh) acc = __fadd_rn(acc, terms[warp][hh][lane]);
            const bool refold = ((bad_rows[lane >> 3] >> (4 * (lane & 7))) & 0xfu) != 0;
            scores[(size_t)b * g.max_comp + c0 + lane] = refold ? __uint_as_float(SI_REFOLD) : v4_rbf16_hw(acc);
        }
        __syncwarp();
    }
    if (!ok) atomicOr(&flags[b], 1);
}

// One thread per (row, block of 32): the row's values as int8 multiples of its unit 2^(pmin - 130); the row's word
// holds pmin (0 = the row is all zeros, 0xff = not of the integer form: the scorer then leaves the column to the
// ordered fold, which reads the bf16 row).
__global__ void v4_index_pack_kernel(V4Geom g, const int32_t* __restrict__ row_begin, const int32_t* __restrict__ row_end,
                                     const uint16_t* __restrict__ index_kv, uint8_t* __restrict__ packed,
                                     uint32_t* __restrict__ packed_exp) {
    const int b = blockIdx.y;
    const int r0 = row_begin ? row_begin[b] : 0, r1 = min(row_end[b], g.max_comp);
    const int id = blockIdx.x * blockDim.x + threadIdx.x, row = r0 + (id >> 2), j = id & 3;
    const bool live = row < r1;
    const size_t off = ((size_t)b * g.max_comp + (live ? row : 0)) * 128 + j * 32;
    uint32_t wv[16];
    int pb = 0;
    if (live) {
        const uint4* src = reinterpret_cast<const uint4*>(index_kv + off);
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
    // the four blocks of a row sit in four neighbouring threads
    int lo = pb > 0 ? pb : 1000, hi = pb > 0 ? pb : -1000;
    lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, 1)); hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, 1));
    lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, 2)); hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, 2));
    bool ok = true;
    float inv, unit;
    v4_row_unit(lo, hi, inv, unit, ok);
    uint32_t out[8];
#pragma unroll
    for (int k4 = 0; k4 < 8; ++k4) out[k4] = v4_pack4(wv[2 * k4], wv[2 * k4 + 1], inv, ok);
    uint32_t bad = ok ? 0u : 1u;
    bad |= __shfl_xor_sync(0xffffffffu, bad, 1);
    bad |= __shfl_xor_sync(0xffffffffu, bad, 2);
    if (live) {
        uint4* dst = reinterpret_cast<uint4*>(packed + off);
        dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
        dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
        if (j == 0) packed_exp[(size_t)b * g.max_comp + row] = bad ? 0xffu : (hi >= lo ? (uint32_t)lo : 0u);
    }
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
    uint32_t n_bad;      // columns the integer scorer left to the ordered fold
};

__global__ void __launch_bounds__(TK_THREADS) v4_select_kernel(V4Geom g, const int32_t* __restrict__ pos,
                                                               const uint16_t* __restrict__ index_q,
                                                               const float* __restrict__ index_w,
                                                               const uint16_t* __restrict__ index_kv,
                                                               int32_t* __restrict__ sel,
                                                               float* __restrict__ scores,
                                                               int32_t* __restrict__ flags, int force_fold) {
    extern __shared__ __align__(16) unsigned char sel_smem_raw[];
    SelSmem& sh = *reinterpret_cast<SelSmem*>(sel_smem_raw);
    float* qT = reinterpret_cast<float*>(sel_smem_raw + ((sizeof(SelSmem) + 15) & ~(size_t)15));
    float* stage = qT + g.index_dim * SC_MAX_HEADS;
    float* sc = stage + TK_WARPS * SC_CB * g.index_dim;
    uint32_t* picked = reinterpret_cast<uint32_t*>(sc + g.max_comp);

    const int b = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    rv_grid_dep_trigger();   // the attention kernel may be scheduled; it waits for this grid before it reads anything
    // Every CTA waits for the scorer first, including those that return early below: the kernel launched after
    // this one relies on "this grid is complete" implying "everything before it is complete", and `sel` may
    // still be read by a kernel of the previous step that the scorer's own wait orders.
    rv_grid_dep_wait();
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
    float* srow = scores + (size_t)b * g.max_comp;   // the scorer's rows and flags (ordered by the wait above)
    const uint16_t* kv = index_kv + (size_t)b * g.max_comp * g.index_dim;
    // the ordered CUDA-core fold over every block: on request, or when the integer scorer could not take the queries
    auto fold_all = [&]() {
        v4_stage_q(index_q + (size_t)b * g.index_heads * g.index_dim, index_w + (size_t)b * g.index_heads, g.index_heads,
                   g.index_dim, qT, sh.wsh);
        __syncthreads();
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
    };
    if (force_fold || (flags[b] & 1)) {
        fold_all();
    } else {
        // take the scorer's row; columns it marked are re-scored by the ordered fold, a few per warp
        if (tid == 0) sh.n_bad = 0u;
        __syncthreads();
        for (int c = tid; c < n_comp; c += TK_THREADS) {
            const float v = srow[c];
            sc[c] = v;
            if (__float_as_uint(v) == SI_REFOLD) {
                const uint32_t i = atomicAdd(&sh.n_bad, 1u);
                if (i < (uint32_t)K) picked[i] = (uint32_t)c;
            }
        }
        __syncthreads();
        const int n_bad = (int)sh.n_bad;
        if (n_bad > K) {                 // more than the list holds: everything again
            __syncthreads();
            fold_all();
        } else if (n_bad > 0) {
            v4_stage_q(index_q + (size_t)b * g.index_heads * g.index_dim, index_w + (size_t)b * g.index_heads,
                       g.index_heads, g.index_dim, qT, sh.wsh);
            __syncthreads();
            for (int i0 = warp * SC_CB; i0 < n_bad; i0 += TK_WARPS * SC_CB) {
                float out[SC_CB];
                v4_score_blocks_warp(qT, sh.wsh, stage + warp * SC_CB * g.index_dim, kv, i0, n_bad, g.index_heads,
                                     g.index_dim, out, picked);
                if (lane < SC_CB && i0 + lane < n_bad) {
                    float v = out[0];
#pragma unroll
                    for (int cb = 1; cb < SC_CB; ++cb) v = lane == cb ? out[cb] : v;
                    sc[picked[i0 + lane]] = v;
                    srow[picked[i0 + lane]] = v;
                }
            }
        }
        if (n_bad > 0 && tid == 0) atomicOr(&flags[b], 2);
    }
    __syncthreads();
    auto key_at = [&](int i) { return v4_total_key(sc[i]); };
    uint32_t pivot, need;
    tk_radix_select(key_at, n_comp, (uint32_t)K, sh.tk, pivot, need);
    tk_compact(key_at, n_comp, (uint32_t)K, pivot, need, sh.tk, picked);
    __syncthreads();
    for (int j = tid; j < K; j += TK_THREADS) row[W + j] = W + (int32_t)picked[j];
}

}  // namespace

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
                        index_kv, sel, scores, flags, tensor ? 0 : 1);
    return rv_launch_status();
}
