// Absorbed MLA decode attention on the 5th-generation tensor cores, all operands fp8.
//
//     out_h = sum_t softmax_t((q_h . [L_t | R_t]) * scale) * L_t        (H = 64, 512 + 64 dims)
//
// The cache rows are e4m3 codes with one f32 scale per token, and tcgen05 kind::f8f6f4
// takes e4m3 operands directly, so the gathered rows are consumed AS THEY LIE in HBM: no
// dequantisation pass and half the shared memory of a 16-bit staging. The two operands that
// are not fp8 by nature are split into two e4m3 terms each (x ~ hi + lo, relative error
// ~2^-8, bf16-like):
//   * q (bf16 in)  -> q_hi and q_lo as 128 "virtual heads" along M, per-head scales;
//   * P (softmax)  -> p_hi, p_lo issued as two MMAs accumulating into the same columns.
// The per-token scale folds into the softmax: with s2 = log2(e) * scale * (q.k) and
// s2' = s2 + log2(s_tok), P' = 2^(s2' - m) = weight * s_tok, so P' x (raw V codes) is already
// the dequantised product and P' is bounded by 2^8 whatever the scales are.
//
// What bounds this kernel is how many gathered rows an SM keeps in flight, so the tile is SMALL and the ring is
// DEEP: 64 tokens per tile, SIX tiles (6 x 36 KiB) in flight. The room comes from keeping q out of shared memory: its
// 512 latent columns live in TENSOR MEMORY as the A operand of the QK MMAs (128 lanes = hi|lo heads, 128 columns of
// four e4m3 codes), which also spares the shared-memory pipe 64 KiB of operand reads per tile; only the 64 rope
// columns of q stay in shared memory. Tokens are the MMA N dimension, which may be 64 while every instruction keeps
// the full M = 128:
//   S[128 (hi|lo heads) x 64 tok] = Qcat . K_tile^T                         2 (rope, A in smem) + 16 (A in TMEM) MMAs, K = 32
//   O^T[512 dims x 64 heads]     += V^T (the SAME shared tile, read MN-major) . P'
//                                   4 blocks x 2 K-steps x {hi, lo} = 16 MMAs (N = 64)
// TMEM (512 columns): S double buffered (2 x 64) + q (128) + O^T (4 x 64).
//
// One CTA per (sequence, split), 14 warps: 0-7 softmax + epilogue, 8 QK issue, 9 PV issue, 10-13 gather (warp g
// fills the tiles g, g + 4, ... in plain program order and does not wait for its copies: the copies signal the
// stage's barrier themselves, so a warp goes straight on to its next tile as soon as that tile's stage is free; a lane
// locates two rows, copies go row by row with 32 lanes on 32 consecutive 16-byte chunks (cp.async into the swizzled
// tile); the row address chain (token -> page -> pool row -> scale) is software-pipelined in register queues).
// A softmax thread is one TMEM lane = one virtual head, and the q rows are ordered so that the hi and lo terms of a
// head sit 16 lanes apart in the SAME warp: lanes 0-15 of warp s hold the hi rows of heads 16 s .. 16 s + 15, lanes
// 16-31 their lo rows. One shuffle per score adds the two terms and leaves each lane with HALF the tokens of its
// head: thread = (head, 16 tokens of the tile), two warps per lane quarter take the two 32-token halves. A head's
// reference maximum, its running sum and its q scale are registers, and P' leaves as one 16-byte store per term
// (heads are the rows of the K-major P' operand, tokens its bytes).
// q arrives as bf16 and is split into its two e4m3 terms by the softmax warps inside the kernel while the
// first tiles are gathered (a thread converts the row of its own TMEM lane and stores it with tcgen05.st); the output
// leaves straight from the accumulator registers (64 contiguous bytes per warp store).
// Online softmax with a LAGGING reference max: as long as no score of a tile exceeds its head's
// reference by more than 3 (log2) the references stand (one barrier-with-OR per tile, no exchange);
// otherwise the exact per-head maxima are taken and O is rescaled through TMEM. P' carries 2^5, so
// it stays <= 256 < 448 and typical weights keep both e4m3 terms in the normal range.
// A batch too small to fill the chip is split: the CTAs of a sequence form one thread-block cluster (up to 8), each takes
// a contiguous range of tiles, and they merge their (maximum, sum, O) through distributed shared memory inside the kernel.
// All waits are bounded (tc_common.cuh).
#include <cooperative_groups.h>

#include "codec.cuh"
#include "common.cuh"
#include "tc_common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int AM_TILE = 64;
constexpr int AM_STAGES = 6;             // K ring depth
constexpr int AM_ROPES = 3;              // rope tiles: released right after the two rope MMAs of a tile, so fewer than stages
constexpr int AM_SBUF = 2;               // S accumulators
constexpr int AM_GW = 4;                 // gather warps
constexpr int AM_H = 64, AM_KVL = 512, AM_ROPE = 64, AM_W = AM_KVL + AM_ROPE;
constexpr int AM_SW = 8;                 // softmax + epilogue warps: TMEM lane quarter = warp % 4, token / head half = warp / 4
constexpr int AM_HPT = 32;               // head columns of O^T a thread owns in the rescale and the epilogue
constexpr int AM_SOFTMAX_THREADS = AM_SW * 32;
constexpr int AM_QKW = AM_SW, AM_PVW = AM_SW + 1, AM_GW0 = AM_SW + 2;   // warp roles: QK issue, PV issue, first gather warp
constexpr int AM_THREADS = (AM_GW0 + AM_GW) * 32;
constexpr int AM_MAX_SPLITS = 8;     // CTAs per sequence = thread-block cluster size
// P'' = 2^(s2' - m_ref + AM_POFF) with m_ref lagging the true maximum by at most AM_LAG, so
// P'' <= 2^(AM_POFF + AM_LAG) = 256 < 448 while typical weights (a few binades below the maximum)
// land where BOTH e4m3 terms are normal numbers. In the code s2 carries the offset (s2 = s2' + AM_POFF)
// and the reference is kept WITHOUT it (m_ref = max s2'), so that the difference s2 - m_ref is the
// exponent of P'' directly.
constexpr float AM_POFF = 5.0f, AM_LAG = 3.0f;

// tensor memory map (columns)
constexpr int TMC_S = 0, TMC_Q = AM_SBUF * AM_TILE, TMC_O = TMC_Q + AM_KVL / 4;
static_assert(TMC_O + 4 * AM_H == 512, "tensor memory budget");

// shared memory map (bytes); every operand tile is 1024-byte aligned
constexpr int SM_K0 = 0;                 // 6 stages x (4 latent chunks x [64 rows][128 B]), 128-byte swizzle
constexpr int SM_KSTAGE = 32768, SM_KCHUNK = 8192;
constexpr int SM_ROPE = SM_K0 + AM_STAGES * SM_KSTAGE;       // 3 x [64 rows][64 B], 64-byte swizzle
constexpr int SM_ROPEBUF = 4096;
constexpr int SM_QR = SM_ROPE + AM_ROPES * SM_ROPEBUF;       // rope columns of q: [128 virtual heads][64 B], 64-byte swizzle
constexpr int SM_P = SM_QR + 8192;       // hi [64 heads][64 tokens], lo the same: K-major, 64-byte swizzle
constexpr int SM_PTERM = 4096;
constexpr int SM_TOK = SM_P + 2 * SM_PTERM;   // f32 [3][6 stages][64 tokens]: scale | log2(scale) + AM_POFF | 1 / scale
constexpr int SM_TOKPLANE = AM_STAGES * AM_TILE * 4;
constexpr int SM_AHI = SM_TOK + 3 * SM_TOKPLANE;   // f32 [64] per-head q scale * softmax scale * log2(e)
constexpr int SM_WMAX = SM_AHI + 256;    // f32 [2][64] exchange between the two token halves
constexpr int SM_FAC = SM_WMAX + 512;    // f32 [64] rescale factor of the current tile; 1 / l in the epilogue
constexpr int SM_BARS = SM_FAC + 256;    // mbarriers
constexpr int SM_MISC = SM_BARS + 256;
constexpr int SM_XS = SM_MISC + 64;      // f32 [2][64]: this CTA's reference maximum and weight sum per head, read by its cluster
constexpr int SM_TOTAL = SM_XS + 512;
constexpr int SM_STAGE = SM_K0;          // f32 [64 heads][512 dims]: this CTA's scaled O, read by its cluster (the ring is idle by then)
static_assert(AM_H * AM_KVL * 4 <= AM_STAGES * SM_KSTAGE, "the O staging fits the ring");

struct AmBars {
    uint64_t k_full[AM_STAGES], k_empty[AM_STAGES], s_full[AM_SBUF], s_empty[AM_SBUF], rope_free[AM_ROPES],
        p_full, pv_done, q_full;
};
static_assert(sizeof(AmBars) <= 256, "barrier block");
static_assert(SM_TOTAL <= 232448, "shared memory budget");
static_assert(SM_QR % 1024 == 0 && SM_P % 1024 == 0 && SM_ROPE % 1024 == 0, "operand tiles are 1024-byte aligned");


struct AttendMmaArgs {
    const uint16_t* q;       // [B][64][576] bf16: absorbed query, latent part then rope part
    float softmax_scale;
    const uint8_t* pool; const float* pscale; const int32_t* block_table;
    const uint32_t* rows; long long row_stride; const int32_t* n_rows;
    int page_tokens, max_pages, n_pool_pages, n_splits;
    uint16_t* out; float* out_m; float* out_lse;
    int* err;
    int min_rows;      // sequences with 0 < n_rows < min_rows are served by the CUDA-core kernel of the same call
    int q_early;       // 1: q was complete before the preceding kernel was launched, so it may be read before the grid-dependency wait
    int max_polls;     // poll limit of every bounded wait
    int withhold;      // self-test: one gather warp never signals its part of the first tile (the waits on it must run out cleanly)
};

__device__ __forceinline__ uint32_t sw64_chunk(uint32_t row, uint32_t chunk) { return row * 64u + ((chunk ^ ((row >> 1) & 3u)) << 4); }

__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)layout << 61;   // 2 = 128-byte swizzle, 4 = 64-byte swizzle
    return d;
}

// Row of the stacked q operand (= TMEM lane of S) that holds term `t` (0 = hi, 1 = lo) of head h: the two terms of a
// head lie 16 lanes apart inside one warp's lane quarter.
__device__ __forceinline__ int q_row(int h, int t) { return 32 * (h >> 4) + 16 * t + (h & 15); }

// ---------------------------------------------------------------------------------------------
// main kernel
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(AM_THREADS, 1)
attend_mma_kernel(AttendMmaArgs A) {
    extern __shared__ __align__(1024) uint8_t smem[];
    AmBars& bars = *reinterpret_cast<AmBars*>(smem + SM_BARS);
    float* s_tok = reinterpret_cast<float*>(smem + SM_TOK);   // three planes of SM_TOKPLANE bytes
    float* s_ahi = reinterpret_cast<float*>(smem + SM_AHI);
    float* s_wmax = reinterpret_cast<float*>(smem + SM_WMAX);
    float* s_fac = reinterpret_cast<float*>(smem + SM_FAC);
    uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(smem + SM_MISC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM_MISC + 4);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, b = blockIdx.y;
    const int P = A.page_tokens;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < AM_STAGES; ++s) { tc::mbar_init(&bars.k_full[s], 32 + 1); tc::mbar_init(&bars.k_empty[s], 1); }
#pragma unroll
        for (int s = 0; s < AM_SBUF; ++s) { tc::mbar_init(&bars.s_full[s], 1); tc::mbar_init(&bars.s_empty[s], AM_SW); }
#pragma unroll
        for (int s = 0; s < AM_ROPES; ++s) tc::mbar_init(&bars.rope_free[s], 1);
        tc::mbar_init(&bars.p_full, AM_SOFTMAX_THREADS);
        tc::mbar_init(&bars.pv_done, 1);
        tc::mbar_init(&bars.q_full, AM_SOFTMAX_THREADS);
        tc::mbar_init_fence();
        *abort_flag = 0;
    }
    if (warp == AM_QKW) tc::tmem_alloc<512>(tmem_base_s);

    tc::fence_proxy_async();
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem = *tmem_base_s;
    const uint32_t TM_S0 = tmem + TMC_S, TM_Q = tmem + TMC_Q, TM_O = tmem + TMC_O;

    // q -> two e4m3 terms per head (once per CTA):
    //   hi = e4m3(q / s), s = absmax / 448;  lo = e4m3(q / s - hi)   =>  q ~ s * (hi + lo)
    // (the residual of a value of typical size is a normal e4m3 number; below 2^-6 it is kept to 2^-10 absolute,
    // 2^-19 of the head's largest value).
    // A thread fills the row of its OWN tensor-memory lane: lane l of warp w is the virtual head
    // (16 (w % 4) + l % 16, term l / 16), and w / 4 picks the half of the 512 latent columns (the rope columns go with
    // half 0). The two lanes of a head (16 apart) share the work: the hi lane reads the even 8-value chunks of the
    // half-row and the lo lane the odd ones, each derives BOTH terms of its chunks and hands the other lane the codes
    // that belong in that lane's row (one shuffle per word). Two passes over the chunks: the absolute maximum, then
    // the codes - 64 values of the row at a time into 16 registers and from there into 16 tensor-memory columns
    // (column c = codes 4c .. 4c + 3, lowest byte first, which is the layout the MMA expects of an 8-bit A
    // operand); the rope codes go to the shared operand tile.
    // The gather warps do not wait for this: the QK issuer does (q_full) before its first MMA.
    // Under a programmatic dependent launch the kernel before this one may still be running. Unless the
    // caller vouches that q was complete before that kernel was even launched (q_early: the fused decode
    // step), q may be that kernel's output and is read only after the dependency wait.
    if (!A.q_early) rv_grid_dep_wait();
    if (warp < AM_SW) {
        const int sq = warp & 3, half = warp >> 2, term = lane >> 4;
        const int h = 16 * sq + (lane & 15);
        const uint16_t* qrow = A.q + ((size_t)b * AM_H + h) * AM_W;
        const uint4* qn = reinterpret_cast<const uint4*>(qrow + half * 256) + term;   // this lane's chunks: qn[2 m], m = 0..15
        const uint4* qr = reinterpret_cast<const uint4*>(qrow + AM_KVL) + term;        // rope (half 0): qr[2 m], m = 0..3
        float amax = 0.0f;
        auto absmax8 = [&](const uint4 v) {
            const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
                amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(ww[i] << 16)), fabsf(__uint_as_float(ww[i] & 0xffff0000u))));
        };
        {
            uint4 v[16];
#pragma unroll
            for (int m = 0; m < 16; ++m) v[m] = qn[2 * m];
#pragma unroll
            for (int m = 0; m < 16; ++m) absmax8(v[m]);
        }
        if (half == 0) {
#pragma unroll
            for (int m = 0; m < 4; ++m) absmax8(qr[2 * m]);
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 16));
        if (lane < 16) s_wmax[half * 64 + h] = amax;
        tc::named_barrier(3, AM_SOFTMAX_THREADS);
        amax = fmaxf(s_wmax[h], s_wmax[64 + h]);
        const float sc = amax > 0.0f ? amax / 448.0f : 1.0f;
        const float inv = 1.0f / sc;
        // 8 values -> their 8 hi codes and 8 lo codes (two 32-bit words each)
        auto codes8 = [&](const uint4 v, uint32_t* hi, uint32_t* lo) {
            const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
            hi[0] = hi[1] = lo[0] = lo[1] = 0u;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float x0 = __uint_as_float(ww[i] << 16) * inv, x1 = __uint_as_float(ww[i] & 0xffff0000u) * inv;
                uint16_t ch, cl;
                asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(ch) : "f"(x1), "f"(x0));
                const float2 xh = rv_e4m3x2_to_f32x2(ch);
                asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(cl) : "f"(x1 - xh.y), "f"(x0 - xh.x));
                hi[i >> 1] |= (uint32_t)ch << (16 * (i & 1));
                lo[i >> 1] |= (uint32_t)cl << (16 * (i & 1));
            }
        };
        const uint32_t lane_addr = ((uint32_t)(sq * 32)) << 16;
#pragma unroll 1
        for (int grp = 0; grp < 4; ++grp) {       // 8 chunks of the half-row = 64 values = 16 columns per store
            uint4 v[4];
#pragma unroll
            for (int m = 0; m < 4; ++m) v[m] = qn[2 * (grp * 4 + m)];
            uint32_t r[16];
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                uint32_t hi[2], lo[2];
                codes8(v[m], hi, lo);
                // this lane's own chunk is 2 m + term of the group; the partner made the codes of chunk 2 m + (1 - term)
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    const uint32_t own = term ? lo[w] : hi[w];
                    const uint32_t got = __shfl_xor_sync(0xffffffffu, term ? hi[w] : lo[w], 16);
                    r[4 * m + w] = term ? got : own;          // even chunk: made by the hi lane
                    r[4 * m + 2 + w] = term ? own : got;      // odd chunk: made by the lo lane
                }
            }
            tc::tmem_st16(TM_Q + lane_addr + half * 64 + grp * 16, r);
        }
        if (half == 0) {
            const int row_hi = q_row(h, 0), row_lo = q_row(h, 1);
#pragma unroll
            for (int m = 0; m < 4; ++m) {          // rope chunk 2 m + term: 8 bytes of the 16-byte chunk m of both rows
                uint32_t hi[2], lo[2];
                codes8(qr[2 * m], hi, lo);
                *reinterpret_cast<uint2*>(smem + SM_QR + sw64_chunk(row_hi, m) + 8 * term) = make_uint2(hi[0], hi[1]);
                *reinterpret_cast<uint2*>(smem + SM_QR + sw64_chunk(row_lo, m) + 8 * term) = make_uint2(lo[0], lo[1]);
            }
            if (term == 0) s_ahi[h] = sc * A.softmax_scale * 1.4426950408889634f;
        }
        tc::tmem_st_wait();
        tc::fence_proxy_async();
        tc::tc_fence_before();
        tc::mbar_arrive(&bars.q_full);
        tc::named_barrier(3, AM_SOFTMAX_THREADS);   // the head scales are read by other warps than the ones that wrote them
    }

    // With q_early everything above read only inputs that predate the preceding kernel, so it overlapped
    // that kernel's tail; the selected rows and their counts are read below.
    rv_grid_dep_wait();
    int nr = A.n_rows[b];
    // a row list whose first entry is the dense marker stands for "row j = token j" over the first n_rows tokens
    const bool listed = A.rows && A.rows[(size_t)b * A.row_stride] != 0xffffffffu;
    {
        const long long cap = listed ? A.row_stride : (long long)A.max_pages * P;
        nr = (int)max(0LL, min((long long)nr, cap));
    }
    // Short contexts belong to the CUDA-core kernel launched by the same call: this CTA touches no output.
    const bool skip = nr > 0 && nr < A.min_rows;
    if (skip) nr = 0;
    const int ntiles_all = (nr + AM_TILE - 1) / AM_TILE;
    const bool clustered = A.n_splits > 1;   // the CTAs of a sequence form one thread-block cluster and merge through its shared memory
    const int tps = (ntiles_all + A.n_splits - 1) / A.n_splits;
    const int r_begin = split * tps * AM_TILE;
    const int r_end = min(nr, r_begin + tps * AM_TILE);
    const int ntiles = r_end > r_begin ? (r_end - r_begin + AM_TILE - 1) / AM_TILE : 0;


    if (warp >= AM_GW0 && ntiles > 0) {
        // ------------------------------ gather producers ------------------------------------------
        // Warp g fills the tiles g, g + 4, g + 8, ... (ring stage = tile % 6) in plain program order and never waits for
        // a copy to land: a thread's copies signal the stage's barrier themselves when they are complete
        // (cp.async.mbarrier.arrive), so the warp goes straight on to its next tile as soon as that tile's stage is
        // free. A lane resolves the addresses of two rows of its warp's tile.
        const int g = warp - AM_GW0;
        bool ok = true;
        // The address chain of a row (selected token -> page -> pool row -> scale) is three dependent global loads, and
        // under load each of them comes back only after the tens of kilobytes of copies queued in front of it. It
        // therefore runs as a software pipeline AM_LOOK of the warp's tiles deep PER LEVEL that keeps the raw loaded
        // words in register queues and touches a word only AM_LOOK iterations after it was requested (the warp issues
        // in order: a use right behind its load would stall every copy after it). For row u of the lane:
        //   tk[u][k]               token of the warp's tile i + 2 AM_LOOK + k, being loaded
        //   tok[u][k], pg[u][k]    token of its tile i + AM_LOOK + k and its page-table entry, being loaded
        //   row[u][k], scl[u][k]   pool row of its tile i + k (NONE: write zeros) and its scale; k = 0 is the current tile
        constexpr uint32_t NONE = 0xffffffffu;
        constexpr int AM_LOOK = 2;
        const uint32_t* rowp = listed ? A.rows + (size_t)b * A.row_stride : nullptr;
        const int32_t* btp = A.block_table + (size_t)b * A.max_pages;
        const int pshift = 31 - __clz(P);                  // page sizes are powers of two (checked by the host entry)
        auto load_tok = [&](int j, int u) -> uint32_t {     // j = tile of the split
            const int ri = r_begin + j * AM_TILE + u * 32 + lane;
            if (j >= ntiles || ri >= r_end) return NONE;
            return rowp ? rowp[ri] : (uint32_t)ri;
        };
        auto load_pg = [&](uint32_t t) -> int32_t {
            if (t == NONE) return -1;
            const uint32_t lp = t >> pshift;
            return lp < (uint32_t)A.max_pages ? btp[lp] : -1;
        };
        auto pool_row = [&](uint32_t t, int32_t pg) -> uint32_t {
            return (t != NONE && pg >= 0 && pg < A.n_pool_pages) ? (uint32_t)pg * (uint32_t)P + (t & (uint32_t)(P - 1)) : NONE;
        };
        auto load_scl = [&](uint32_t r) -> float { return r != NONE ? A.pscale[r] : 0.0f; };
        uint32_t tk[2][AM_LOOK], tok[2][AM_LOOK], row[2][AM_LOOK];
        int32_t pg[2][AM_LOOK];
        float scl[2][AM_LOOK];
#pragma unroll
        for (int u = 0; u < 2; ++u) {   // prologue: all token loads at once, then the page entries, then the scales of the first tiles
            uint32_t t0[AM_LOOK];
            int32_t p0[AM_LOOK];
#pragma unroll
            for (int k = 0; k < AM_LOOK; ++k) {
                t0[k] = load_tok(g + AM_GW * k, u); tok[u][k] = load_tok(g + AM_GW * (AM_LOOK + k), u);
                tk[u][k] = load_tok(g + AM_GW * (2 * AM_LOOK + k), u);
            }
#pragma unroll
            for (int k = 0; k < AM_LOOK; ++k) { p0[k] = load_pg(t0[k]); pg[u][k] = load_pg(tok[u][k]); }
#pragma unroll
            for (int k = 0; k < AM_LOOK; ++k) { row[u][k] = pool_row(t0[k], p0[k]); scl[u][k] = load_scl(row[u][k]); }
        }
        // Each lane owns the addresses of two rows, but the COPIES are issued row by row with the 32 lanes of
        // the warp on 32 consecutive 16-byte chunks (the pool row travels by shuffle): one warp
        // instruction then reads 512 contiguous bytes instead of 32 scattered 16-byte pieces. A row past the end
        // (or on an unmapped page) is written as exact zeros by the same instruction with a source size of 0:
        // 0 x (stale NaN code) would poison O.
        for (int j = g; j < ntiles && ok; j += AM_GW) {
            const int s = j % AM_STAGES, use = j / AM_STAGES;
            ok = tc::mbar_wait_warp(&bars.k_empty[s], (use & 1) ^ 1, abort_flag, 41, A.max_polls);
            if (!ok) break;
            uint8_t* kbuf = smem + SM_K0 + s * SM_KSTAGE;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
#pragma unroll 8
                for (int it = 0; it < 32; ++it) {      // latent part: row 32 u + it, chunk = lane
                    const uint32_t r = __shfl_sync(0xffffffffu, row[u][0], it);
                    uint8_t* dst = kbuf + (lane >> 3) * SM_KCHUNK + tc::sw128_chunk(u * 32 + it, lane & 7);
                    tc::cp_async16_zfill(tc::smem_u32(dst), A.pool + (r != NONE ? (size_t)r * AM_W + lane * 16 : 0), r != NONE ? 16u : 0u);
                }
            }
            // a rope tile is free as soon as the two rope MMAs of the tile that used it last are done
            const int rb = j % AM_ROPES;
            ok = tc::mbar_wait_warp(&bars.rope_free[rb], ((j / AM_ROPES) & 1) ^ 1, abort_flag, 42, A.max_polls);
            if (!ok) break;
            uint8_t* rope = smem + SM_ROPE + rb * SM_ROPEBUF;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
#pragma unroll
                for (int it = 0; it < 4; ++it) {       // rope part: 8 rows per instruction, 4 chunks each
                    const int rl = it * 8 + (lane >> 2);
                    const uint32_t r = __shfl_sync(0xffffffffu, row[u][0], rl);
                    uint8_t* dst = rope + sw64_chunk(u * 32 + rl, lane & 3);
                    tc::cp_async16_zfill(tc::smem_u32(dst), A.pool + (r != NONE ? (size_t)r * AM_W + 512 + (lane & 3) * 16 : 0), r != NONE ? 16u : 0u);
                }
            }
            // the stage is full when every lane's copies have landed (32 arrivals by the copies themselves) and the token
            // scales are written (one plain arrival, which also publishes those stores)
            tc::cp_async_mbar_arrive_noinc(&bars.k_full[s]);
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const float sc = scl[u][0];
                const bool live = row[u][0] != NONE && sc > 0.0f;
                float* tp = s_tok + s * AM_TILE + u * 32 + lane;
                tp[0] = live ? sc : 0.0f;
                tp[SM_TOKPLANE / 4] = live ? __log2f(sc) + AM_POFF : -INFINITY;
                tp[2 * (SM_TOKPLANE / 4)] = live ? __frcp_rn(sc) : 0.0f;
            }
            __syncwarp();
            if (lane == 0 && !(A.withhold && j == 0)) tc::mbar_arrive(&bars.k_full[s]);
            // advance the chain: every value consumed here was requested AM_LOOK iterations ago
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const uint32_t row_new = pool_row(tok[u][0], pg[u][0]);
                const uint32_t tok_new = tk[u][0];
#pragma unroll
                for (int k = 0; k + 1 < AM_LOOK; ++k) {
                    row[u][k] = row[u][k + 1]; scl[u][k] = scl[u][k + 1]; tok[u][k] = tok[u][k + 1]; pg[u][k] = pg[u][k + 1]; tk[u][k] = tk[u][k + 1];
                }
                row[u][AM_LOOK - 1] = row_new; scl[u][AM_LOOK - 1] = load_scl(row_new);
                tok[u][AM_LOOK - 1] = tok_new; pg[u][AM_LOOK - 1] = load_pg(tok_new);
                tk[u][AM_LOOK - 1] = load_tok(j + AM_GW * 3 * AM_LOOK, u);
            }
        }
    } else if (warp == AM_QKW) {
        // ------------------------------ QK issuer -------------------------------------------------
        // The two MMA streams, QK(0..n-1) and PV(0..n-1), are each in order and are issued by ONE thread each, from two
        // warps: a thread blocks on the barriers of its own next instruction group only, so neither stream's control
        // latency (barrier observed -> fence -> issue -> commit) sits in the other's way and the tensor pipe takes
        // whichever group arrives first. QK runs ahead of the softmax by up to the four S buffers / ring stages.
        if (lane == 0 && ntiles > 0) {
            const uint32_t id_qk = tc::idesc_e4m3(128, AM_TILE, 0, 0);
            const uint64_t d_qr = smem_desc(tc::smem_u32(smem + SM_QR), 16, 512, 4);
            bool ok = tc::mbar_wait(&bars.q_full, 0, abort_flag, 51, A.max_polls);
            for (int i = 0; i < ntiles && ok; ++i) {   // S(i) = Qcat . K(i)^T
                const int s = i % AM_STAGES, use = i / AM_STAGES, rb = i % AM_ROPES, sb = i % AM_SBUF, suse = i / AM_SBUF;
                ok = tc::mbar_wait(&bars.k_full[s], use & 1, abort_flag, 52, A.max_polls) &&
                     tc::mbar_wait(&bars.s_empty[sb], (suse & 1) ^ 1, abort_flag, 53, A.max_polls);
                if (!ok) break;
                tc::fence_proxy_async();   // the copies wrote through the generic proxy, the MMAs read through the async one
                tc::tc_fence_after();
                const uint64_t d_k = smem_desc(tc::smem_u32(smem + SM_K0 + s * SM_KSTAGE), 16, 1024, 2);
                const uint64_t d_rope = smem_desc(tc::smem_u32(smem + SM_ROPE + rb * SM_ROPEBUF), 16, 512, 4);
                const uint32_t d = TM_S0 + sb * AM_TILE;
                // rope columns first (A from shared memory): their tile is released as soon as these two are done
#pragma unroll
                for (int k = 0; k < 2; ++k) tc::mma_f8(d, d_qr + (uint64_t)(k * 2), d_rope + (uint64_t)(k * 2), id_qk, k != 0);
                tc::mma_commit(&bars.rope_free[rb]);
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int k = 0; k < 4; ++k)   // A from tensor memory: 32 codes = 8 columns per step; descriptor address fields count 16-byte units
                        tc::mma_f8_ta(d, TM_Q + (uint32_t)(c * 32 + k * 8), d_k + (uint64_t)((c * SM_KCHUNK + k * 32) >> 4), id_qk, 1);
                tc::mma_commit(&bars.s_full[sb]);
            }
        }
    } else if (warp == AM_PVW) {
        // ------------------------------ PV issuer -------------------------------------------------
        if (lane == 0 && ntiles > 0) {
            const uint32_t id_pv = tc::idesc_e4m3(128, AM_H, 1, 0);
            const uint64_t d_phi = smem_desc(tc::smem_u32(smem + SM_P), 16, 512, 4);
            const uint64_t d_plo = smem_desc(tc::smem_u32(smem + SM_P + SM_PTERM), 16, 512, 4);
            bool ok = true;
            for (int j = 0; j < ntiles && ok; ++j) {   // O^T += V(j)^T . P'(j)
                const int s = j % AM_STAGES;
                ok = tc::mbar_wait(&bars.p_full, j & 1, abort_flag, 54, A.max_polls);
                if (!ok) break;
                tc::fence_proxy_async();
                tc::tc_fence_after();
                const uint64_t d_v = smem_desc(tc::smem_u32(smem + SM_K0 + s * SM_KSTAGE), SM_KCHUNK, 1024, 2);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
#pragma unroll
                    for (int k = 0; k < 2; ++k)   // p_hi
                        tc::mma_f8(TM_O + c * 64, d_v + (uint64_t)((c * SM_KCHUNK + k * 4096) >> 4), d_phi + (uint64_t)(k * 2), id_pv, (j | k) != 0);
#pragma unroll
                    for (int k = 0; k < 2; ++k)   // p_lo, same accumulator
                        tc::mma_f8(TM_O + c * 64, d_v + (uint64_t)((c * SM_KCHUNK + k * 4096) >> 4), d_plo + (uint64_t)(k * 2), id_pv, 1);
                }
                tc::mma_commit(&bars.k_empty[s]);
                tc::mma_commit(&bars.pv_done);
            }
        }
    } else if (warp < AM_SW) {
        // ------------------------------ softmax + epilogue ---------------------------------------
        // S: TMEM lane = virtual head. Warp (sq, th): lane quarter sq = warp % 4 (heads 16 sq .. 16 sq + 15, hi terms in
        // lanes 0-15 and lo terms in lanes 16-31), token half th = warp / 4 (columns 32 th .. 32 th + 31 of the tile).
        // After the hi + lo exchange lane l keeps the 16 tokens 32 th + 16 (l / 16) .. + 15 of head 16 sq + l % 16.
        // O^T: TMEM lane = latent dim 32 sq + lane of each 128-dim block, head columns 32 th .. 32 th + 31.
        const int sq = warp & 3, th = warp >> 2, tb = lane >> 4;
        const int hd = 16 * sq + (lane & 15);
        const int row = sq * 32 + lane;
        const uint32_t lane_base = ((uint32_t)(sq * 32)) << 16;
        const int h0 = th * AM_HPT;
        const float a_h = s_ahi[hd];
        float l_acc = 0.0f;                                // sum of this thread's weights of head hd
        float m_ref = -INFINITY;                           // reference max of head hd (the same in its four threads)
        bool ok = ntiles > 0;
        for (int i = 0; i < ntiles && ok; ++i) {
            const int s = i % AM_STAGES, use = i / AM_STAGES, sb = i % AM_SBUF, suse = i / AM_SBUF;
            ok = tc::mbar_wait_warp(&bars.k_full[s], use & 1, abort_flag, 61, A.max_polls) &&
                 tc::mbar_wait_warp(&bars.s_full[sb], suse & 1, abort_flag, 62, A.max_polls);
            if (!ok) break;
            tc::tc_fence_after();
            // this thread's 16 tokens: four 16-byte loads per plane (the two half-warps read 64 bytes apart: no bank conflict)
            const float4* ti = reinterpret_cast<const float4*>(s_tok + s * AM_TILE + 32 * th + 16 * tb);
            float s2[16];
            float dmax = -INFINITY;               // max over this thread's tokens of s2' - reference
            {
                uint32_t r[32];
                tc::tmem_ld32(TM_S0 + sb * AM_TILE + lane_base + 32 * th, r);
                tc::tmem_ld_wait();
                tc::tc_fence_before();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&bars.s_empty[sb]);
#pragma unroll
                for (int j4 = 0; j4 < 4; ++j4) {
                    const float4 ts = ti[j4], tc2 = ti[SM_TOKPLANE / 16 + j4];
                    const float sc4[4] = {ts.x, ts.y, ts.z, ts.w}, c24[4] = {tc2.x, tc2.y, tc2.z, tc2.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = 4 * j4 + e;
                        const float mine = __uint_as_float(tb ? r[16 + j] : r[j]);
                        const float give = __uint_as_float(tb ? r[j] : r[16 + j]);
                        const float raw = mine + __shfl_xor_sync(0xffffffffu, give, 16);
                        // rows past the end are exact zeros in shared memory, so their raw scores are 0 and an
                        // additive -inf makes every weight of theirs exactly 0 without a select per element
                        s2[j] = fmaf(raw, a_h * sc4[e], c24[e]);
                        dmax = fmaxf(dmax, s2[j] - m_ref);   // reference is -inf before the first tile
                    }
                }
            }

            // Fast path: no score of the tile exceeds its head's reference by more than AM_LAG, so the
            // references stand and nothing has to be exchanged. One barrier-with-OR decides for the CTA.
            uint32_t slow;
            {
                const uint32_t mine_slow = dmax > AM_LAG + AM_POFF ? 1u : 0u;   // NaN-free: dmax is -inf or finite or +inf (s2 carries AM_POFF, the reference does not)
                asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\t"
                             "bar.red.or.pred q, 1, %2, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                             : "=r"(slow) : "r"(mine_slow), "n"(AM_SOFTMAX_THREADS) : "memory");
            }
            if (slow) {
                // exact per-head tile max: this thread's 16 tokens, its partner lane's, the other token half's warp
                {
                    float mx = s2[0];
#pragma unroll
                    for (int j = 1; j < 16; ++j) mx = fmaxf(mx, s2[j]);
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                    if (lane < 16) s_wmax[th * 64 + hd] = mx;
                }
                tc::named_barrier(2, AM_SOFTMAX_THREADS);
                float fac = 1.0f;
                {
                    const float tm = fmaxf(s_wmax[hd], s_wmax[64 + hd]) - AM_POFF;
                    if (m_ref == -INFINITY) { if (tm > -INFINITY) m_ref = tm; }          // first live tile of this head
                    else if (tm > m_ref) { fac = exp2f(m_ref - tm); m_ref = tm; }          // any growth is taken now
                    if (th == 0 && lane < 16) s_fac[hd] = fac;
                }
                tc::named_barrier(2, AM_SOFTMAX_THREADS);
                // bring O^T and l to the new references. PV(i-1) must have landed first.
                if (i >= 1) { ok = tc::mbar_wait_warp(&bars.pv_done, (i - 1) & 1, abort_flag, 63, A.max_polls); if (!ok) break; }
                tc::tc_fence_after();
                if (i >= 1) {
                    uint32_t r[AM_HPT];
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {   // this thread's dim lane, its head columns of each block
                        tc::tmem_ld32(TM_O + lane_base + c * 64 + h0, r);
                        tc::tmem_ld_wait();
#pragma unroll
                        for (int h = 0; h < AM_HPT; ++h) r[h] = __float_as_uint(__uint_as_float(r[h]) * s_fac[h0 + h]);
                        tc::tmem_st32(TM_O + lane_base + c * 64 + h0, r);
                    }
                    tc::tmem_st_wait();
                }
                l_acc *= fac;
                tc::tc_fence_before();
            }
            // P'' = 2^(s2' - m) = weight * s_tok * 2^AM_POFF as two e4m3 terms (via f16: p <= 256 and the
            // residual p - hi are exact enough in half precision); l accumulates the plain weight.
            // A head that has seen no live token yet has no reference: its scores are all -inf and weigh 0.
            const float m_use = m_ref == -INFINITY ? 0.0f : m_ref;
            uint32_t hi_w[4], lo_w[4];
#pragma unroll
            for (int j = 0; j < 16; j += 4) {
                const float4 ti4 = ti[2 * (SM_TOKPLANE / 16) + (j >> 2)];
                const float inv4[4] = {ti4.x, ti4.y, ti4.z, ti4.w};
                uint32_t chs[2], cls[2];
#pragma unroll
                for (int e = 0; e < 4; e += 2) {
                    float p0, p1;
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(s2[j + e] - m_use));
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(s2[j + e + 1] - m_use));
                    l_acc = fmaf(p0, inv4[e], l_acc);
                    l_acc = fmaf(p1, inv4[e + 1], l_acc);
                    const __half2 ph = __floats2half2_rn(p0, p1);
                    const uint32_t phb = *reinterpret_cast<const uint32_t*>(&ph);
                    uint16_t ch, cl;
                    uint32_t hfb;
                    asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(ch) : "r"(phb));
                    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(hfb) : "h"(ch));
                    const __half2 res = __hsub2(ph, *reinterpret_cast<const __half2*>(&hfb));
                    asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(cl) : "r"(*reinterpret_cast<const uint32_t*>(&res)));
                    chs[e >> 1] = ch; cls[e >> 1] = cl;
                }
                hi_w[j >> 2] = chs[0] | (chs[1] << 16);
                lo_w[j >> 2] = cls[0] | (cls[1] << 16);
            }
            ok = tc::mbar_wait_warp(&bars.pv_done, (i & 1) ^ 1, abort_flag, 64, A.max_polls);   // PV(i - 1) has read the P' tile
            if (!ok) break;
            {
                // row = head, bytes = tokens: this thread's 16 tokens are the 16-byte chunk 2 th + tb of its head's row
                uint8_t* prow = smem + SM_P + sw64_chunk(hd, 2 * th + tb);
                *reinterpret_cast<uint4*>(prow) = make_uint4(hi_w[0], hi_w[1], hi_w[2], hi_w[3]);
                *reinterpret_cast<uint4*>(prow + SM_PTERM) = make_uint4(lo_w[0], lo_w[1], lo_w[2], lo_w[3]);
            }
            tc::fence_proxy_async();
            tc::mbar_arrive(&bars.p_full);
        }

        // ---- epilogue ----
        if (ok && ntiles > 0) ok = tc::mbar_wait_warp(&bars.pv_done, (ntiles - 1) & 1, abort_flag, 65, A.max_polls);
        tc::tc_fence_after();
        // l per head: its four threads (two lanes 16 apart in each of the two token-half warps) meet by one shuffle
        // and one exchange through shared memory.
        tc::named_barrier(1, AM_SOFTMAX_THREADS);
        {
            const float mine = l_acc + __shfl_xor_sync(0xffffffffu, l_acc, 16);
            if (lane < 16) s_wmax[th * 64 + hd] = mine;
        }
        tc::named_barrier(1, AM_SOFTMAX_THREADS);
        if (th == 0 && lane < 16) {
            const int h = hd;
            const float l = s_wmax[h] + s_wmax[64 + h];
            const float m_nat = (m_ref - AM_POFF) * 0.6931471805599453f;   // natural-log units (l and O carry 2^AM_POFF)
            if (clustered) {
                float* xs = reinterpret_cast<float*>(smem + SM_XS);
                xs[h] = (l > 0.0f && ok) ? m_ref : -INFINITY;
                xs[64 + h] = (l > 0.0f && ok) ? l : 0.0f;
            } else if (skip) {
                // nothing: the sequence's output and statistics are written by the CUDA-core kernel
            } else {
                if (A.out_m) A.out_m[(size_t)b * AM_H + h] = l > 0.0f ? m_nat : -INFINITY;
                if (A.out_lse) A.out_lse[(size_t)b * AM_H + h] = l > 0.0f ? m_nat + logf(l) : -INFINITY;
            }
            s_fac[h] = l > 0.0f ? 1.0f / l : 0.0f;
        }
        tc::named_barrier(1, AM_SOFTMAX_THREADS);
        // O^T: this thread's TMEM lane is one latent dim of each 128-dim block; its head columns. For a given head
        // the 32 lanes of a warp hold 32 consecutive dims, so a warp's store covers 64 contiguous bytes of the bf16
        // output row (two full sectors) and the output goes to global memory straight from the registers (a split
        // sequence is merged inside its cluster instead, below).
        float inv_l[AM_HPT];   // 1 / l of this thread's heads (registers: the stores below must not wait on loads)
#pragma unroll
        for (int h = 0; h < AM_HPT; h += 4) {
            const float4 m4 = *reinterpret_cast<const float4*>(s_fac + h0 + h);
            inv_l[h] = m4.x; inv_l[h + 1] = m4.y; inv_l[h + 2] = m4.z; inv_l[h + 3] = m4.w;
        }
#pragma unroll 1
        for (int c = 0; c < 4 && !skip && !clustered; ++c) {
            const int dim = c * 128 + row;
            uint32_t r[AM_HPT];
            if (ntiles > 0 && ok) {
                tc::tmem_ld32(TM_O + lane_base + c * 64 + h0, r);
                tc::tmem_ld_wait();
            } else {
#pragma unroll
                for (int h = 0; h < AM_HPT; ++h) r[h] = 0u;
            }
            uint16_t* gp = A.out + ((size_t)b * AM_H + h0) * AM_KVL + dim;
#pragma unroll
            for (int hq = 0; hq < AM_HPT; ++hq) gp[hq * AM_KVL] = rv_f32_to_bf16(__uint_as_float(r[hq]) * inv_l[hq]);
        }
    }

    if (clustered) {
        // ---- merge of a sequence's splits inside its thread-block cluster ----
        // Every CTA has published its reference maximum and weight sum per head; each scales its own O^T to the
        // common reference and the total sum and lays it out as f32 [head][dim] in its (now idle) ring; then CTA r adds up
        // the heads [64 r / n, 64 (r + 1) / n) over all CTAs through distributed shared memory (plain loads of mapped
        // addresses) and writes them. All threads of all CTAs take part in the three cluster barriers, whatever a
        // bounded wait did before: a CTA that gave up publishes weight sums of zero.
        cg::cluster_group cluster = cg::this_cluster();
        const int n = A.n_splits;
        float* xs = reinterpret_cast<float*>(smem + SM_XS);
        float* stage = reinterpret_cast<float*>(smem + SM_STAGE);
        __syncthreads();
        const bool live = ntiles > 0 && *abort_flag == 0;
        cluster.sync();                                                       // [1] every CTA's (m, l)
        if (warp < AM_SW) {
            const int sq = warp & 3, th = warp >> 2;
            const uint32_t lane_base = ((uint32_t)(sq * 32)) << 16;
            const int h0 = th * AM_HPT;
            if (tid < AM_H) {
                const int h = tid;
                float mg = -INFINITY;
                for (int q = 0; q < n; ++q) mg = fmaxf(mg, cluster.map_shared_rank(xs, q)[h]);
                float L = 0.0f;
                for (int q = 0; q < n; ++q) {
                    const float* px = cluster.map_shared_rank(xs, q);
                    const float lq = px[64 + h];
                    if (lq > 0.0f) L += lq * exp2f(px[h] - mg);
                }
                const float lm = xs[64 + h];
                s_fac[h] = (L > 0.0f && lm > 0.0f) ? exp2f(xs[h] - mg) / L : 0.0f;
                if (split == 0 && !skip) {
                    const float m_nat = (mg - AM_POFF) * 0.6931471805599453f;
                    if (A.out_m) A.out_m[(size_t)b * AM_H + h] = L > 0.0f ? m_nat : -INFINITY;
                    if (A.out_lse) A.out_lse[(size_t)b * AM_H + h] = L > 0.0f ? m_nat + logf(L) : -INFINITY;
                }
            }
            tc::named_barrier(1, AM_SOFTMAX_THREADS);
            tc::tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                const int dim = c * 128 + sq * 32 + lane;
                uint32_t r[AM_HPT];
                if (live) {
                    tc::tmem_ld32(TM_O + lane_base + c * 64 + h0, r);
                    tc::tmem_ld_wait();
                } else {
#pragma unroll
                    for (int h = 0; h < AM_HPT; ++h) r[h] = 0u;
                }
#pragma unroll
                for (int hq = 0; hq < AM_HPT; ++hq)   // lanes = consecutive dims: conflict-free stores
                    stage[(h0 + hq) * AM_KVL + dim] = live ? __uint_as_float(r[hq]) * s_fac[h0 + hq] : 0.0f;
            }
        }
        cluster.sync();                                                       // [2] every CTA's scaled O
        if (warp < AM_SW && !skip) {
            const int hb = split * AM_H / n, he = (split + 1) * AM_H / n;
            for (int e = tid; e < (he - hb) * (AM_KVL / 4); e += AM_SOFTMAX_THREADS) {
                const int h = hb + e / (AM_KVL / 4), d4 = e % (AM_KVL / 4);
                float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                for (int q = 0; q < n; ++q) {
                    const float4 v = *reinterpret_cast<const float4*>(cluster.map_shared_rank(stage, q) + h * AM_KVL + d4 * 4);
                    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                }
                const uint32_t w0 = (uint32_t)rv_f32_to_bf16(acc.x) | ((uint32_t)rv_f32_to_bf16(acc.y) << 16);
                const uint32_t w1 = (uint32_t)rv_f32_to_bf16(acc.z) | ((uint32_t)rv_f32_to_bf16(acc.w) << 16);
                *reinterpret_cast<uint2*>(A.out + ((size_t)b * AM_H + h) * AM_KVL + d4 * 4) = make_uint2(w0, w1);
            }
        }
        cluster.sync();                                                       // [3] nobody reads this CTA's memory any more
    }

    tc::tc_fence_before();
    __syncthreads();
    if (warp == AM_QKW) tc::tmem_dealloc<512>(tmem);
    if (tid == 0 && *abort_flag) atomicCAS(A.err, 0, *abort_flag);
}

// A CTA takes a whole SM (shared memory), and the CTAs of a sequence form one thread-block cluster (co-scheduled
// inside a GPC). A batch is split only as far as all its clusters are resident at once: the largest cluster size
// (<= 8) for which the device reports room for B clusters; anything more would run as a second wave.
int mma_splits(int B) {
    static int cache[149];   // 0 = not asked yet
    if (B <= 0 || B > 74) return 1;
    if (cache[B]) return cache[B];
    cudaFuncSetAttribute(attend_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_TOTAL);
    int n = 148 / B;
    if (n > AM_MAX_SPLITS) n = AM_MAX_SPLITS;
    for (; n > 1; --n) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)n, (unsigned)B); cfg.blockDim = dim3(AM_THREADS); cfg.dynamicSmemBytes = SM_TOTAL;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = (unsigned)n; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        int active = 0;
        if (cudaOccupancyMaxActiveClusters(&active, attend_mma_kernel, &cfg) == cudaSuccess && active >= B) break;
        (void)cudaGetLastError();
    }
    cache[B] = n < 1 ? 1 : n;
    return cache[B];
}

}  // namespace

extern "C" bool rivoli_attend_mma_supported(const DsaGeom* g) {
    return g->n_heads == AM_H && g->kv_lora == AM_KVL && g->rope_dim == AM_ROPE;
}

// scratch layout: [err 256 B]. The error word is sticky: it keeps the first failure
// until rivoli_attend_mma_status reads and clears it, so it must be zero before the first call.
extern "C" size_t rivoli_attend_mma_scratch_bytes(const DsaGeom* g, int B) {
    (void)g; (void)B;
    return 256;
}

extern "C" int rivoli_attend_simt_short_rows(const DsaGeom* g, const uint16_t* q, const uint8_t* latent_pool,
                                             const float* latent_scale, const int32_t* block_table,
                                             const uint32_t* rows, int row_stride, const int32_t* n_rows, int B,
                                             uint16_t* out, float* out_m, float* out_lse, int rows_hi,
                                             cudaStream_t st);

// Below this many attended rows a sequence is served by the f32 CUDA-core kernel instead: with one tile
// or less the two-term fp8 operands of the tensor-core kernel (bf16-class, ~2^-9) no longer average out
// against the 1e-3 absolute tolerance on near-zero outputs.
constexpr int AM_MIN_ROWS = 128;

// Self-test state (rivoli_attend_mma_test_hook): overrides of the next launches, host side only.
static int g_am_min_rows_override = -1, g_am_withhold_once = 0, g_am_max_polls = tc::kMaxPolls;

// Test hook, not for production callers. min_rows >= 0 replaces AM_MIN_ROWS until reset with -1 (0 sends every
// sequence to the tensor-core kernel); withhold != 0 makes the NEXT launch leave out one barrier arrival so that
// its bounded waits run out (the launch returns, the status call reports 1008 and later launches are unaffected);
// max_polls > 0 sets the poll limit of the bounded waits (<= 0 restores the default).
extern "C" __attribute__((visibility("default"))) void rivoli_attend_mma_test_hook(int min_rows, int withhold,
                                                                                    int max_polls) {
    g_am_min_rows_override = min_rows;
    g_am_withhold_once = withhold;
    g_am_max_polls = max_polls > 0 ? max_polls : tc::kMaxPolls;
}

// q_early != 0: the caller guarantees q was complete before the kernel preceding this call in the stream
// was launched (the fused decode step), so the query conversion may overlap that kernel's tail.
// min_rows_hint: a lower bound the caller knows for n_rows over the batch (0 = unknown). With a bound of
// AM_MIN_ROWS or more no sequence needs the CUDA-core arm and its launch is left out.
extern "C" int rivoli_attend_mma_paged_bf16(const DsaGeom* g, const uint16_t* q, const uint8_t* latent_pool,
                                            const float* latent_scale, const int32_t* block_table,
                                            const uint32_t* rows, int row_stride, const int32_t* n_rows, int B,
                                            uint16_t* out, float* out_m, float* out_lse, void* scratch,
                                            int q_early, int min_rows_hint, void* stream) {
    if (!scratch) return 1001;
    if (((uintptr_t)latent_pool | (uintptr_t)scratch | (uintptr_t)q | (uintptr_t)out) & 15) return 1005;
    cudaStream_t st = (cudaStream_t)stream;
    int* err = reinterpret_cast<int*>(scratch);
    const int n_splits = mma_splits(B);
    int min_rows = g_am_min_rows_override >= 0 ? g_am_min_rows_override : AM_MIN_ROWS;
    if (min_rows_hint >= min_rows) min_rows = 0;          // the caller vouches that no sequence is that short
    const int withhold = g_am_withhold_once;
    g_am_withhold_once = 0;

    // short contexts first (a programmatic dependent of whatever precedes this call; its CTAs leave at once
    // for every other sequence), then the tensor-core kernel as a dependent of that launch
    if (min_rows > 1)
        if (int e = rivoli_attend_simt_short_rows(g, q, latent_pool, latent_scale, block_table, rows, row_stride, n_rows,
                                                  B, out, out_m, out_lse, min_rows, st))
            return e;
    rv_drain_error();
    AttendMmaArgs a{q, g->softmax_scale, latent_pool, latent_scale, block_table, rows, row_stride, n_rows,
                    g->page_tokens, g->max_pages_per_seq, g->n_pool_pages, n_splits,
                    out, out_m, out_lse, err,
                    min_rows, q_early ? 1 : 0, g_am_max_polls, withhold};
    cudaFuncSetAttribute(attend_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM_TOTAL);
    // one CTA per (sequence, split); the splits of a sequence are one thread-block cluster and merge inside the kernel
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)n_splits, (unsigned)B); cfg.blockDim = dim3(AM_THREADS);
    cfg.dynamicSmemBytes = (size_t)SM_TOTAL; cfg.stream = st;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    at[1].id = cudaLaunchAttributeClusterDimension;
    at[1].val.clusterDim.x = (unsigned)n_splits; at[1].val.clusterDim.y = 1; at[1].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = n_splits > 1 ? 2 : 1;
    (void)cudaLaunchKernelEx(&cfg, attend_mma_kernel, a);
    return rv_launch_status();
}

// Synchronises `stream`; 1008 if a bounded device-side wait of the last call gave up.
extern "C" int rivoli_attend_mma_status(void* scratch, void* stream) {
    int h = 0;
    cudaError_t e = cudaMemcpyAsync(&h, scratch, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return -(int)e;
    if (h) cudaMemsetAsync(scratch, 0, sizeof(int), (cudaStream_t)stream);
    return h ? 1008 : 0;
}

