// Exact, deterministic top-k row selection (the DSA attend row set).
//
// Order = score descending, index ascending on ties, -0.0 == +0.0; the selected SET is
// emitted ascending by index and nothing is written past min(k, nt). Same contract as the
// reference's crates/backend/kernels/indexer.hip:143-257 and the host rule
// crates/core/src/routing.rs:42-61 + sort (crates/engine/tests/kernel_vector.rs:126-131).
//
// One CTA of 1024 threads per sequence. The order-preserving keys are staged ONCE in
// shared memory (up to 56 Ki scores = 224 KiB; B200 has 227 KiB per CTA), so the four
// radix passes and the compaction sweep never go back to HBM: the kernel reads each score
// exactly once. Longer sequences fall back to re-reading global memory (L2 resident).
// Compaction uses ballots and a fixed scan order: no atomics decide an output slot.
#include "common.cuh"

constexpr int TK_THREADS = 1024;
constexpr int TK_WARPS = TK_THREADS / 32;
constexpr int TK_SMEM_KEYS = 56 * 1024;

// Ascending key iff ascending float; -0.0 canonicalised to +0.0 (indexer.hip:156-159).
__device__ __forceinline__ uint32_t topk_key(float v) {
    uint32_t b = (v == 0.0f) ? 0u : __float_as_uint(v);
    return b ^ ((uint32_t)((int32_t)b >> 31) | 0x80000000u);
}

__global__ void __launch_bounds__(TK_THREADS)
index_topk_kernel(const float* __restrict__ scores, long long score_stride, const int32_t* __restrict__ seq_len,
                  int nt_single, int k, uint32_t* __restrict__ rows, long long row_stride,
                  int32_t* __restrict__ n_sel, int smem_keys, int nt_cap) {
    extern __shared__ uint32_t skeys[];
    __shared__ uint32_t hist[256];
    __shared__ uint32_t wcnt[TK_WARPS];
    __shared__ uint32_t sh_pivot, sh_need;

    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nt = min(seq_len ? seq_len[b] : nt_single, nt_cap);  // never read past a score row
    const float* s = scores + (size_t)b * score_stride;
    uint32_t* out = rows + (size_t)b * row_stride;
    const int kk = min(k, nt);
    if (tid == 0 && n_sel) n_sel[b] = kk > 0 ? kk : 0;
    if (kk <= 0) return;
    if (kk == nt) {  // everything is selected: the ascending set is the identity
        for (int i = tid; i < nt; i += TK_THREADS) out[i] = (uint32_t)i;
        return;
    }
    const bool staged = nt <= smem_keys;
    if (staged) {
        for (int i = tid; i < nt; i += TK_THREADS) skeys[i] = topk_key(s[i]);
        __syncthreads();
    }
    auto key_at = [&](int i) -> uint32_t { return staged ? skeys[i] : topk_key(s[i]); };

    // Four 8-bit passes, MSB first: converge on the key of the k-th largest score and on how
    // many of the entries tied at it the selection takes.
    uint32_t pivot = 0u, mask = 0u, need = (uint32_t)kk;
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0u;
        __syncthreads();
        // Warp-aggregated counting: tie-heavy score arrays (ReLU zeros) put whole warps in one
        // bin, and one atomic per distinct bin per warp keeps that from serialising.
        for (int base = 0; base < nt; base += TK_THREADS) {
            const int i = base + tid;
            uint32_t bin = 0xffffffffu;
            if (i < nt) {
                const uint32_t u = key_at(i);
                if ((u & mask) == pivot) bin = (u >> shift) & 0xffu;
            }
            const uint32_t peers = __match_any_sync(0xffffffffu, bin);
            if (bin != 0xffffffffu && lane == __ffs(peers) - 1) atomicAdd(&hist[bin], (uint32_t)__popc(peers));
        }
        __syncthreads();
        if (warp == 0) {
            // lane owns bins 8*lane .. 8*lane+7; above[] = entries in strictly higher bins
            uint32_t h[8], tot = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) { h[j] = hist[lane * 8 + j]; tot += h[j]; }
            uint32_t incl = tot;  // inclusive suffix sum over lanes (lane 31 highest bins)
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_down_sync(0xffffffffu, incl, o);
                if (lane + o < 32) incl += v;
            }
            uint32_t acc = incl - tot;  // entries in lanes above this one
#pragma unroll
            for (int j = 7; j >= 0; --j) {
                if (acc < need && need <= acc + h[j]) {
                    sh_pivot = pivot | ((uint32_t)(lane * 8 + j) << shift);
                    sh_need = need - acc;
                }
                acc += h[j];
            }
        }
        __syncthreads();
        pivot = sh_pivot;
        need = sh_need;
        mask |= 0xffu << shift;
    }

    // Compaction, ascending: slot(i) = #(key > pivot before i) + min(#(key == pivot before i), need).
    uint32_t base_gt = 0u, base_eq = 0u;
    for (int base = 0; base < nt; base += TK_THREADS) {
        const int i = base + tid;
        const bool live = i < nt;
        const uint32_t u = live ? key_at(i) : 0u;
        const bool gt = live && u > pivot, eq = live && u == pivot;
        const uint32_t mg = __ballot_sync(0xffffffffu, gt), me = __ballot_sync(0xffffffffu, eq);
        if (lane == 0) wcnt[warp] = (uint32_t)__popc(mg) | ((uint32_t)__popc(me) << 16);
        __syncthreads();
        uint32_t pre = 0u, tot = 0u;
#pragma unroll 8
        for (int w2 = 0; w2 < TK_WARPS; ++w2) {
            const uint32_t c = wcnt[w2];
            if (w2 < warp) pre += c;
            tot += c;
        }
        const uint32_t lt = (1u << lane) - 1u;
        const uint32_t g = base_gt + (pre & 0xffffu) + (uint32_t)__popc(mg & lt);
        const uint32_t e = base_eq + (pre >> 16) + (uint32_t)__popc(me & lt);
        if (gt || (eq && e < need)) out[g + (e < need ? e : need)] = (uint32_t)i;
        base_gt += tot & 0xffffu;
        base_eq += tot >> 16;
        __syncthreads();
        if (base_gt + min(base_eq, need) >= (uint32_t)kk) break;  // uniform: every row is placed
    }
}

static int launch_topk(const float* scores, long long score_stride, const int32_t* seq_len, int nt_single,
                       int B, int k, uint32_t* rows, long long row_stride, int32_t* n_sel, int max_nt,
                       cudaStream_t st) {
    // Per device and cheap, so it is simply repeated on every launch.
    cudaFuncSetAttribute(index_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         TK_SMEM_KEYS * (int)sizeof(uint32_t));
    const int staged = max_nt <= TK_SMEM_KEYS ? max_nt : 0;
    rv_drain_error();
    index_topk_kernel<<<B, TK_THREADS, (size_t)staged * sizeof(uint32_t), st>>>(
        scores, score_stride, seq_len, nt_single, k, rows, row_stride, n_sel, staged, max_nt);
    return rv_launch_status();
}

RIVOLI_API int rivoli_index_topk(const float* scores, int nt, int k, unsigned int* rows) {
    if (nt <= 0 || k <= 0) return 1001;
    if (k > nt) k = nt;
    return launch_topk(scores, 0, nullptr, nt, 1, k, rows, 0, nullptr, nt, 0);
}

RIVOLI_API int rivoli_index_topk_batched(const float* scores, int score_stride, const int32_t* seq_len,
                                         int B, int k, uint32_t* rows, int32_t* n_sel, void* stream) {
    if (B <= 0 || k <= 0 || score_stride <= 0 || !scores || !seq_len || !rows) return 1001;
    return launch_topk(scores, score_stride, seq_len, 0, B, k, rows, k, n_sel, score_stride,
                       (cudaStream_t)stream);
}
