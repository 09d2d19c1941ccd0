// Exact, deterministic top-k row selection (the DSA attend row set).
//
// Order = score descending, index ascending on ties, -0.0 == +0.0; the selected SET is
// emitted ascending by index and nothing is written past min(k, nt). Same contract as the
// reference's crates/backend/kernels/indexer.hip:143-257 and the host rule
// crates/core/src/routing.rs:42-61 + sort (crates/engine/tests/kernel_vector.rs:126-131).
//
// One CTA of 1024 threads per sequence. The order-preserving keys are staged ONCE in
// shared memory (up to 47 Ki scores = 188 KiB; B200 has 227 KiB per CTA), so the four
// radix passes and the compaction sweep never go back to HBM: the kernel reads each score
// exactly once. Longer sequences fall back to re-reading global memory (L2 resident).
// Compaction uses ballots and a fixed scan order: no atomics decide an output slot.
#include "common.cuh"
#include "topk_core.cuh"

constexpr int TK_SMEM_KEYS = 47 * 1024;   // 188 KiB of keys + 34 KiB of per-warp histograms < 227 KiB

__global__ void __launch_bounds__(TK_THREADS)
index_topk_kernel(const float* __restrict__ scores, long long score_stride, const int32_t* __restrict__ seq_len,
                  int nt_single, int k, uint32_t* __restrict__ rows, long long row_stride,
                  int32_t* __restrict__ n_sel, int smem_keys, int nt_cap) {
    extern __shared__ uint32_t skeys[];
    __shared__ TkShared sh;

    const int b = blockIdx.x, tid = threadIdx.x;
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
    uint32_t pivot, need;
    tk_radix_select(key_at, nt, (uint32_t)kk, sh, pivot, need);
    tk_compact(key_at, nt, (uint32_t)kk, pivot, need, sh, out);
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
