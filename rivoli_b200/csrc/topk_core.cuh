// Block-wide exact top-k primitives over order-preserving u32 keys (1024-thread CTAs).
// Selection order = key descending, index ascending on ties; output ascending by index.
// Contract and tie rule: crates/backend/kernels/indexer.hip:143-257 of the reference.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

constexpr int TK_THREADS = 1024;
constexpr int TK_WARPS = TK_THREADS / 32;

// Ascending key iff ascending float; -0.0 canonicalised to +0.0 (indexer.hip:156-159).
__device__ __forceinline__ uint32_t topk_key(float v) {
    uint32_t b = (v == 0.0f) ? 0u : __float_as_uint(v);
    return b ^ ((uint32_t)((int32_t)b >> 31) | 0x80000000u);
}
__device__ __forceinline__ float topk_unkey(uint32_t k) {
    const uint32_t b = (k & 0x80000000u) ? (k ^ 0x80000000u) : ~k;
    return __uint_as_float(b);
}

struct TkShared {
    uint32_t whist[TK_WARPS][256];   // one histogram per warp: no cross-warp atomic contention
    uint32_t hist[256];
    uint32_t wcnt[TK_WARPS];
    uint32_t red[2][TK_WARPS];       // double-buffered block reductions (tk_block_sum)
    uint32_t pivot, need;
};

// The part of TkShared the register-resident primitives need (block reductions and scans).
struct TkSharedLite {
    uint32_t wcnt[TK_WARPS];
    uint32_t red[2][TK_WARPS];
};

// Block-wide sum with ONE barrier per call: per-warp partials go to red[buf], every warp then
// re-reduces the 32 partials. `buf` alternates between calls, which is what makes the single
// barrier sufficient (a warp can be at most one call ahead of the slowest one).
template <class SH>
__device__ __forceinline__ uint32_t tk_block_sum(uint32_t v, SH& sh, int& buf) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = __reduce_add_sync(0xffffffffu, v);
    if (lane == 0) sh.red[buf][warp] = v;
    __syncthreads();
    const uint32_t t = __reduce_add_sync(0xffffffffu, sh.red[buf][lane]);
    buf ^= 1;
    return t;
}

template <class SH>
__device__ __forceinline__ uint32_t tk_block_max(uint32_t v, SH& sh, int& buf) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = __reduce_max_sync(0xffffffffu, v);
    if (lane == 0) sh.red[buf][warp] = v;
    __syncthreads();
    const uint32_t t = __reduce_max_sync(0xffffffffu, sh.red[buf][lane]);
    buf ^= 1;
    return t;
}

// k-th largest key by bisection on the key bits, MSB first, over keys held in REGISTERS
// (any fixed assignment of elements to threads; slots past the end hold 0 and never count).
// After `nbits` steps the result T has its low (32 - nbits) bits clear and satisfies
//   #(key >= T) >= kk   and   #(key >= T + 2^(32-nbits)) < kk   (or that sum overflows),
// so with nbits = 32 T is exactly the kk-th largest key. No atomics, no data-dependent cost:
// tie-dominated arrays take the same time as random ones.
template <int EPT, class SH>
__device__ __forceinline__ uint32_t tk_bisect(const uint32_t (&key)[EPT], uint32_t kk, int nbits, SH& sh, int& buf) {
    uint32_t T = 0u;
    for (int bit = 31; bit >= 32 - nbits; --bit) {
        const uint32_t cand = T | (1u << bit);
        uint32_t c = 0;
#pragma unroll
        for (int j = 0; j < EPT; ++j) c += key[j] >= cand ? 1u : 0u;
        if (tk_block_sum(c, sh, buf) >= kk) T = cand;
    }
    return T;
}

// Ascending compaction for keys held in registers with CONTIGUOUS ownership (thread t holds
// elements t*EPT .. t*EPT+EPT-1): one packed block-wide exclusive scan of (#key > pivot,
// #key == pivot), then every thread writes its own selected indices in order. Same slot rule
// as tk_compact. One barrier. Every thread must call it.
template <int EPT, class SH>
__device__ __forceinline__ void tk_compact_contig(const uint32_t (&key)[EPT], int nt, uint32_t pivot, uint32_t need,
                                                  SH& sh, uint32_t* __restrict__ out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int i0 = tid * EPT;
    uint32_t v = 0u;
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        const bool live = i0 + j < nt;
        v += (live && key[j] > pivot) ? 1u : 0u;
        v += (live && key[j] == pivot) ? 0x10000u : 0u;
    }
    uint32_t incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) sh.wcnt[warp] = incl;
    __syncthreads();
    const uint32_t cw = sh.wcnt[lane];
    const uint32_t excl = __reduce_add_sync(0xffffffffu, lane < warp ? cw : 0u) + incl - v;
    uint32_t g = excl & 0xffffu, e = excl >> 16;
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        const int i = i0 + j;
        if (i < nt) {
            if (key[j] > pivot) { out[g + (e < need ? e : need)] = (uint32_t)i; ++g; }
            else if (key[j] == pivot) { if (e < need) out[g + e] = (uint32_t)i; ++e; }
        }
    }
}

template <int EPT, class SH>
__device__ __forceinline__ uint32_t tk_count_gt(const uint32_t (&key)[EPT], uint32_t T, SH& sh, int& buf) {
    uint32_t c = 0;
#pragma unroll
    for (int j = 0; j < EPT; ++j) c += key[j] > T ? 1u : 0u;
    return tk_block_sum(c, sh, buf);
}

// Four 8-bit passes, MSB first: the key of the kk-th largest entry and how many of the
// entries tied at it the selection takes. KeyAt(i) returns the key of element i.
// Every thread of the CTA must call it. Each warp counts into its own histogram, so tie-heavy
// arrays (ReLU zeros) never serialise the whole CTA on one bin.
template <class KeyAt>
__device__ __forceinline__ void tk_radix_select(KeyAt key_at, int nt, uint32_t kk, TkShared& sh, uint32_t& pivot_out,
                                                uint32_t& need_out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t pivot = 0u, mask = 0u, need = kk;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = tid; i < TK_WARPS * 256; i += TK_THREADS) (&sh.whist[0][0])[i] = 0u;
        __syncthreads();
        for (int base = 0; base < nt; base += TK_THREADS) {
            const int i = base + tid;
            uint32_t bin = 0xffffffffu;
            if (i < nt) {
                const uint32_t u = key_at(i);
                if ((u & mask) == pivot) bin = (u >> shift) & 0xffu;
            }
            // shared-memory atomic on this warp's own histogram: only lanes of one warp can collide
            if (bin != 0xffffffffu) atomicAdd(&sh.whist[warp][bin], 1u);
        }
        __syncthreads();
        if (tid < 256) {
            uint32_t t = 0;
#pragma unroll 8
            for (int w2 = 0; w2 < TK_WARPS; ++w2) t += sh.whist[w2][tid];
            sh.hist[tid] = t;
        }
        __syncthreads();
        if (warp == 0) {
            // lane owns bins 8*lane .. 8*lane+7; acc = entries in strictly higher bins
            uint32_t h[8], tot = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) { h[j] = sh.hist[lane * 8 + j]; tot += h[j]; }
            uint32_t incl = tot;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_down_sync(0xffffffffu, incl, o);
                if (lane + o < 32) incl += v;
            }
            uint32_t acc = incl - tot;
#pragma unroll
            for (int j = 7; j >= 0; --j) {
                if (acc < need && need <= acc + h[j]) {
                    sh.pivot = pivot | ((uint32_t)(lane * 8 + j) << shift);
                    sh.need = need - acc;
                }
                acc += h[j];
            }
        }
        __syncthreads();
        pivot = sh.pivot;
        need = sh.need;
        mask |= 0xffu << shift;
    }
    pivot_out = pivot;
    need_out = need;
}

// Ascending compaction: slot(i) = #(key > pivot before i) + min(#(key == pivot before i), need).
// Ballots and a fixed scan order decide every slot; no atomics. Every thread must call it.
template <class KeyAt>
__device__ __forceinline__ void tk_compact(KeyAt key_at, int nt, uint32_t kk, uint32_t pivot, uint32_t need, TkShared& sh,
                                           uint32_t* __restrict__ out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t base_gt = 0u, base_eq = 0u;
    for (int base = 0; base < nt; base += TK_THREADS) {
        const int i = base + tid;
        const bool live = i < nt;
        const uint32_t u = live ? key_at(i) : 0u;
        const bool gt = live && u > pivot, eq = live && u == pivot;
        const uint32_t mg = __ballot_sync(0xffffffffu, gt), me = __ballot_sync(0xffffffffu, eq);
        if (lane == 0) sh.wcnt[warp] = (uint32_t)__popc(mg) | ((uint32_t)__popc(me) << 16);
        __syncthreads();
        // prefix over the 32 warp counts: lane w holds warp w's packed count
        const uint32_t cw = sh.wcnt[lane];
        const uint32_t pre = __reduce_add_sync(0xffffffffu, lane < warp ? cw : 0u);
        const uint32_t tot = __reduce_add_sync(0xffffffffu, cw);
        const uint32_t lt = (1u << lane) - 1u;
        const uint32_t g = base_gt + (pre & 0xffffu) + (uint32_t)__popc(mg & lt);
        const uint32_t e = base_eq + (pre >> 16) + (uint32_t)__popc(me & lt);
        if (gt || (eq && e < need)) out[g + (e < need ? e : need)] = (uint32_t)i;
        base_gt += tot & 0xffffu;
        base_eq += tot >> 16;
        __syncthreads();
        if (base_gt + min(base_eq, need) >= kk) break;  // uniform: every row is placed
    }
}
