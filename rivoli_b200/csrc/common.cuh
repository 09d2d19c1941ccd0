// Shared host/device helpers for librivolikernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/rivoli_kernels.h"

#define RIVOLI_API extern "C" __attribute__((visibility("default")))

// Launch epilogue of every entry point: 0 or -(cudaError_t), after draining any stale
// error before the launch so the code read back belongs to this launch.
static inline void rv_drain_error() { (void)cudaGetLastError(); }
static inline int rv_launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : -(int)e;
}

// Programmatic dependent launch: a kernel launched this way may begin (its prologue, up to its own
// rv_grid_dep_wait()) while the kernel before it in the stream is still running, once every CTA of that
// kernel has called rv_grid_dep_trigger() or exited. rv_grid_dep_wait() returns when the preceding kernel
// has completed and its writes are visible. Both are no-ops in a kernel launched the ordinary way.
#ifdef __CUDACC__
__device__ __forceinline__ void rv_grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void rv_grid_dep_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
template <class... KArgs, class... Args>
static inline void rv_launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                       Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    (void)cudaLaunchKernelEx(&cfg, kernel, args...);   // the caller reads the launch status afterwards
}
#endif

// Measurement hook (rivoli_dsa_step_set_timing_events): when set, the decode-step entry points record event k
// on their stream before kernel k of the step (and the last one after it), so that a benchmark can read each
// kernel's own duration. An event record between two launches also takes away their programmatic overlap,
// which is what a per-kernel time wants; it is off (NULL) in every other use.
extern "C" cudaEvent_t* rivoli_step_timing_events();
static inline void rv_stage_event(int k, cudaStream_t st) {
    cudaEvent_t* ev = rivoli_step_timing_events();
    if (ev) (void)cudaEventRecord(ev[k], st);
}

static inline bool rv_is_pow2(int x) { return x > 0 && (x & (x - 1)) == 0; }

// Geometry guard shared by every paged entry point. Decided on the host; nothing is
// dereferenced on the device when it fails.
static inline int rv_check_geom(const DsaGeom* g) {
    if (!g) return 1001;
    if (g->n_heads <= 0 || g->kv_lora <= 0 || g->rope_dim <= 0 || g->index_heads <= 0 ||
        g->index_dim <= 0 || g->page_tokens <= 0 || g->top_k <= 0 || g->max_pages_per_seq <= 0 ||
        g->n_pool_pages <= 0)
        return 1001;
    if (g->kv_lora > 512 || (g->kv_lora % 128) != 0) return 1004;
    if ((g->rope_dim % 16) != 0 || g->rope_dim > 128) return 1004;
    if ((g->index_dim % 16) != 0 || g->index_dim > 512) return 1004;
    if (!rv_is_pow2(g->page_tokens)) return 1003;
    if (g->n_heads > 128 || g->index_heads > 64) return 1002;
    return 0;
}

__device__ __forceinline__ float rv_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float rv_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
