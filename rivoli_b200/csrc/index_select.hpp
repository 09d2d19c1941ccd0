// Interface between the indexer's host entry points (index_mma.cu) and the cluster selection kernel
// (index_select.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/rivoli_kernels.h"

constexpr int SEL_MAX_CLUSTER = 8;   // portable cluster size

struct SelArgs {
    DsaGeom g;
    const float* scores; int score_stride; const int32_t* seq_len;
    const uint8_t* qcodes; const float* qscales; const float* w; const float* cb;
    const uint8_t* index_pool; const float* index_scale; const int32_t* block_table;
    uint32_t* rows; int32_t* n_sel; int k;
    unsigned int* stats;   // [B][2]: band size, sure-in count (may be NULL)
    int vec_ok;            // score rows and key scales allow 16-byte loads
};

namespace rivoli {
// Cluster size, tokens per thread and threads per CTA for a batch of B sequences of up to score_stride tokens:
// cluster * threads * ept >= score_stride. False if score_stride exceeds 8 * 512 * 32 = 131,072 tokens.
bool select_cluster_plan(int B, int score_stride, int* cluster, int* ept, int* threads);
// Launches the selection as a programmatic dependent of the kernel before it in the stream. 0, a guard code or
// -(cudaError_t).
int launch_index_select_cluster(const SelArgs& a, int B, cudaStream_t st);
}  // namespace rivoli
