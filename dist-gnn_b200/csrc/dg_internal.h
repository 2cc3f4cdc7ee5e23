// Internal declarations shared by the translation units of libdist_gnn_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "dist_gnn_b200.h"

#define DG_CUDA(expr)                                        \
    do {                                                     \
        cudaError_t _e = (expr);                             \
        if (_e != cudaSuccess) return (int)_e;               \
    } while (0)

#define DG_DEFAULT_HEAVY_THRESHOLD 1024
#define DG_DEFAULT_CHUNK           1024

// One chunk of a split (heavy) row: entries [e0, e1) of row `row`; its partial sum lands in scratch row `slot`.
struct dg_chunk {
    int64_t e0, e1;
    int32_t row;
    int32_t slot;
};
// One split row: its chunks are scratch rows [slot0, slot0 + nchunks).
struct dg_heavy_row {
    int32_t row;
    int32_t slot0;
    int32_t nchunks;
    int32_t pad;
};

struct dg_plan {
    int device;
    int32_t m, k;
    int64_t nnz;
    int32_t heavy_threshold, chunk;
    int64_t* rowptr;          // device, m + 1
    const int32_t* col;       // device, borrowed
    dg_chunk* chunks;         // device, n_chunks
    dg_heavy_row* heavy;      // device, n_heavy
    int32_t n_chunks, n_heavy;
    int64_t heavy_nnz, max_row_nnz, touched_columns;
    float* scratch;           // device, n_chunks x scratch_ld floats, grown on demand
    int64_t scratch_floats;
};

// Launches the product with an explicit scratch area (n_chunks x F floats); shared by the plan-owned and the
// fixed-scratch entry points.
int dg_spmm_launch(const dg_plan* plan, const float* val, const float* B, int64_t ldb, float* C, int64_t ldc,
                   int32_t F, float alpha, float beta, uint32_t flags, const float* row_scale, const float* bias,
                   float* scratch, cudaStream_t stream);
int dg_check_spmm_args(const dg_plan* plan, const float* val, const float* B, int64_t ldb, const float* C, int64_t ldc,
                       int32_t F, uint32_t flags, const float* row_scale, const float* bias);
