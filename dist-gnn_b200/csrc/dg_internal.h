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

// Rows longer than the threshold are cut into chunks, one warp each.  A warp walks its entries one dependent gather after
// the other, so the longest row or chunk bounds a kernel's duration from below: 256 entries keep that tail short for the
// small column blocks of an 8-rank stage loop (2.0x faster than 1024 there) and are 4 % faster on the whole graph too.
#define DG_DEFAULT_HEAVY_THRESHOLD 256
#define DG_DEFAULT_CHUNK           256

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

// One row whose entries span more than one task of the streaming kernel: its partial sums sit in carry slots
// 2*t_first+1 (the piece that starts the row) and 2*t (t_first < t <= t_last, pieces that continue it).
struct dg_split_row {
    int32_t row;
    int32_t t_first;
    int32_t t_last;
    int32_t pad;
};

#define DG_DEFAULT_TASK_NNZ 1024

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
    float* scratch;           // device, grown on demand to dg_scratch_floats(plan, F)
    int64_t scratch_floats;
    // streaming kernel: the entry list cut into tasks of task_nnz entries, one warp each
    int32_t task_nnz, n_tasks, n_split;
    int32_t* task_first_row;  // device, n_tasks: the row that holds entry t * task_nnz
    dg_split_row* split;      // device, n_split rows that span tasks, ascending
    int* status;              // device word: set non-zero by a kernel that gave up on a bounded wait
};

// Scratch floats one product of width F may touch: split-row chunks (row kernels) or two carry rows per task (streaming).
static inline int64_t dg_scratch_floats(const dg_plan* p, int32_t F)
{
    const int64_t a = (int64_t)p->n_chunks * F, b = 2 * (int64_t)p->n_tasks * F;
    return a > b ? a : b;
}
int dg_stream_selected();     // non-zero while dg_select_kernel(2) is in force
int dg_spmm_stream_eligible(const dg_plan* plan, const float* B, int64_t ldb, const float* C, int64_t ldc, int32_t F);
int dg_spmm_stream_launch(const dg_plan* plan, const float* val, const float* B, int64_t ldb, float* C, int64_t ldc,
                          int32_t F, float alpha, float beta, uint32_t flags, const float* row_scale, const float* bias,
                          float* scratch, cudaStream_t stream, int* launches);

// Launches the product with an explicit scratch area (n_chunks x F floats); shared by the plan-owned and the
// fixed-scratch entry points.
int dg_spmm_launch(const dg_plan* plan, const float* val, const float* B, int64_t ldb, float* C, int64_t ldc,
                   int32_t F, float alpha, float beta, uint32_t flags, const float* row_scale, const float* bias,
                   float* scratch, cudaStream_t stream);
int dg_spmm_launch_rows(const dg_plan* plan, const float* val, const float* B, int64_t ldb, float* C, int64_t ldc,
                        int32_t F, float alpha, float beta, uint32_t flags, const float* row_scale, const float* bias,
                        float* scratch, cudaStream_t stream);
int dg_plan_build(const int32_t* row, const int32_t* col, int64_t nnz, int32_t m, int32_t k, int32_t heavy_threshold,
                  int32_t chunk, bool lean, void* stream, dg_plan** out);
int dg_spmm_prepare(const dg_plan* plan, int32_t F, cudaStream_t stream);
int dg_check_spmm_args(const dg_plan* plan, const float* val, const float* B, int64_t ldb, const float* C, int64_t ldc,
                       int32_t F, uint32_t flags, const float* row_scale, const float* bias);
