/*
 * dist_gnn_b200 - C ABI of the B200 (sm_100a) broadcast-SpMM library.
 *
 * This is the boundary a binding of the reference project talks to: plain pointers and sizes, no
 * framework types.  It replaces, for the 1D / 1.5D broadcast-based distributed SpMM of
 * light_dist_gnn, (a) the cuSPARSE wrapper spmm_cusparse (light_dist_gnn/spmm_cpp/spmm.cpp:17-33) and
 * (b) the per-stage torch.distributed.broadcast + spmm loop (light_dist_gnn/models/gcn.py:16-30;
 * 1.5D: 1D_CAGNET/dist_15d.py:61-106).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer on the current CUDA device unless the name says host_;
 *   - dense matrices are row-major fp32, sparse indices int32 (base 0), row offsets int64;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream); all work is
 *     enqueued asynchronously unless stated otherwise;
 *   - every function returns 0 on success, a negative DG_ERR_* for rejected arguments, a positive
 *     cudaError_t for CUDA failures and 10000 + ncclResult_t for NCCL failures; nothing throws.
 */
#ifndef DIST_GNN_B200_H
#define DIST_GNN_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DG_OK                 0
#define DG_ERR_NULL          -1   /* a required pointer is NULL */
#define DG_ERR_DIMS          -2   /* negative or inconsistent sizes / leading dimensions */
#define DG_ERR_INDEX         -3   /* row ids not ascending, or an index outside [0,m) x [0,k) */
#define DG_ERR_UNSUPPORTED   -4   /* valid request this build does not implement */
#define DG_ERR_STATE         -5   /* object used in the wrong state (e.g. destroyed, wrong device) */
#define DG_ERR_SCRATCH       -6   /* request needs more scratch than the fixed-size variant holds */
#define DG_NCCL_ERROR_BASE    10000

/* epilogue_flags of dg_spmm_csr: out[i,:] = act( row_scale[i] * (alpha*A*B + beta*C)[i,:] + bias ) */
#define DG_EPI_ROW_SCALE      1u  /* multiply row i by row_scale[i]  (e.g. a D^-1/2 factor kept out of A's values) */
#define DG_EPI_BIAS           2u  /* add bias[f] to column f */
#define DG_EPI_RELU           4u  /* max(x, 0) last */

typedef struct dg_plan dg_plan;   /* CSR view + degree bins of one sparse block, lives on one device */
typedef struct dg_comm dg_comm;   /* one NCCL communicator with its side stream and events */

typedef struct dg_plan_stats {
    int64_t nnz;
    int32_t m, k;
    int32_t heavy_threshold;      /* rows with more entries than this are split into chunks */
    int32_t chunk;                /* entries per chunk of a split row */
    int32_t heavy_rows;           /* number of split rows */
    int32_t heavy_chunks;         /* total chunks (scratch rows) */
    int64_t heavy_nnz;            /* entries inside split rows */
    int64_t max_row_nnz;
    int64_t touched_columns;      /* distinct column ids in the block (for compulsory-traffic accounting) */
} dg_plan_stats;

const char* dg_strerror(int code);
int dg_version(void);

/* ---- plan: COO (row-sorted, as torch's coalesce() leaves it) -> CSR row offsets + degree bins -----------------
 * Replaces the per-call descriptor set-up of spmm.cpp:19-24 (and the coo2csr of spmm_original.cpp:140-146) by a
 * one-off step.  `row` is only read during creation; `col` is BORROWED: it must stay valid and unchanged for the
 * life of the plan.  Validates ordering and ranges on the device and returns DG_ERR_INDEX instead of launching
 * anything on bad input.  Synchronises `stream` once (one-off cost).  heavy_threshold/chunk <= 0 pick defaults. */
int dg_plan_create(const int32_t* row, const int32_t* col, int64_t nnz, int32_t m, int32_t k,
                   void* stream, dg_plan** out);
int dg_plan_create_ex(const int32_t* row, const int32_t* col, int64_t nnz, int32_t m, int32_t k,
                      int32_t heavy_threshold, int32_t chunk, void* stream, dg_plan** out);
int dg_plan_destroy(dg_plan* plan);
int dg_plan_get_stats(const dg_plan* plan, dg_plan_stats* host_out);
/* The streaming kernel cuts the entry list into tasks of `task_nnz` entries (one warp each; default 1024).  This
 * rebuilds the task tables for another size (<= 0 restores the default); synchronises `stream`. */
int dg_plan_set_task_size(dg_plan* plan, int32_t task_nnz, void* stream);
/* Kernel family of the local product: 0 = automatic (the row kernels), 1 = row kernels only, 2 = the streaming kernel
 * (asynchronous copies through shared memory, entry-balanced tasks) wherever the operands allow it (rows of B and C
 * 16-byte aligned and at least 64 floats wide).  Process-wide; also settable with DG_SPMM_KERNEL=rows|stream. */
int dg_select_kernel(int family);
/* Reads the plan's device status word (synchronises `stream`).  Reserved for kernels with bounded device-side waits;
 * no current kernel waits on anything, so it reads 0. */
int dg_plan_device_status(const dg_plan* plan, int* host_status, void* stream);
/* copies the m+1 row offsets to host memory (synchronises `stream`); used to check CSR indexing bit for bit */
int dg_plan_copy_rowptr(const dg_plan* plan, int64_t* host_rowptr, void* stream);

/* ---- local product: C = epilogue(alpha * A * B + beta * C) ------------------------------------------------------
 * A = plan (m x k) with values `val` (nnz, in the COO order the plan was built from); B is k x F with leading
 * dimension ldb, C is m x F with leading dimension ldc (in floats).  beta == 0 never reads C.  Replaces
 * cusparseSpMM(COO_ALG4) at spmm.cpp:26-28.  Results are bit-reproducible run to run (no float atomics).
 * Split rows use plan-owned scratch that grows on first use for a wider F (that call allocates and
 * synchronises); two products on the same plan must not overlap in time. */
int dg_spmm_csr(const dg_plan* plan, const float* val, const float* B, int64_t ldb, float* C, int64_t ldc,
                int32_t F, float alpha, float beta, uint32_t epilogue_flags, const float* row_scale,
                const float* bias, void* stream);

/* ---- the same product without any device allocation (no counterpart in the reference) --------------------------------
 * For hosts that cannot let a library call cudaMalloc: all device memory already sits in their own pool, or they run
 * a latency-critical loop that must not take the device-wide synchronisation an allocation implies.  Identical
 * arguments and results to dg_spmm_csr, but the partial sums of split rows go to a fixed 16 MiB array inside the
 * library image (held by every GPU that loads the library, shared by all calls on that GPU).  Returns DG_ERR_SCRATCH
 * when heavy_chunks * F exceeds dg_static_scratch_capacity() floats.  Calls that overlap in time on one GPU race on
 * the array.  The array is materialised on a device (16 MiB, by the CUDA module loader) the first time its address is
 * resolved there: dg_static_scratch_prepare() does that for the current device and is meant to be called once where an
 * allocation is still acceptable (beside dg_plan_create, before any stream capture); without it the first
 * dg_spmm_csr_static on a device does it.  Always runs the row kernels; not counted by dg_profile_begin/_end. */
int dg_spmm_csr_static(const dg_plan* plan, const float* val, const float* B, int64_t ldb, float* C, int64_t ldc,
                       int32_t F, float alpha, float beta, uint32_t epilogue_flags, const float* row_scale,
                       const float* bias, void* stream);
int64_t dg_static_scratch_capacity(void);
int dg_static_scratch_prepare(void);

/* ---- drop-in for spmm_cusparse(row, col, val, A_row, A_col, B, C, alpha, beta) (spmm.cpp:17) ----------------------
 * Same nine operands plus the dense width F and the stream; B is k x F and C is m x F, both contiguous.
 * Builds a transient plan per call (allocates and synchronises); callers that reuse a block should hold a plan. */
int dg_spmm_coo(const int32_t* row, const int32_t* col, const float* val, int64_t nnz, int32_t m, int32_t k,
                const float* B, float* C, int32_t F, float alpha, float beta, void* stream);

/* ---- communicators (NCCL over NVLink / NVSwitch) ------------------------------------------------------------------
 * Replace the torch.distributed process groups the stage loop broadcasts in (light_dist_gnn/dist_utils/env.py:47-54;
 * 1.5D row / column groups: 1D_CAGNET/utils.py:36-49).  One process per GPU; rank 0 makes an id, every rank passes
 * the same 128 bytes to dg_comm_create with the device it will use current.  dg_comm_split makes the sub-groups. */
int dg_comm_unique_id(char host_id_out[128]);
int dg_comm_create(const char host_id[128], int rank, int nranks, dg_comm** out);
int dg_comm_split(dg_comm* parent, int color, int key, dg_comm** out);
int dg_comm_destroy(dg_comm* comm);
int dg_comm_rank(const dg_comm* comm, int* rank, int* nranks);
/* in-place sum over the communicator, enqueued on `stream` (dW of gcn.py:52; the partial z of dist_15d.py:104) */
int dg_comm_allreduce_sum(dg_comm* comm, float* buf, int64_t count, void* stream);
int dg_comm_broadcast(dg_comm* comm, float* buf, int64_t count, int root, void* stream);

typedef struct dg_stage_times {   /* device times of the last timed stage loop on a communicator, milliseconds */
    float comm_ms;                /* sum over stages of broadcast durations on the side stream */
    float spmm_ms;                /* sum over stages of local-product durations on the compute stream */
    float total_ms;               /* first enqueue to last completion */
    int32_t stages;
} dg_stage_times;

/* ---- the stage loop: z = sum_s A[.,part_s] * X_{root_s} --------------------------------------------------------------
 * Replaces models/gcn.py:16-30.  For stage s the block of rank roots[s] (of `comm`) is broadcast on the
 * communicator's side stream into recv[s % nbuf] (the root sends `x_local` in place) while the compute stream
 * multiplies the block of stage s-1; events chain the two streams, nothing blocks the host.
 *   group               stages fused into one product (>= 1).  With group = 1 this is the reference's loop stage for
 *                       stage.  With group = k the broadcasts of k consecutive stages are issued as one NCCL group
 *                       and land side by side in one receive buffer (k*n rows), and ONE product multiplies the joined
 *                       n x (k*n) sparse block: fewer read-modify-write passes over z and longer rows per product,
 *                       the same ascending (stage, column) summation order inside every row
 *   plans[g], vals[g]   plan and values of the sparse block of product g = stages [g*group, (g+1)*group): n x (k_g*n)
 *   x_local             this rank's n x F block (sent in place; with group = 1 also read in place, never copied)
 *   recv[0..nbuf)       nbuf >= 2 device buffers of group*n*F floats owned by the caller
 *   z                   n x F result on the compute stream; overwritten (the first product runs with beta = 0)
 *   timed != 0          record per-product events; read them with dg_comm_last_times after synchronising
 * With a NULL comm or a single rank the loop degenerates to local products and no collective (group must be 1). */
int dg_bcast_spmm_1d(dg_comm* comm, int32_t n_stages, const int32_t* host_roots, int32_t group,
                     const dg_plan* const* host_plans, const float* const* host_vals,
                     const float* x_local, int32_t n, int32_t F, float* const* host_recv, int32_t nbuf,
                     float* z, int timed, void* compute_stream);
/* 1.5D (dist_15d.py:61-106): the same loop inside the column communicator, then the sum of the partial z over
 * the row communicator (replication group). */
int dg_bcast_spmm_15d(dg_comm* col_comm, dg_comm* row_comm, int32_t n_stages, const int32_t* host_roots, int32_t group,
                      const dg_plan* const* host_plans, const float* const* host_vals,
                      const float* x_local, int32_t n, int32_t F, float* const* host_recv, int32_t nbuf,
                      float* z, int timed, void* compute_stream);
/* The same distributed product with a receive area for every remote block and the products in the caller's order
 * (replaces gcn.py:16-30 / dist_15d.py:61-106 like the two functions above).  All n_stages broadcasts are queued back to
 * back on the side stream in the order of host_roots - the same on every rank - and never wait for a buffer; the
 * products run on the compute stream in the order listed, each as soon as broadcast host_last_stage[p] (an index into
 * host_roots, -1 = needs no transfer) has landed.  Listing this rank's own block first starts the arithmetic while the
 * first transfer is still in flight; the price is (n_stages - 1) * n * F floats of receive area and a per-rank sum
 * order (own block first) that differs from the reference's ascending order by rounding only.
 *   bcast_group         consecutive broadcasts issued as one NCCL group (>= 1; the same value on every rank)
 *   host_landing[s]     where the block of stage s lands on this rank (n*F floats); NULL at a stage this rank roots
 *                       means "send from x_local, keep no second copy"
 *   host_plans/vals[p]  sparse block of product p: n x (rows of its operand); host_operands[p] its dense operand:
 *                       x_local, or a pointer into the landing area where the blocks it covers lie side by side
 *   host_last_stage     non-decreasing over the products that need transfers, and its maximum is n_stages - 1
 *   row_comm            NULL, or the 1.5D replication group over which the finished z is summed */
int dg_bcast_spmm_ordered(dg_comm* comm, dg_comm* row_comm, int32_t n_stages, const int32_t* host_roots,
                          int32_t bcast_group, float* const* host_landing, int32_t n_products, const dg_plan* const* host_plans,
                          const float* const* host_vals, const float* const* host_operands,
                          const int32_t* host_last_stage, const float* x_local, int32_t n, int32_t F, float* z,
                          int timed, void* compute_stream);
/* ---- the same distributed product with the remote blocks pulled by the copy engines (no counterpart in the reference;
 * replaces gcn.py:16-30 / dist_15d.py:61-106 like dg_bcast_spmm_ordered) ---------------------------------------------
 * Set-up, once per communicator and buffer size (collective in the sense that every rank must do it):
 *   dg_comm_peer_alloc   allocates this rank's two send buffers of `floats` floats each and writes their two 64-byte
 *                        CUDA IPC handles to host_handles_out (128 bytes);
 *   (the host exchanges the handles, e.g. with an all-gather of bytes)
 *   dg_comm_peer_open    maps every rank's buffers; host_handles_all holds nranks x 128 bytes in communicator rank order;
 *   dg_comm_peer_close   unmaps them again (before the owners free theirs: close on all ranks, meet, then destroy).
 * dg_peer_spmm has the arguments of dg_bcast_spmm_ordered without bcast_group.  It copies x_local into this rank's send
 * buffer, meets the other ranks in a one-float all-reduce on the side stream, and then issues one device-to-device
 * copy per remote stage - from the root's send buffer into host_landing[s] - in the order of host_roots; a stage this
 * rank roots is read from x_local (host_landing[s] == NULL) or copied locally.  Different ranks may list different
 * stages in different orders (each typically starts with the rank after itself, so that no buffer serves two readers at
 * once); the only call every rank of the communicator must make is dg_peer_spmm itself, once per distributed product.
 * DG_ERR_STATE before the set-up, DG_ERR_SCRATCH when n * F exceeds the send buffers. */
int dg_comm_peer_alloc(dg_comm* comm, int64_t floats, char host_handles_out[128]);
int dg_comm_peer_open(dg_comm* comm, const char* host_handles_all);
int dg_comm_peer_close(dg_comm* comm);
int64_t dg_comm_peer_capacity(const dg_comm* comm);
int dg_peer_spmm(dg_comm* comm, dg_comm* row_comm, int32_t n_stages, const int32_t* host_roots, float* const* host_landing,
                 int32_t n_products, const dg_plan* const* host_plans, const float* const* host_vals,
                 const float* const* host_operands, const int32_t* host_last_stage, const float* x_local, int32_t n,
                 int32_t F, float* z, int timed, void* compute_stream);
/* dg_peer_spmm moving only the rows that are needed.  A sparse block A[r, s] touches a subset of the rows of X_s (on
 * skewed graphs less than half at 8 ranks); the owner s packs, for every reader r, exactly those rows into its send
 * buffer (host_pack_rows[q]: device list of row ids of x_local, ascending; list q starts at row host_pack_offsets[q] of
 * the send buffer) and reader r pulls host_stage_rows[s] rows starting at row host_stage_offsets[s] of the root's send
 * buffer.  The reader's plan for that block must use the packed numbering (column id = position in its list), so the
 * arithmetic per output row, and its order, are those of the unpacked product.  The lists are fixed per graph: the
 * readers compute them once and hand them to the owners.  Own stages (host_roots[s] == rank) are read from x_local. */
int dg_peer_spmm_packed(dg_comm* comm, dg_comm* row_comm, int32_t n_packs, const int32_t* const* host_pack_rows,
                        const int64_t* host_pack_counts, const int64_t* host_pack_offsets, int32_t n_stages,
                        const int32_t* host_roots, const int64_t* host_stage_offsets, const int64_t* host_stage_rows,
                        float* const* host_landing, int32_t n_products, const dg_plan* const* host_plans,
                        const float* const* host_vals, const float* const* host_operands, const int32_t* host_last_stage,
                        const float* x_local, int32_t n, int32_t F, float* z, int timed, void* compute_stream);
/* The same loop with the gather done by the READER: every rank publishes its whole block (as dg_peer_spmm does: send
 * buffers of n * F floats) and packs nothing; for stage s the reader launches a small pull kernel on the side stream
 * that copies the host_stage_rows[s] rows listed in host_stage_lists[s] (device row ids of the root's block, ascending)
 * out of the root's send buffer into host_landing[s], with plain loads over NVLink (no multicast, no waiting on the
 * peer: the meeting point before it made the block complete).  Plans of remote blocks use the packed numbering, as
 * above; nothing has to be exchanged between the ranks beforehand.  F must be a multiple of 4. */
int dg_peer_spmm_gather(dg_comm* comm, dg_comm* row_comm, int32_t n_stages, const int32_t* host_roots,
                        const int32_t* const* host_stage_lists, const int64_t* host_stage_rows, float* const* host_landing,
                        int32_t n_products, const dg_plan* const* host_plans, const float* const* host_vals,
                        const float* const* host_operands, const int32_t* host_last_stage, const float* x_local, int32_t n,
                        int32_t F, float* z, int timed, void* compute_stream);
/* 1D only: the same distributed product pipelined along the feature dimension (replaces gcn.py:16-30 as a whole).  The
 * n x F operand is cut into n_chunks column chunks (host_chunk_widths, summing to F).  Chunk c of every rank is
 * all-gathered on the side stream into host_area[c % 2] ((nranks*n) x w_c, rank r's rows at r*n) while the compute
 * stream multiplies chunk c-1 by `plan`, the rank's whole n x (nranks*n) row block, writing columns of z directly
 * (leading dimension F, beta = 0: z is written once).  Rows keep their full length, so the product runs as on one
 * GPU, and the sum inside a row is over ascending (source rank, column) as in the reference's stage loop.
 *   host_pack[0..2)   two buffers of n * max(w_c) floats for the packed chunk to send (unused when n_chunks == 1)
 *   host_area[0..2)   two buffers of nranks * n * max(w_c) floats */
int dg_allgather_spmm(dg_comm* comm, const dg_plan* plan, const float* val, const float* x_local, int32_t n, int32_t F,
                      int32_t n_chunks, const int32_t* host_chunk_widths, float* const* host_pack,
                      float* const* host_area, float* z, int timed, void* compute_stream);
int dg_comm_last_times(dg_comm* comm, dg_stage_times* host_out);

/* ---- dense transform on the tensor cores ----------------------------------------------------------------------------
 * C[M x N] = act(A[M x K] * Bt[N x K]^T), fp32 in and out, replacing torch.mm at models/gcn.py:41 (Bt = W^T) and :49
 * (Bt = W).  Three tcgen05 TF32 passes on head/tail splits with an fp32 accumulator in tensor memory give fp32-level
 * accuracy (about 5e-7 relative).  Bt is passed already split (dg_dense_split: head keeps sign, exponent and 10 mantissa
 * bits, tail = x - head); A is split inside the kernel.  Limits (dg_dense_supported returns 0 otherwise, and
 * dg_dense_nt DG_ERR_UNSUPPORTED): M < 2^31, lda and ldb multiples of 4 floats, A / Bt 16-byte aligned.  A result wider
 * than 256 columns is computed in panels of 256 (A is streamed once per panel).
 * relu != 0 applies max(x, 0) on the way out.  dg_dense_status reads the device status word (synchronises `stream`):
 * non-zero if a kernel gave up on one of its bounded waits since the last dg_dense_status_reset (its output is then
 * invalid; nothing hangs).  dg_dense_wait_selftest runs the give-up path on purpose, safely: one CTA allocates tensor
 * memory, waits a few thousand polls on a barrier nothing arrives at, reports that the wait ran out (*host_gave_up = 1),
 * frees its tensor memory and returns; the status word of the real kernels is not touched. */
int dg_dense_split(const float* src, float* head, float* tail, int64_t count, void* stream);
int dg_dense_supported(int64_t M, int32_t N, int32_t K, int64_t lda, int64_t ldb, const void* A, const void* Bt_head, const void* Bt_tail);
int dg_dense_nt(const float* A, int64_t lda, const float* Bt_head, const float* Bt_tail, int64_t ldb, float* C, int64_t ldc,
                int64_t M, int32_t N, int32_t K, int32_t relu, void* stream);
/* The same product with the derivative of a ReLU applied on the way out: element (i, j) is zeroed where
 * mask[i * ldm + j] <= 0 (mask = the activation the gradient flows back through; the `grad * (h > 0)` that autograd runs
 * as a separate pass after torch.mm at models/gcn.py:49).  mask == NULL is dg_dense_nt. */
int dg_dense_nt_masked(const float* A, int64_t lda, const float* Bt_head, const float* Bt_tail, int64_t ldb, float* C,
                       int64_t ldc, int64_t M, int32_t N, int32_t K, int32_t relu, const float* mask, int64_t ldm,
                       void* stream);
/* Weight-gradient product D[Km x Nn] = X[n x Km]^T * G[n x Nn] (torch.mm at models/gcn.py:50), same arithmetic (three
 * TF32 passes, fp32 accumulator in tensor memory) with BOTH operands split inside the kernel.  The n rows are shared
 * out over at most max_ctas CTAs.  The tensor cores truncate when they add into their accumulator, an error that grows
 * with the number of rows, so every 256 rows a CTA adds its
 * accumulators, rounded to nearest, into its partial result in `scratch` and restarts them; a second kernel adds the
 * partials in CTA order, so the result is bit-reproducible and within about 6e-6 of the exact product for any n.
 * `scratch` is 16-byte aligned and holds ctas * roundup(min(Km, 256), 128) * roundup(min(Nn, 256), 16) floats
 * (DG_ERR_SCRATCH otherwise).  Wider results are computed as 256 x 256 panels of D, one after the other.
 * Limits: n < 2^31, ldx and ldg multiples of 4 floats, X / G 16-byte aligned. */
int dg_dense_tn_supported(int64_t n, int32_t Km, int32_t Nn, int64_t ldx, int64_t ldg, const void* X, const void* G);
int dg_dense_tn(const float* X, int64_t ldx, const float* G, int64_t ldg, float* D, int64_t ldd, int64_t n, int32_t Km,
                int32_t Nn, float* scratch, int64_t scratch_floats, int32_t max_ctas, void* stream);
int dg_dense_status(int* host_status, void* stream);
int dg_dense_status_reset(void* stream);
int dg_dense_wait_selftest(int* host_gave_up, void* stream);

/* ---- instrumentation (no counterpart in the reference, whose timer synchronises the device around every call,
 * light_dist_gnn/dist_utils/timer.py:16-24) ------------------------------------------------------------------------
 * Between dg_profile_begin and dg_profile_end every local product is bracketed by a CUDA event pair on the stream it
 * is launched on.  dg_profile_end synchronises the device and reports the summed device time of the products, their
 * algorithmic traffic  8*nnz + 4*(m+1) + 4*F*touched_columns + 4*F*m*(1 + [beta != 0])  in bytes, the no-reuse gather
 * volume  8*nnz + 4*(m+1) + 4*F*nnz + 4*F*m*(1 + [beta != 0]),  2*nnz*F flops, and how many kernels of this library
 * were launched (products only; NCCL's own kernels are not counted). */
typedef struct dg_profile {
    double spmm_ms;
    double alg_bytes;
    double gather_bytes;
    double flops;
    int64_t products;
    int64_t kernel_launches;
} dg_profile;
int dg_profile_begin(void);
int dg_profile_end(dg_profile* host_out);

#ifdef __cplusplus
}
#endif
#endif /* DIST_GNN_B200_H */
