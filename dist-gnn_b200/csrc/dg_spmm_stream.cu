// Streaming SpMM for sm_100a: the gathered rows of B are staged through shared memory with asynchronous copies.
//
// Same product as the row kernels of dg_spmm.cu (C = epilogue(alpha * A * B + beta * C), replacing
// cusparseSpMM at light_dist_gnn/spmm_cpp/spmm.cpp:26-28), for operands whose rows are 16-byte aligned and at
// least 256 bytes wide.  What changes is how the memory system is driven:
//   * the entry list of the block is cut into tasks of task_nnz entries regardless of row boundaries (perfect load
//     balance, no separate heavy-row pass); one warp owns one task;
//   * the warp copies the needed piece of row col[e] of B (up to 1 KB) straight from global to its ring of S stages
//     in shared memory with 16-byte cp.async (L1 bypassed), one commit group per stage.  No register waits for data
//     in flight, so a warp keeps tens of KB outstanding instead of ~4 KB - the row kernels were bound by memory
//     latency, not by DRAM or L2 bandwidth;
//   * it then reads each staged row back with conflict-free 128-bit shared loads and accumulates in entry order (the
//     order of the CPU oracle inside a row).
// Rows cut by a task boundary leave raw partial sums in two carry rows per task; k_stream_fixup adds them in task
// order and applies the epilogue, so results stay bit-reproducible (no float atomics).
// Status: opt-in (dg_select_kernel(2) or DG_SPMM_KERNEL=stream).  Measured on B200, R-MAT 1 M nodes, degree 48, F = 256:
// row kernels 5.86 ms, this kernel 6.83 ms at its best setting (2 stages x 4 rows, 24+ warps per SM); at degree 6 it is
// 7 % faster (3.33 vs 3.57 ms).  A first version issued one cp.async.bulk per gathered row with mbarrier completion:
// the bulk-copy engine sustained only about one row-sized copy per 100 cycles per SM (19.3 ms), so it is not used for
// gathers.  A plain random 1 KB-row gather reaches 7.3 TB/s from HBM and 18.8 TB/s from L2 on this GPU; at the 54 % L2 hit
// rate of these graphs that bounds any gather kernel near 10.9 TB/s, and the row kernels run at 9.2 TB/s.
// Nothing in this kernel spins on a flag or barrier.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include "dg_internal.h"

namespace {

struct StreamArgs {
    const int64_t* rowptr;
    const int32_t* col;
    const float* val;
    const float* B;
    float* C;
    const float* row_scale;
    const float* bias;
    const int32_t* task_first_row;
    const dg_split_row* split;
    float* carry;                           // 2 * n_tasks rows of F floats
    int64_t ldb, ldc, nnz;
    int32_t m, F, n_tasks, task_nnz;
    int32_t tile_floats;                    // floats of a B row handled by one column chunk (multiple of 4, <= 256)
    int32_t rps;                            // entries (rows of B) per stage
    int32_t warp_bytes;                     // shared memory per warp
    float alpha, beta;
    uint32_t flags;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ float epilogue(const StreamArgs& a, float sum, float cold, int32_t row, int32_t colidx)
{
    float out = a.alpha * sum;
    if (a.beta != 0.f) out = fmaf(a.beta, cold, out);
    if (a.flags & DG_EPI_ROW_SCALE) out *= __ldg(a.row_scale + row);
    if (a.flags & DG_EPI_BIAS) out += __ldg(a.bias + colidx);
    if (a.flags & DG_EPI_RELU) out = fmaxf(out, 0.f);
    return out;
}

// One warp per task.  TPL = float4 per lane per staged row (1: pieces up to 512 B, 2: up to 1 KB); S = ring depth.
template <int TPL, int S>
__global__ void __launch_bounds__(256) k_spmm_stream(const StreamArgs a)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= a.n_tasks) return;                         // no CTA-wide barrier below: a whole warp may leave
    const int chunk0 = blockIdx.y * a.tile_floats;      // first column of this column chunk
    const int piece = min(a.tile_floats, a.F - chunk0); // floats of each row this chunk handles (multiple of 4)
    const int tile_bytes = a.tile_floats * 4;
    const int rps = a.rps;
    unsigned char* base = smem_raw + (size_t)warp * a.warp_bytes;
    const uint32_t rows_s = smem_u32(base);
    float* vals = reinterpret_cast<float*>(base + (size_t)S * rps * tile_bytes);

    const int64_t E0 = (int64_t)t * a.task_nnz;
    const int64_t E1 = min(E0 + (int64_t)a.task_nnz, a.nnz);
    const int nb = (int)((E1 - E0 + rps - 1) / rps);    // batches (= stage fills) of this task
    const bool act0 = lane * 4 < piece;
    const bool act1 = TPL == 2 && 128 + lane * 4 < piece;
    const float* b_lane = a.B + chunk0 + lane * 4;

    // (col, val) of the entries, 32 at a time: group g covers E0 + 32 g .. + 31, one entry per lane
    int32_t c_cur = 0, c_nxt = 0;
    float v_cur = 0.f, v_nxt = 0.f;
    auto load_group = [&](int64_t g, int32_t& c, float& v) {
        const int64_t e = E0 + 32 * g + lane;
        if (e < E1) { c = __ldcs(a.col + e); v = __ldcs(a.val + e); }
    };
    load_group(0, c_cur, v_cur);
    load_group(1, c_nxt, v_nxt);

    auto issue = [&](int b) {                           // fill stage b % S with batch b; always exactly one commit group
        if (b < nb) {
            const int s = b % S;
            const int64_t eb = E0 + (int64_t)b * rps;
            const int cnt = (int)min((int64_t)rps, E1 - eb);
            const int off = (b * rps) & 31;             // position of the batch inside its 32-entry group
            const int j = lane - off;
            if (j >= 0 && j < cnt) vals[s * rps + j] = v_cur;
            uint32_t dst = rows_s + (uint32_t)(s * rps * tile_bytes) + lane * 16;
            for (int k = 0; k < cnt; ++k, dst += tile_bytes) {
                const int32_t c = __shfl_sync(0xffffffffu, c_cur, off + k);
                const float* src = b_lane + (size_t)c * (size_t)a.ldb;
                if (act0) cp_async16(dst, src);
                if (TPL == 2 && act1) cp_async16(dst + 512u, src + 128);
            }
            if (off + rps >= 32) {                      // that was the last batch of the group: rotate, prefetch one more
                c_cur = c_nxt; v_cur = v_nxt;
                load_group((int64_t)(b * rps) / 32 + 2, c_nxt, v_nxt);
            }
        }
        cp_async_commit();
    };

    // row bookkeeping: row r is being accumulated; its entries end at row_end; the ends of the next rows come from
    // two lane-distributed windows of 32 row offsets each
    int32_t r = __ldg(a.task_first_row + t);
    int32_t win = r;                                    // re_cur[lane] = rowptr[win + 1 + lane]
    auto load_ends = [&](int32_t first) -> int64_t {
        const int64_t i = (int64_t)first + 1 + lane;
        return i <= a.m ? __ldg(a.rowptr + i) : INT64_MAX;
    };
    int64_t re_cur = load_ends(win), re_nxt = load_ends(win + 32);
    bool began_before = __ldg(a.rowptr + r) < E0;       // the first row may have started in an earlier task

    for (int b = 0; b < S; ++b) issue(b);               // prologue: S stages in flight

    int64_t row_end = __shfl_sync(0xffffffffu, re_cur, 0);
    float4 acc0 = make_float4(0.f, 0.f, 0.f, 0.f), acc1 = make_float4(0.f, 0.f, 0.f, 0.f);

    auto store_row = [&](float* dst, int32_t row, bool raw) {   // dst points at column chunk0 of the target row
        if (act0) {
            float4 o = acc0;
            if (!raw) {
                float4 old = make_float4(0.f, 0.f, 0.f, 0.f);
                if (a.beta != 0.f) old = *reinterpret_cast<const float4*>(dst + lane * 4);
                const int c = chunk0 + lane * 4;
                o = make_float4(epilogue(a, acc0.x, old.x, row, c), epilogue(a, acc0.y, old.y, row, c + 1),
                                epilogue(a, acc0.z, old.z, row, c + 2), epilogue(a, acc0.w, old.w, row, c + 3));
            }
            *reinterpret_cast<float4*>(dst + lane * 4) = o;
        }
        if (TPL == 2 && act1) {
            float4 o = acc1;
            if (!raw) {
                float4 old = make_float4(0.f, 0.f, 0.f, 0.f);
                if (a.beta != 0.f) old = *reinterpret_cast<const float4*>(dst + 128 + lane * 4);
                const int c = chunk0 + 128 + lane * 4;
                o = make_float4(epilogue(a, acc1.x, old.x, row, c), epilogue(a, acc1.y, old.y, row, c + 1),
                                epilogue(a, acc1.z, old.z, row, c + 2), epilogue(a, acc1.w, old.w, row, c + 3));
            }
            *reinterpret_cast<float4*>(dst + 128 + lane * 4) = o;
        }
        acc0 = make_float4(0.f, 0.f, 0.f, 0.f);
        acc1 = make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto finish_row = [&]() {                           // row r ends here: write it (or its carry) and move to row r + 1
        if (began_before) store_row(a.carry + (size_t)(2 * (int64_t)t) * a.F + chunk0, r, true);
        else store_row(a.C + (size_t)r * (size_t)a.ldc + chunk0, r, false);
        began_before = false;
        ++r;
        if (r - win == 32) { win += 32; re_cur = re_nxt; re_nxt = load_ends(win + 32); }
        row_end = __shfl_sync(0xffffffffu, re_cur, r - win);
    };

    if (t == 0)                                         // rows before the first entry are empty: they still get beta * C
        for (int32_t rr = 0; rr < r; ++rr) store_row(a.C + (size_t)rr * (size_t)a.ldc + chunk0, rr, false);

    for (int b = 0; b < nb; ++b) {
        cp_async_wait<S - 1>();                         // this lane's copies of batch b have landed ...
        __syncwarp();                                   // ... and so have the other lanes'
        const int s = b % S;
        const int64_t eb = E0 + (int64_t)b * rps;
        const int cnt = (int)min((int64_t)rps, E1 - eb);
        const unsigned char* stage_rows = base + (size_t)s * rps * tile_bytes + lane * 16;
        const float* stage_vals = vals + s * rps;
        for (int k = 0; k < cnt; ++k) {
            const int64_t e = eb + k;
            while (e == row_end && r < a.m) finish_row();
            const float v = stage_vals[k];
            if (act0) {
                const float4 x = *reinterpret_cast<const float4*>(stage_rows + (size_t)k * tile_bytes);
                acc0.x = fmaf(v, x.x, acc0.x); acc0.y = fmaf(v, x.y, acc0.y);
                acc0.z = fmaf(v, x.z, acc0.z); acc0.w = fmaf(v, x.w, acc0.w);
            }
            if (TPL == 2 && act1) {
                const float4 x = *reinterpret_cast<const float4*>(stage_rows + (size_t)k * tile_bytes + 512);
                acc1.x = fmaf(v, x.x, acc1.x); acc1.y = fmaf(v, x.y, acc1.y);
                acc1.z = fmaf(v, x.z, acc1.z); acc1.w = fmaf(v, x.w, acc1.w);
            }
        }
        __syncwarp();                                   // every lane is done reading the stage before it is refilled
        issue(b + S);
    }
    cp_async_wait<0>();
    // end of the task: rows that end exactly here (and empty rows behind them), then the open row if it has entries here
    while (E1 == row_end && r < a.m) finish_row();
    if (r < a.m && (began_before || __ldg(a.rowptr + r) < E1))
        store_row(a.carry + (size_t)(2 * (int64_t)t + (began_before ? 0 : 1)) * a.F + chunk0, r, true);
}

// One CTA per row that spans tasks: carry pieces are added in task order, then the epilogue.
__global__ void __launch_bounds__(128) k_stream_fixup(const StreamArgs a)
{
    const dg_split_row sr = a.split[blockIdx.x];
    float* crow = a.C + (size_t)sr.row * (size_t)a.ldc;
    for (int f = threadIdx.x; f < a.F; f += blockDim.x) {
        float sum = a.carry[(size_t)(2 * (int64_t)sr.t_first + 1) * a.F + f];
        for (int32_t tt = sr.t_first + 1; tt <= sr.t_last; ++tt) sum += a.carry[(size_t)(2 * (int64_t)tt) * a.F + f];
        const float old = a.beta != 0.f ? crow[f] : 0.f;
        crow[f] = epilogue(a, sum, old, sr.row, f);
    }
}

struct Tuning {
    int choice;     // 0 automatic, 1 row kernels only, 2 streaming whenever eligible
    int stages;     // ring depth: 2, 4 or 8
    int rps;        // entries per stage (0: derive from the row width)
    int warps;      // warps per CTA (0: as many as shared memory allows, at most 8)
};

Tuning& tuning()
{
    static Tuning t = [] {
        Tuning v{};
        const char* e = std::getenv("DG_SPMM_KERNEL");
        v.choice = !e ? 0 : !std::strcmp(e, "rows") ? 1 : !std::strcmp(e, "stream") ? 2 : 0;
        v.stages = 2;       // ring depth, entries per stage and warps per CTA: the measured best; 0 = derived from the row width
        v.rps = 0;
        v.warps = 0;
        return v;
    }();
    return t;
}

template <int TPL, int S>
int launch_stream(const StreamArgs& a, dim3 grid, int threads, size_t smem, cudaStream_t stream)
{
    DG_CUDA(cudaFuncSetAttribute(k_spmm_stream<TPL, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    k_spmm_stream<TPL, S><<<grid, threads, smem, stream>>>(a);
    return DG_OK;
}

}  // namespace

extern "C" int dg_select_kernel(int family)
{
    if (family < 0 || family > 2) return DG_ERR_DIMS;
    tuning().choice = family;
    return DG_OK;
}

int dg_stream_selected() { return tuning().choice == 2; }

int dg_spmm_stream_eligible(const dg_plan* plan, const float* B, int64_t ldb, const float* C, int64_t ldc, int32_t F)
{
    if (tuning().choice != 2) return 0;      // opt-in: on B200 the row kernels are at least as fast (see the header comment)
    if (plan->n_tasks == 0 || !plan->task_first_row) return 0;
    if (F % 4 || ldb % 4 || ldc % 4 || F < 64) return 0;
    if (reinterpret_cast<uintptr_t>(B) % 16 || reinterpret_cast<uintptr_t>(C) % 16) return 0;
    return 1;
}

int dg_spmm_stream_launch(const dg_plan* plan, const float* val, const float* B, int64_t ldb, float* C, int64_t ldc,
                          int32_t F, float alpha, float beta, uint32_t flags, const float* row_scale, const float* bias,
                          float* scratch, cudaStream_t stream, int* launches)
{
    const Tuning& tune = tuning();
    StreamArgs a{};
    a.rowptr = plan->rowptr; a.col = plan->col; a.val = val; a.B = B; a.C = C;
    a.row_scale = row_scale; a.bias = bias; a.task_first_row = plan->task_first_row; a.split = plan->split;
    a.carry = scratch;
    a.ldb = ldb; a.ldc = ldc; a.nnz = plan->nnz; a.m = plan->m; a.F = F; a.n_tasks = plan->n_tasks; a.task_nnz = plan->task_nnz;
    a.alpha = alpha; a.beta = beta; a.flags = flags;
    a.tile_floats = std::min(F, 256);
    const int tile_bytes = a.tile_floats * 4;
    const int S = tune.stages == 2 || tune.stages == 8 ? tune.stages : 4;
    a.rps = tune.rps > 0 ? tune.rps : (tile_bytes > 512 ? 4 : tile_bytes > 256 ? 8 : 16);
    if (a.rps > 32) a.rps = 32;
    while (32 % a.rps) --a.rps;                         // a batch must not straddle two 32-entry groups
    a.warp_bytes = ((S * a.rps * tile_bytes + S * a.rps * 4) + 127) / 128 * 128;
    int warps = std::max(1, std::min(8, (226 * 1024) / a.warp_bytes));
    if (tune.warps > 0) warps = std::min(warps, tune.warps);
    const int col_chunks = (F + a.tile_floats - 1) / a.tile_floats;
    const size_t smem = (size_t)warps * a.warp_bytes;
    dim3 grid((unsigned)((plan->n_tasks + warps - 1) / warps), (unsigned)col_chunks);
    int rc;
    if (tile_bytes > 512) rc = S == 2 ? launch_stream<2, 2>(a, grid, warps * 32, smem, stream) : S == 8 ? launch_stream<2, 8>(a, grid, warps * 32, smem, stream) : launch_stream<2, 4>(a, grid, warps * 32, smem, stream);
    else rc = S == 2 ? launch_stream<1, 2>(a, grid, warps * 32, smem, stream) : S == 8 ? launch_stream<1, 8>(a, grid, warps * 32, smem, stream) : launch_stream<1, 4>(a, grid, warps * 32, smem, stream);
    if (rc) return rc;
    *launches = 1;
    if (plan->n_split > 0) {
        k_stream_fixup<<<(unsigned)plan->n_split, 128, 0, stream>>>(a);
        *launches = 2;
    }
    return (int)cudaGetLastError();
}
