// Plan construction: row-sorted COO -> CSR row offsets, index validation, heavy-row chunk table, column census.
//
// Replaces the per-call descriptor set-up of the reference's cuSPARSE wrapper (light_dist_gnn/spmm_cpp/spmm.cpp:19-24)
// and the coo2csr conversion of its CUDA-10 variant (spmm_original.cpp:140-146) by a one-off device pass.
#include <algorithm>
#include <new>
#include <vector>
#include "dg_internal.h"

namespace {

struct HeavyTriple {
    int64_t e0, e1;
    int32_t row, pad;
};

// Thread e in [0, nnz]: checks entry e and fills rowptr for the rows that start between entry e-1 and entry e.
__global__ void k_validate_rowptr(const int32_t* __restrict__ row, const int32_t* __restrict__ col, int64_t nnz,
                                  int32_t m, int32_t k, int64_t* __restrict__ rowptr, int* __restrict__ bad)
{
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e > nnz) return;
    const int32_t prev = e > 0 ? row[e - 1] : -1;
    const int32_t cur = e < nnz ? row[e] : m;
    bool ok = prev >= -1 && prev < m && cur >= 0 && cur <= m && prev <= cur;
    if (e < nnz) {
        const int32_t c = col[e];
        ok = ok && cur < m && c >= 0 && c < k;
    }
    if (!ok) {
        atomicExch(bad, 1);
        return;
    }
    for (int32_t r = prev + 1; r <= cur; ++r) rowptr[r] = e;
}

__global__ void k_row_census(const int64_t* __restrict__ rowptr, int32_t m, int32_t threshold,
                             HeavyTriple* __restrict__ heavy, int32_t capacity, int32_t* __restrict__ n_heavy,
                             unsigned long long* __restrict__ max_deg, unsigned long long* __restrict__ heavy_nnz)
{
    const int32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    unsigned long long deg = 0;
    if (i < m) {
        const int64_t e0 = rowptr[i], e1 = rowptr[i + 1];
        deg = (unsigned long long)(e1 - e0);
        if ((int64_t)deg > threshold) {
            const int32_t slot = atomicAdd(n_heavy, 1);
            if (slot < capacity) heavy[slot] = HeavyTriple{e0, e1, i, 0};
            atomicAdd(heavy_nnz, deg);
        }
    }
    // warp max before the atomic keeps contention low
    for (int off = 16; off > 0; off >>= 1) {
        const unsigned long long o = __shfl_xor_sync(0xffffffffu, deg, off);
        deg = o > deg ? o : deg;
    }
    if ((threadIdx.x & 31) == 0 && deg > 0) atomicMax(max_deg, deg);
}

__global__ void k_mark_columns(const int32_t* __restrict__ col, int64_t nnz, uint32_t* __restrict__ bitmap)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < nnz; e += stride) {
        const int32_t c = col[e];
        const uint32_t bit = 1u << (c & 31);
        if (!(bitmap[c >> 5] & bit)) atomicOr(&bitmap[c >> 5], bit);
    }
}

__global__ void k_count_bits(const uint32_t* __restrict__ bitmap, int64_t words, unsigned long long* __restrict__ total)
{
    unsigned long long local = 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < words; w += stride) local += __popc(bitmap[w]);
    for (int off = 16; off > 0; off >>= 1) local += __shfl_xor_sync(0xffffffffu, local, off);
    if ((threadIdx.x & 31) == 0 && local) atomicAdd(total, local);
}

// Thread t: the row that holds entry t * task_nnz, i.e. the smallest r with rowptr[r + 1] > t * task_nnz.
__global__ void k_task_first_row(const int64_t* __restrict__ rowptr, int32_t m, int64_t task_nnz, int32_t n_tasks,
                                 int32_t* __restrict__ first_row)
{
    const int32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_tasks) return;
    const int64_t e = (int64_t)t * task_nnz;
    int32_t lo = 0, hi = m;            // answer in [0, m): entry e exists, so some row ends beyond it
    while (lo < hi) {
        const int32_t mid = lo + (hi - lo) / 2;
        if (rowptr[mid + 1] > e) hi = mid; else lo = mid + 1;
    }
    first_row[t] = lo;
}

// Rows whose entries fall into more than one task.
__global__ void k_split_census(const int64_t* __restrict__ rowptr, int32_t m, int64_t task_nnz,
                               dg_split_row* __restrict__ out, int32_t capacity, int32_t* __restrict__ count)
{
    const int32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= m) return;
    const int64_t e0 = rowptr[i], e1 = rowptr[i + 1];
    if (e1 <= e0) return;
    const int64_t t0 = e0 / task_nnz, t1 = (e1 - 1) / task_nnz;
    if (t0 == t1) return;
    const int32_t slot = atomicAdd(count, 1);
    if (slot < capacity) out[slot] = dg_split_row{i, (int32_t)t0, (int32_t)t1, 0};
}

// First column of every chunk (the entries of a row are in ascending column order, so this is where its window starts).
__global__ void k_chunk_first_column(const dg_chunk* __restrict__ chunks, int32_t n_chunks, const int32_t* __restrict__ col,
                                     int32_t* __restrict__ first)
{
    const int32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < n_chunks) first[c] = col[chunks[c].e0];
}

struct DeviceTemp {   // frees its allocations on scope exit
    std::vector<void*> ptrs;
    ~DeviceTemp() { for (void* p : ptrs) cudaFree(p); }
    template <class T> cudaError_t alloc(T** out, size_t count) {
        cudaError_t e = cudaMalloc((void**)out, std::max<size_t>(count, 1) * sizeof(T));
        if (e == cudaSuccess) ptrs.push_back(*out);
        return e;
    }
};

int build_tasks(dg_plan* p, int32_t task_nnz, cudaStream_t stream)
{
    cudaFree(p->task_first_row);
    cudaFree(p->split);
    p->task_first_row = nullptr;
    p->split = nullptr;
    p->task_nnz = task_nnz;
    p->n_tasks = (int32_t)((p->nnz + task_nnz - 1) / task_nnz);
    p->n_split = 0;
    if (p->n_tasks == 0) return DG_OK;
    const int T = 256;
    DG_CUDA(cudaMalloc((void**)&p->task_first_row, (size_t)p->n_tasks * sizeof(int32_t)));
    k_task_first_row<<<(p->n_tasks + T - 1) / T, T, 0, stream>>>(p->rowptr, p->m, task_nnz, p->n_tasks, p->task_first_row);
    DeviceTemp tmp;
    dg_split_row* d_rows = nullptr;
    int32_t* d_count = nullptr;
    const int32_t capacity = p->n_tasks;      // a row can only be cut at one of the n_tasks - 1 task boundaries
    DG_CUDA(tmp.alloc(&d_rows, (size_t)capacity));
    DG_CUDA(tmp.alloc(&d_count, 1));
    DG_CUDA(cudaMemsetAsync(d_count, 0, sizeof(int32_t), stream));
    k_split_census<<<(p->m + T - 1) / T, T, 0, stream>>>(p->rowptr, p->m, task_nnz, d_rows, capacity, d_count);
    int32_t h_count = 0;
    DG_CUDA(cudaMemcpyAsync(&h_count, d_count, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
    DG_CUDA(cudaStreamSynchronize(stream));
    DG_CUDA(cudaGetLastError());
    if (h_count > capacity) return DG_ERR_STATE;
    if (h_count > 0) {
        std::vector<dg_split_row> rows((size_t)h_count);
        DG_CUDA(cudaMemcpy(rows.data(), d_rows, rows.size() * sizeof(dg_split_row), cudaMemcpyDeviceToHost));
        std::sort(rows.begin(), rows.end(), [](const dg_split_row& a, const dg_split_row& b) { return a.row < b.row; });
        DG_CUDA(cudaMalloc((void**)&p->split, rows.size() * sizeof(dg_split_row)));
        DG_CUDA(cudaMemcpy(p->split, rows.data(), rows.size() * sizeof(dg_split_row), cudaMemcpyHostToDevice));
        p->n_split = h_count;
    }
    return DG_OK;
}

}  // namespace

extern "C" int dg_plan_set_task_size(dg_plan* p, int32_t task_nnz, void* stream)
{
    if (!p) return DG_ERR_NULL;
    if (task_nnz <= 0) task_nnz = DG_DEFAULT_TASK_NNZ;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev != p->device) return DG_ERR_STATE;
    DG_CUDA(cudaStreamSynchronize((cudaStream_t)stream));     // earlier products may still read the old tables
    return build_tasks(p, task_nnz, (cudaStream_t)stream);
}

extern "C" int dg_plan_device_status(const dg_plan* p, int* host_status, void* stream)
{
    if (!p || !host_status) return DG_ERR_NULL;
    DG_CUDA(cudaMemcpyAsync(host_status, p->status, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    DG_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return DG_OK;
}

// lean: a plan that will serve one product and be destroyed (dg_spmm_coo): the distinct-column census (statistics only)
// and the task tables of the streaming kernel are left out; touched_columns then reads k.
int dg_plan_build(const int32_t* row, const int32_t* col, int64_t nnz, int32_t m, int32_t k, int32_t heavy_threshold,
                  int32_t chunk, bool lean, void* stream_, dg_plan** out)
{
    if (!out) return DG_ERR_NULL;
    *out = nullptr;
    if (nnz < 0 || m < 0 || k < 0) return DG_ERR_DIMS;
    if (nnz > 0 && (!row || !col)) return DG_ERR_NULL;
    if (nnz > 0 && (m == 0 || k == 0)) return DG_ERR_DIMS;
    if (heavy_threshold <= 0) heavy_threshold = DG_DEFAULT_HEAVY_THRESHOLD;
    if (chunk <= 0) chunk = DG_DEFAULT_CHUNK;
    cudaStream_t stream = (cudaStream_t)stream_;

    dg_plan* p = new (std::nothrow) dg_plan();
    if (!p) return (int)cudaErrorMemoryAllocation;
    *p = dg_plan{};
    p->m = m; p->k = k; p->nnz = nnz; p->col = col;
    p->heavy_threshold = heavy_threshold; p->chunk = chunk;
    int rc = DG_OK;
    auto fail = [&](int code) { dg_plan_destroy(p); return code; };
    if ((rc = (int)cudaGetDevice(&p->device)) != 0) return fail(rc);
    if ((rc = (int)cudaMalloc((void**)&p->rowptr, ((size_t)m + 1) * sizeof(int64_t))) != 0) return fail(rc);

    DeviceTemp tmp;
    int* d_bad = nullptr;
    int32_t* d_nheavy = nullptr;
    unsigned long long* d_counters = nullptr;     // [0] max degree, [1] heavy nnz, [2] touched columns
    HeavyTriple* d_heavy = nullptr;
    uint32_t* d_bitmap = nullptr;
    const int32_t capacity = (int32_t)std::min<int64_t>(nnz / heavy_threshold + 1, m);
    const int64_t words = ((int64_t)k + 31) / 32;
    if ((rc = (int)tmp.alloc(&d_bad, 1)) || (rc = (int)tmp.alloc(&d_nheavy, 1)) || (rc = (int)tmp.alloc(&d_counters, 3)) ||
        (rc = (int)tmp.alloc(&d_heavy, (size_t)capacity)) || (rc = (int)tmp.alloc(&d_bitmap, (size_t)words)))
        return fail(rc);
    cudaMemsetAsync(d_bad, 0, sizeof(int), stream);
    cudaMemsetAsync(d_nheavy, 0, sizeof(int32_t), stream);
    cudaMemsetAsync(d_counters, 0, 3 * sizeof(unsigned long long), stream);
    cudaMemsetAsync(d_bitmap, 0, (size_t)std::max<int64_t>(words, 1) * sizeof(uint32_t), stream);

    const int T = 256;
    k_validate_rowptr<<<(unsigned)((nnz + 1 + T - 1) / T), T, 0, stream>>>(row, col, nnz, m, k, p->rowptr, d_bad);
    int h_bad = 0;
    if ((rc = (int)cudaMemcpyAsync(&h_bad, d_bad, sizeof(int), cudaMemcpyDeviceToHost, stream)) ||
        (rc = (int)cudaStreamSynchronize(stream)))
        return fail(rc);
    if (h_bad) return fail(DG_ERR_INDEX);

    if (m > 0) k_row_census<<<(m + T - 1) / T, T, 0, stream>>>(p->rowptr, m, heavy_threshold, d_heavy, capacity, d_nheavy,
                                                             d_counters, d_counters + 1);
    if (nnz > 0 && !lean) {
        const unsigned blocks = (unsigned)std::min<int64_t>((nnz + T - 1) / T, 148 * 16);
        k_mark_columns<<<blocks, T, 0, stream>>>(col, nnz, d_bitmap);
        k_count_bits<<<(unsigned)std::min<int64_t>((words + T - 1) / T, 148 * 8), T, 0, stream>>>(d_bitmap, words, d_counters + 2);
    }
    int32_t h_nheavy = 0;
    unsigned long long h_counters[3] = {0, 0, 0};
    if ((rc = (int)cudaMemcpyAsync(&h_nheavy, d_nheavy, sizeof(int32_t), cudaMemcpyDeviceToHost, stream)) ||
        (rc = (int)cudaMemcpyAsync(h_counters, d_counters, sizeof(h_counters), cudaMemcpyDeviceToHost, stream)) ||
        (rc = (int)cudaStreamSynchronize(stream)) || (rc = (int)cudaGetLastError()))
        return fail(rc);
    p->max_row_nnz = (int64_t)h_counters[0];
    p->heavy_nnz = (int64_t)h_counters[1];
    p->touched_columns = lean ? (int64_t)k : (int64_t)h_counters[2];
    if (h_nheavy > capacity) return fail(DG_ERR_STATE);   // cannot happen: every heavy row holds > threshold entries

    if (h_nheavy > 0) {
        std::vector<HeavyTriple> rows((size_t)h_nheavy);
        if ((rc = (int)cudaMemcpy(rows.data(), d_heavy, rows.size() * sizeof(HeavyTriple), cudaMemcpyDeviceToHost))) return fail(rc);
        std::sort(rows.begin(), rows.end(), [](const HeavyTriple& a, const HeavyTriple& b) { return a.row < b.row; });
        std::vector<dg_chunk> chunks;
        std::vector<dg_heavy_row> heavy;
        for (const HeavyTriple& r : rows) {
            dg_heavy_row h{r.row, (int32_t)chunks.size(), 0, 0};
            for (int64_t e = r.e0; e < r.e1; e += chunk)
                chunks.push_back(dg_chunk{e, std::min<int64_t>(e + chunk, r.e1), r.row, (int32_t)chunks.size()});
            h.nchunks = (int32_t)chunks.size() - h.slot0;
            heavy.push_back(h);
        }
        p->n_chunks = (int32_t)chunks.size();
        p->n_heavy = (int32_t)heavy.size();
        if ((rc = (int)cudaMalloc((void**)&p->chunks, chunks.size() * sizeof(dg_chunk))) ||
            (rc = (int)cudaMalloc((void**)&p->heavy, heavy.size() * sizeof(dg_heavy_row))) ||
            (rc = (int)cudaMemcpy(p->chunks, chunks.data(), chunks.size() * sizeof(dg_chunk), cudaMemcpyHostToDevice)) ||
            (rc = (int)cudaMemcpy(p->heavy, heavy.data(), heavy.size() * sizeof(dg_heavy_row), cudaMemcpyHostToDevice)))
            return fail(rc);
        // Visiting order of the chunks.  A chunk's scratch slot is fixed above, so the list itself may be walked in any order
        // without changing a bit of the result.  Chunks are handed to warps in list order, eight per CTA, CTAs in launch
        // order; sorted by the column their window starts at, the warps that run at the same time gather from the same
        // band of B's rows instead of from all of B, which is what lets the L2 hold the band's popular rows (whole benchmark
        // graph, F = 256: 11.8 -> 9.6 ms per product; F = 100: 6.1 -> 4.9 ms).
        if (chunks.size() > 1) {
            int32_t* d_first = nullptr;
            if ((rc = (int)tmp.alloc(&d_first, chunks.size()))) return fail(rc);
            k_chunk_first_column<<<(unsigned)((chunks.size() + T - 1) / T), T, 0, stream>>>(p->chunks, p->n_chunks, col, d_first);
            std::vector<int32_t> first(chunks.size());
            if ((rc = (int)cudaMemcpyAsync(first.data(), d_first, first.size() * sizeof(int32_t), cudaMemcpyDeviceToHost, stream)) ||
                (rc = (int)cudaStreamSynchronize(stream)))
                return fail(rc);
            std::vector<int32_t> order(chunks.size());
            for (size_t i = 0; i < order.size(); ++i) order[i] = (int32_t)i;
            std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return first[a] < first[b]; });
            std::vector<dg_chunk> sorted(chunks.size());
            for (size_t i = 0; i < order.size(); ++i) sorted[i] = chunks[order[i]];
            if ((rc = (int)cudaMemcpy(p->chunks, sorted.data(), sorted.size() * sizeof(dg_chunk), cudaMemcpyHostToDevice))) return fail(rc);
        }
    }
    if ((rc = (int)cudaMalloc((void**)&p->status, sizeof(int))) || (rc = (int)cudaMemset(p->status, 0, sizeof(int)))) return fail(rc);
    if (!lean && (rc = build_tasks(p, DG_DEFAULT_TASK_NNZ, stream))) return fail(rc);
    *out = p;
    return DG_OK;
}

extern "C" int dg_plan_create_ex(const int32_t* row, const int32_t* col, int64_t nnz, int32_t m, int32_t k,
                                 int32_t heavy_threshold, int32_t chunk, void* stream, dg_plan** out)
{
    return dg_plan_build(row, col, nnz, m, k, heavy_threshold, chunk, false, stream, out);
}

extern "C" int dg_plan_create(const int32_t* row, const int32_t* col, int64_t nnz, int32_t m, int32_t k, void* stream,
                              dg_plan** out)
{
    return dg_plan_create_ex(row, col, nnz, m, k, 0, 0, stream, out);
}

extern "C" int dg_plan_destroy(dg_plan* p)
{
    if (!p) return DG_OK;
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != p->device) cudaSetDevice(p->device);
    cudaFree(p->rowptr);
    cudaFree(p->chunks);
    cudaFree(p->heavy);
    cudaFree(p->scratch);
    cudaFree(p->task_first_row);
    cudaFree(p->split);
    cudaFree(p->status);
    if (prev != p->device && prev >= 0) cudaSetDevice(prev);
    delete p;
    return DG_OK;
}

extern "C" int dg_plan_get_stats(const dg_plan* p, dg_plan_stats* o)
{
    if (!p || !o) return DG_ERR_NULL;
    o->nnz = p->nnz; o->m = p->m; o->k = p->k;
    o->heavy_threshold = p->heavy_threshold; o->chunk = p->chunk;
    o->heavy_rows = p->n_heavy; o->heavy_chunks = p->n_chunks;
    o->heavy_nnz = p->heavy_nnz; o->max_row_nnz = p->max_row_nnz; o->touched_columns = p->touched_columns;
    return DG_OK;
}

extern "C" int dg_plan_copy_rowptr(const dg_plan* p, int64_t* host_rowptr, void* stream)
{
    if (!p || !host_rowptr) return DG_ERR_NULL;
    DG_CUDA(cudaMemcpyAsync(host_rowptr, p->rowptr, ((size_t)p->m + 1) * sizeof(int64_t), cudaMemcpyDeviceToHost,
                            (cudaStream_t)stream));
    DG_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return DG_OK;
}
