// Distributed product whose remote blocks are PULLED over NVLink by the copy engines instead of broadcast by NCCL.
//
// Replaces the same stage loop of the reference (light_dist_gnn/models/gcn.py:16-30; 1.5D: 1D_CAGNET/dist_15d.py:61-106)
// as dg_bcast_spmm_ordered, with one difference in how a block travels: every rank keeps two send buffers that its
// peers have mapped through CUDA IPC.  Per distributed product a rank copies its block into the send buffer of this
// product, all ranks meet in a one-float all-reduce on the side stream (the only collective: it orders "every block is
// in place" before "anyone reads"), and then each rank issues one device-to-device copy per remote block it needs,
// straight from the owner's send buffer into its own receive area.  The copies run on the DMA engines: they take no
// SMs from the products that run beside them, need no matching call on the owner's side, and each block's arrival
// releases the product that reads it.  Nothing in here spins on the device; all ordering is stream order, events and
// that one collective.
//
// Send buffer reuse: product k uses buffer k % 2.  Overwriting it at product k is safe once every peer has finished
// the reads of product k-2, and a peer enters the all-reduce of product k-1 only after those reads (same stream), so
// the completion of that all-reduce on this rank - which the compute stream waited for during product k-1 - is enough.
#include <nccl.h>
#include <cstdlib>
#include <cstring>
#include <vector>
#include "dg_internal.h"
#include "dg_comm.h"

namespace {

int peer_release(dg_comm* c)
{
    int first_error = DG_OK;
    for (int r = 0; r < (int)c->peer_ptr.size() / 2; ++r) {
        if (r == c->rank) continue;
        for (int b = 0; b < 2; ++b) {
            float* p = c->peer_ptr[2 * r + b];
            if (p) {
                cudaError_t e = cudaIpcCloseMemHandle(p);
                if (e != cudaSuccess && first_error == DG_OK) first_error = (int)e;
            }
        }
    }
    c->peer_ptr.clear();
    return first_error;
}

// One remote block, cut into `lanes` pieces that are copied concurrently (one copy engine does not fill the link):
// piece 0 on the side stream, the others on lane streams that start after everything queued on the side stream so far
// and that the side stream joins again afterwards, so that "arrived" on the side stream still means the whole block.
int pull_block(dg_comm* c, float* dst, const float* src, size_t count, int lanes)
{
    int rc;
    if (lanes > 1 && count >= (size_t)lanes * 65536) {
        while ((int)c->peer_lanes.size() < lanes - 1) {
            int prio_low = 0, prio_high = 0;
            cudaStream_t st;
            DG_CUDA(cudaDeviceGetStreamPriorityRange(&prio_low, &prio_high));
            DG_CUDA(cudaStreamCreateWithPriority(&st, cudaStreamNonBlocking, prio_high));
            c->peer_lanes.push_back(st);
        }
        if ((rc = make_events(c->ev_lane, (size_t)lanes, cudaEventDisableTiming))) return rc;
        const size_t piece = ((count + lanes - 1) / lanes + 63) / 64 * 64;
        DG_CUDA(cudaEventRecord(c->ev_lane[0], c->side));
        for (int l = 1; l < lanes; ++l) {
            const size_t a = (size_t)l * piece, e = a + piece < count ? a + piece : count;
            if (a >= e) break;
            cudaStream_t st = c->peer_lanes[l - 1];
            DG_CUDA(cudaStreamWaitEvent(st, c->ev_lane[0], 0));
            DG_CUDA(cudaMemcpyAsync(dst + a, src + a, (e - a) * sizeof(float), cudaMemcpyDeviceToDevice, st));
            DG_CUDA(cudaEventRecord(c->ev_lane[l], st));
        }
        DG_CUDA(cudaMemcpyAsync(dst, src, (piece < count ? piece : count) * sizeof(float), cudaMemcpyDeviceToDevice, c->side));
        for (int l = 1; l < lanes; ++l) {
            if ((size_t)l * piece >= count) break;
            DG_CUDA(cudaStreamWaitEvent(c->side, c->ev_lane[l], 0));
        }
        return DG_OK;
    }
    DG_CUDA(cudaMemcpyAsync(dst, src, count * sizeof(float), cudaMemcpyDeviceToDevice, c->side));
    return DG_OK;
}

}  // namespace

extern "C" int dg_comm_peer_alloc(dg_comm* c, int64_t floats, char host_handles_out[128])
{
    if (!c || !host_handles_out) return DG_ERR_NULL;
    if (floats <= 0) return DG_ERR_DIMS;
    if (!c->peer_ptr.empty()) return DG_ERR_STATE;                // peers still mapped: dg_comm_peer_close first
    DeviceGuard guard(c->device);
    DG_CUDA(cudaStreamSynchronize(c->side));
    for (int b = 0; b < 2; ++b) {
        if (c->peer_send[b]) DG_CUDA(cudaFree(c->peer_send[b]));
        c->peer_send[b] = nullptr;
    }
    c->peer_floats = 0;
    if (!c->peer_token) {
        DG_CUDA(cudaMalloc(&c->peer_token, sizeof(float)));
        DG_CUDA(cudaMemset(c->peer_token, 0, sizeof(float)));
        DG_CUDA(cudaEventCreateWithFlags(&c->ev_barrier, cudaEventDisableTiming));
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "a CUDA IPC memory handle is expected to be 64 bytes");
    for (int b = 0; b < 2; ++b) {
        DG_CUDA(cudaMalloc(&c->peer_send[b], (size_t)floats * sizeof(float)));
        cudaIpcMemHandle_t h;
        DG_CUDA(cudaIpcGetMemHandle(&h, c->peer_send[b]));
        memcpy(host_handles_out + 64 * b, &h, 64);
    }
    c->peer_floats = floats;
    c->peer_loops = 0;
    return DG_OK;
}

extern "C" int dg_comm_peer_open(dg_comm* c, const char* host_handles_all)
{
    if (!c || !host_handles_all) return DG_ERR_NULL;
    if (!c->peer_send[0] || !c->peer_ptr.empty()) return DG_ERR_STATE;
    DeviceGuard guard(c->device);
    c->peer_ptr.assign(2 * (size_t)c->nranks, nullptr);
    for (int r = 0; r < c->nranks; ++r) {
        for (int b = 0; b < 2; ++b) {
            if (r == c->rank) {
                c->peer_ptr[2 * r + b] = c->peer_send[b];
                continue;
            }
            cudaIpcMemHandle_t h;
            memcpy(&h, host_handles_all + 128 * (size_t)r + 64 * b, 64);
            void* p = nullptr;
            cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) {
                peer_release(c);
                return (int)e;
            }
            c->peer_ptr[2 * r + b] = static_cast<float*>(p);
        }
    }
    return DG_OK;
}

extern "C" int dg_comm_peer_close(dg_comm* c)
{
    if (!c) return DG_ERR_NULL;
    DeviceGuard guard(c->device);
    DG_CUDA(cudaStreamSynchronize(c->side));
    return peer_release(c);
}

extern "C" int64_t dg_comm_peer_capacity(const dg_comm* c)
{
    return c && !c->peer_ptr.empty() ? c->peer_floats : 0;
}

// Called by dg_comm_destroy.
int dg_comm_peer_destroy(dg_comm* c)
{
    peer_release(c);
    for (int b = 0; b < 2; ++b) {
        if (c->peer_send[b]) cudaFree(c->peer_send[b]);
        c->peer_send[b] = nullptr;
    }
    for (cudaStream_t st : c->peer_lanes) {
        cudaStreamSynchronize(st);
        cudaStreamDestroy(st);
    }
    c->peer_lanes.clear();
    for (cudaEvent_t e : c->ev_lane) cudaEventDestroy(e);
    c->ev_lane.clear();
    if (c->peer_token) {
        cudaFree(c->peer_token);
        cudaEventDestroy(c->ev_barrier);
        c->peer_token = nullptr;
    }
    return DG_OK;
}

namespace {

// dst[i, :] = x[rows[i], :] for a list of row ids (the rows of this rank's block that one peer's sparse block touches)
__global__ void k_pack_rows_v4(const float4* __restrict__ x, int64_t ldx4, const int32_t* __restrict__ rows, int64_t n_rows,
                               int32_t F4, float4* __restrict__ dst)
{
    const int64_t total = n_rows * F4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / F4;
        const int32_t c = (int32_t)(i - r * F4);
        dst[i] = __ldg(x + (int64_t)__ldg(rows + r) * ldx4 + c);
    }
}
__global__ void k_pack_rows(const float* __restrict__ x, int64_t ldx, const int32_t* __restrict__ rows, int64_t n_rows,
                            int32_t F, float* __restrict__ dst)
{
    const int64_t total = n_rows * F;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / F;
        dst[i] = __ldg(x + (int64_t)__ldg(rows + r) * ldx + (i - r * F));
    }
}

// Reader-side gather over NVLink: dst[i, :] = src[rows[i], :] where src is a PEER's block as mapped into this process.  Two
// CTAs per SM at most and four independent 16-byte loads in flight per thread (about 5 MB over the GPU, what the link's
// latency needs to stay busy), so the pull takes a quarter of the SMs' warp slots away from the products that run beside
// it and none of the owner's SMs or memory bandwidth beyond the rows actually read.  Plain loads and stores only: no
// multicast, no waiting on the peer (the meeting point before it made the block complete).
// Measured on 2 GPUs (benchmark graph, F = 256): 557 GB/s against 511 GB/s for the copy-engine pull of owner-packed rows,
// but the products beside it slow down (5.9 against 5.4 ms) and the loop takes 6.3 against 5.6 ms, so where products set the
// pace the copy engines stay the default; the gather is the option for transfer-bound loops.
__global__ void __launch_bounds__(256) k_pull_rows_v4(const float4* __restrict__ src, int64_t ld4, const int32_t* __restrict__ rows,
                                                      int64_t n_rows, int32_t F4, float4* __restrict__ dst)
{
    const int64_t total = n_rows * F4;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += 4 * stride) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int64_t i = i0 + u * stride;
            if (i < total) {
                const int64_t r = i / F4;
                v[u] = src[(int64_t)__ldg(rows + r) * ld4 + (i - r * F4)];
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int64_t i = i0 + u * stride;
            if (i < total) __stcs(dst + i, v[u]);
        }
    }
}

// Packed mode (pack_rows != nullptr): instead of the whole block, the send buffer holds for every reader the rows that
// reader's sparse block touches, one list after the other (pack_offsets in rows); stage s then pulls stage_rows[s] rows
// from row offset stage_offsets[s] of its root's send buffer.
struct PeerPacks {
    int32_t n_packs = 0;
    const int32_t* const* rows = nullptr;        // device row-id lists
    const int64_t* counts = nullptr;             // rows per list
    const int64_t* offsets = nullptr;            // first row of every list inside this rank's send buffer
    const int64_t* stage_offsets = nullptr;      // per stage: first row inside the root's send buffer
    const int64_t* stage_rows = nullptr;         // per stage: rows to pull
    // Gather mode (stage_lists != nullptr): every rank publishes its WHOLE block (as peer_copy does) and packs nothing; stage s
    // gathers the stage_rows[s] rows listed in stage_lists[s] (device row ids, ascending) out of the root's block with
    // k_pull_rows_v4 on the side stream.
    const int32_t* const* stage_lists = nullptr;
};

int peer_loop(dg_comm* comm, dg_comm* row_comm, const PeerPacks& packs, int32_t n_stages, const int32_t* roots,
              float* const* landing, int32_t n_products, const dg_plan* const* plans, const float* const* vals,
              const float* const* operands, const int32_t* last_stage, const float* x_local, int32_t n, int32_t F,
              float* z, int timed, void* compute_stream)
{
    cudaStream_t compute = (cudaStream_t)compute_stream;
    const bool gather = packs.stage_lists != nullptr;
    const bool packed = !gather && (packs.rows != nullptr || packs.stage_rows != nullptr);
    if (!comm) return DG_ERR_NULL;
    if (gather) {
        if (n_stages > 0 && !packs.stage_rows) return DG_ERR_NULL;
        if (F % 4) return DG_ERR_UNSUPPORTED;                     // rows are moved as 16-byte pieces
        for (int s = 0; s < n_stages; ++s) {
            if (packs.stage_rows[s] < 0 || packs.stage_rows[s] > n) return DG_ERR_DIMS;
            if (packs.stage_rows[s] > 0 && !packs.stage_lists[s]) return DG_ERR_NULL;
        }
    }
    if (comm->poisoned) return DG_ERR_STATE;
    if (packed) {
        if (packs.n_packs < 0 || (packs.n_packs > 0 && (!packs.rows || !packs.counts || !packs.offsets))) return DG_ERR_NULL;
        if (n_stages > 0 && (!packs.stage_offsets || !packs.stage_rows)) return DG_ERR_NULL;
        for (int q = 0; q < packs.n_packs; ++q) {
            if (packs.counts[q] < 0 || packs.offsets[q] < 0 || (packs.counts[q] > 0 && !packs.rows[q])) return DG_ERR_DIMS;
            if ((packs.offsets[q] + packs.counts[q]) * (int64_t)F > comm->peer_floats) return DG_ERR_SCRATCH;
        }
        // what this rank reads from its peers: every rank allocates send buffers of the same size (peer_floats), so a range
        // that fits this rank's buffers fits the root's; a layout that disagrees between ranks is refused here, on the
        // host, instead of sending a copy engine past the end of a peer's mapping
        for (int s = 0; s < n_stages; ++s) {
            if (packs.stage_rows[s] < 0 || packs.stage_offsets[s] < 0) return DG_ERR_DIMS;
            if ((packs.stage_offsets[s] + packs.stage_rows[s]) * (int64_t)F > comm->peer_floats) return DG_ERR_SCRATCH;
        }
    }
    if (n_stages < 0 || n_products < 0 || n < 0 || F < 0) return DG_ERR_DIMS;
    if ((n_stages > 0 && (!roots || !landing)) || (n_products > 0 && (!plans || !vals || !operands || !last_stage))) return DG_ERR_NULL;
    const size_t count = (size_t)n * (size_t)F;
    if (count && (!x_local || !z)) return DG_ERR_NULL;
    if (comm->peer_ptr.empty()) return DG_ERR_STATE;              // dg_comm_peer_alloc / _open come first
    if (!packed && (int64_t)count > comm->peer_floats) return DG_ERR_SCRATCH;          // plain and gather modes publish the whole block
    for (int s = 0; s < n_stages; ++s) {
        if (roots[s] < 0 || roots[s] >= comm->nranks) return DG_ERR_DIMS;
        if (count && roots[s] != comm->rank && !landing[s]) return DG_ERR_NULL;
    }
    int prev = -1;
    for (int p = 0; p < n_products; ++p) {                        // products consume the copies in the order they are issued
        if (!plans[p] || (count && !operands[p])) return DG_ERR_NULL;
        if (plans[p]->m != n || last_stage[p] >= n_stages || (last_stage[p] >= 0 && last_stage[p] < prev)) return DG_ERR_DIMS;
        if (last_stage[p] > prev) prev = last_stage[p];
    }
    int rc;
    DeviceGuard guard(comm->device);
    if ((rc = make_events(comm->ev_arrived, (size_t)n_products, cudaEventDisableTiming))) return rc;
    comm->timed_stages = 0;
    if (timed) {
        if ((rc = make_events(comm->t_comm, 2 * (size_t)n_products, cudaEventDefault))) return rc;
        if ((rc = make_events(comm->t_spmm, 2 * (size_t)n_products, cudaEventDefault))) return rc;
    }
    for (int p = 0; p < n_products; ++p)                          // scratch growth (it allocates) happens before anything is enqueued
        if ((rc = dg_spmm_prepare(plans[p], F, compute))) return rc;
    // From here on a failure leaves this rank out of step with its peers (a missed meeting point, a send-buffer parity that
    // differs): the guard then marks the communicator and later loops are refused.
    IssueGuard issue(comm);
    if (timed) DG_CUDA(cudaEventRecord(comm->t_begin, compute));
    if (n_products == 0 && count) DG_CUDA(cudaMemsetAsync(z, 0, count * sizeof(float), compute));
    const int b = (int)(comm->peer_loops & 1);
    // this rank's block goes where its peers can read it; everything queued so far on the compute stream comes first.
    // (Packing on the side stream instead, beside the rank's own product, was measured neutral on 2 and 4 GPUs and 3 % slower
    // on 8 - the products slow down by more than the pack no longer costs in front of them - and a warp-per-row pack kernel
    // was no faster.)
    if (packed) {
        for (int q = 0; q < packs.n_packs && count; ++q) {
            if (packs.counts[q] == 0) continue;
            float* dst = comm->peer_send[b] + packs.offsets[q] * (int64_t)F;
            const int64_t total = packs.counts[q] * (int64_t)(F % 4 == 0 ? F / 4 : F);
            const unsigned grid = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
            if (F % 4 == 0 && (reinterpret_cast<uintptr_t>(x_local) & 15) == 0)
                k_pack_rows_v4<<<grid, 256, 0, compute>>>(reinterpret_cast<const float4*>(x_local), F / 4, packs.rows[q], packs.counts[q], F / 4,
                                                          reinterpret_cast<float4*>(dst));
            else
                k_pack_rows<<<grid, 256, 0, compute>>>(x_local, F, packs.rows[q], packs.counts[q], F, dst);
        }
        DG_CUDA(cudaGetLastError());
    } else if (count) {
        DG_CUDA(cudaMemcpyAsync(comm->peer_send[b], x_local, count * sizeof(float), cudaMemcpyDeviceToDevice, compute));
    }
    DG_CUDA(cudaEventRecord(comm->ev_input, compute));
    DG_CUDA(cudaStreamWaitEvent(comm->side, comm->ev_input, 0));
    DG_NCCL(ncclAllReduce(comm->peer_token, comm->peer_token, 1, ncclFloat, ncclMax, comm->comm, comm->side));
    DG_CUDA(cudaEventRecord(comm->ev_barrier, comm->side));
    const int lanes = 2;                                          // pieces of a block in flight side by side (measured best of 1, 2, 4)
    int issued = 0;                                               // copies of stages [0, issued) are on the side stream
    for (int p = 0; p < n_products; ++p) {
        if (timed) DG_CUDA(cudaEventRecord(comm->t_comm[2 * p], comm->side));
        for (; issued <= last_stage[p]; ++issued) {
            const int s = issued;
            if (!count || roots[s] == comm->rank) {
                if (count && landing[s] && !packed && !gather)    // the caller wants its own block inside the landing area too
                    DG_CUDA(cudaMemcpyAsync(landing[s], x_local, count * sizeof(float), cudaMemcpyDeviceToDevice, comm->side));
                continue;
            }
            if (gather) {
                const int64_t rows_s = packs.stage_rows[s];
                if (rows_s > 0) {
                    int sms = 148;
                    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, comm->device);
                    const int64_t total = rows_s * (F / 4);
                    const int64_t cap = 2 * (int64_t)sms;         // CTAs per SM: 1 / 2 / 4 / 8 -> 284 / 557 / 539 / 589 GB/s at F = 256 on 2 GPUs

                    const unsigned grid = (unsigned)((total + 1023) / 1024 < cap ? (total + 1023) / 1024 : cap);
                    k_pull_rows_v4<<<grid, 256, 0, comm->side>>>(reinterpret_cast<const float4*>(comm->peer_ptr[2 * roots[s] + b]), F / 4,
                                                                 packs.stage_lists[s], rows_s, F / 4, reinterpret_cast<float4*>(landing[s]));
                    DG_CUDA(cudaGetLastError());
                }
            } else if (packed) {
                const size_t part = (size_t)packs.stage_rows[s] * (size_t)F;
                if (part && (rc = pull_block(comm, landing[s], comm->peer_ptr[2 * roots[s] + b] + packs.stage_offsets[s] * (int64_t)F, part, lanes)))
                    return rc;
            } else if ((rc = pull_block(comm, landing[s], comm->peer_ptr[2 * roots[s] + b], count, lanes))) {
                return rc;
            }
        }
        if (timed) DG_CUDA(cudaEventRecord(comm->t_comm[2 * p + 1], comm->side));
        if (last_stage[p] >= 0) {
            DG_CUDA(cudaEventRecord(comm->ev_arrived[p], comm->side));
            DG_CUDA(cudaStreamWaitEvent(compute, comm->ev_arrived[p], 0));
        }
        if (timed) DG_CUDA(cudaEventRecord(comm->t_spmm[2 * p], compute));
        rc = dg_spmm_csr(plans[p], vals[p], operands[p], F, z, F, F, 1.f, p ? 1.f : 0.f, 0u, nullptr, nullptr, compute);
        if (rc) return rc;
        if (timed) DG_CUDA(cudaEventRecord(comm->t_spmm[2 * p + 1], compute));
    }
    // later work on the compute stream (the next product's copy into the other send buffer included) is ordered after
    // this product's meeting point even on a rank that read nothing remote
    DG_CUDA(cudaStreamWaitEvent(compute, comm->ev_barrier, 0));
    if (row_comm) {
        rc = dg_comm_allreduce_sum(row_comm, z, (int64_t)n * F, compute_stream);
        if (rc) return rc;
    }
    if (timed) {
        DG_CUDA(cudaEventRecord(comm->t_end, compute));
        comm->timed_stages = n_products;
    }
    comm->peer_loops++;                                           // the loop is fully issued: the next one uses the other send buffer
    issue.done();
    return DG_OK;
}

}  // namespace

extern "C" int dg_peer_spmm(dg_comm* comm, dg_comm* row_comm, int32_t n_stages, const int32_t* roots, float* const* landing,
                            int32_t n_products, const dg_plan* const* plans, const float* const* vals,
                            const float* const* operands, const int32_t* last_stage, const float* x_local, int32_t n,
                            int32_t F, float* z, int timed, void* compute_stream)
{
    return peer_loop(comm, row_comm, PeerPacks{}, n_stages, roots, landing, n_products, plans, vals, operands, last_stage, x_local, n, F,
                     z, timed, compute_stream);
}

extern "C" int dg_peer_spmm_packed(dg_comm* comm, dg_comm* row_comm, int32_t n_packs, const int32_t* const* pack_rows,
                                   const int64_t* pack_counts, const int64_t* pack_offsets, int32_t n_stages, const int32_t* roots,
                                   const int64_t* stage_offsets, const int64_t* stage_rows, float* const* landing,
                                   int32_t n_products, const dg_plan* const* plans, const float* const* vals,
                                   const float* const* operands, const int32_t* last_stage, const float* x_local, int32_t n,
                                   int32_t F, float* z, int timed, void* compute_stream)
{
    if (!stage_offsets && n_stages > 0) return DG_ERR_NULL;
    PeerPacks packs;
    packs.n_packs = n_packs; packs.rows = pack_rows; packs.counts = pack_counts; packs.offsets = pack_offsets;
    packs.stage_offsets = stage_offsets; packs.stage_rows = stage_rows;
    static const int64_t none = 0;
    if (!packs.stage_rows) packs.stage_rows = &none;              // marks packed mode even with no stage to pull
    return peer_loop(comm, row_comm, packs, n_stages, roots, landing, n_products, plans, vals, operands, last_stage, x_local, n, F, z,
                     timed, compute_stream);
}

extern "C" int dg_peer_spmm_gather(dg_comm* comm, dg_comm* row_comm, int32_t n_stages, const int32_t* roots,
                                   const int32_t* const* stage_lists, const int64_t* stage_rows, float* const* landing,
                                   int32_t n_products, const dg_plan* const* plans, const float* const* vals,
                                   const float* const* operands, const int32_t* last_stage, const float* x_local, int32_t n,
                                   int32_t F, float* z, int timed, void* compute_stream)
{
    if (n_stages > 0 && (!stage_lists || !stage_rows)) return DG_ERR_NULL;
    PeerPacks packs;
    static const int32_t* const no_lists[1] = {nullptr};
    packs.stage_lists = stage_lists ? stage_lists : no_lists;
    packs.stage_rows = stage_rows;
    return peer_loop(comm, row_comm, packs, n_stages, roots, landing, n_products, plans, vals, operands, last_stage, x_local, n, F, z,
                     timed, compute_stream);
}
