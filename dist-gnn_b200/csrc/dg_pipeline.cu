// NCCL communicators and the pipelined broadcast-SpMM stage loop.
//
// Replaces the stage loop of the reference (light_dist_gnn/models/gcn.py:16-30): there every stage is
// synchronize -> dist.broadcast -> synchronize -> spmm -> synchronize on one stream.  Here the broadcasts of all
// stages are enqueued on a side stream, the local products on the compute stream, and CUDA events tie stage s's
// product to stage s's broadcast and stage s+nbuf's broadcast to stage s's product (receive-buffer reuse), so the
// transfer of stage s+1 crosses NVLink while stage s multiplies.  The host never blocks.
// The 1.5D variant (1D_CAGNET/dist_15d.py:61-106) is the same loop inside the column communicator followed by a
// sum of the partial result over the replication (row) communicator.
#include <nccl.h>
#include <cstring>
#include <new>
#include <vector>
#include "dg_internal.h"
#include "dg_comm.h"

namespace {

int finish_comm(ncclComm_t nc, dg_comm** out)
{
    dg_comm* c = new (std::nothrow) dg_comm();
    if (!c) return (int)cudaErrorMemoryAllocation;
    c->comm = nc;
    c->timed_stages = 0;
    DG_NCCL(ncclCommUserRank(nc, &c->rank));
    DG_NCCL(ncclCommCount(nc, &c->nranks));
    DG_NCCL(ncclCommCuDevice(nc, &c->device));
    int prio_low = 0, prio_high = 0;   // highest priority: the few CTAs of a broadcast must not queue behind a product's grid
    DG_CUDA(cudaDeviceGetStreamPriorityRange(&prio_low, &prio_high));
    DG_CUDA(cudaStreamCreateWithPriority(&c->side, cudaStreamNonBlocking, prio_high));
    DG_CUDA(cudaEventCreateWithFlags(&c->ev_input, cudaEventDisableTiming));
    DG_CUDA(cudaEventCreate(&c->t_begin));
    DG_CUDA(cudaEventCreate(&c->t_end));
    *out = c;
    return DG_OK;
}

// `group` consecutive stages share one product: plans[g] is n x (stages_in_group * n).
int check_loop_args(int32_t n_stages, const int32_t* roots, int32_t group, const dg_plan* const* plans,
                    const float* const* vals, const float* x_local, int32_t n, int32_t F, float* const* recv,
                    int32_t nbuf, float* z, int nranks)
{
    if (n_stages < 0 || n < 0 || F < 0 || group < 1) return DG_ERR_DIMS;
    if (nranks == 1 && group != 1) return DG_ERR_DIMS;
    if (n_stages > 0 && (!roots || !plans || !vals)) return DG_ERR_NULL;
    if ((int64_t)n * F > 0 && (!x_local || !z)) return DG_ERR_NULL;
    for (int s = 0; s < n_stages; ++s)
        if (roots[s] < 0 || roots[s] >= nranks) return DG_ERR_DIMS;
    for (int g = 0; g * group < n_stages; ++g) {
        const int in_group = n_stages - g * group < group ? n_stages - g * group : group;
        if (!plans[g]) return DG_ERR_NULL;
        if (plans[g]->m != n || (int64_t)plans[g]->k != (int64_t)in_group * n) return DG_ERR_DIMS;
    }
    if (nranks > 1) {
        if (nbuf < 2 || !recv) return DG_ERR_DIMS;
        for (int b = 0; b < nbuf; ++b)
            if (!recv[b] && (int64_t)n * F > 0) return DG_ERR_NULL;
    }
    return DG_OK;
}

int stage_loop(dg_comm* comm, int32_t n_stages, const int32_t* roots, int32_t group, const dg_plan* const* plans,
               const float* const* vals, const float* x_local, int32_t n, int32_t F, float* const* recv, int32_t nbuf,
               float* z, int timed, cudaStream_t compute)
{
    const int nranks = comm ? comm->nranks : 1;
    int rc = check_loop_args(n_stages, roots, group, plans, vals, x_local, n, F, recv, nbuf, z, nranks);
    if (rc) return rc;
    const int n_groups = (n_stages + group - 1) / group;
    const size_t count = (size_t)n * (size_t)F;
    if (n_stages == 0) {
        if (count) DG_CUDA(cudaMemsetAsync(z, 0, count * sizeof(float), compute));
        return DG_OK;
    }
    if (nranks == 1) {   // no collective: every stage multiplies this rank's own block
        for (int s = 0; s < n_stages; ++s) {
            rc = dg_spmm_csr(plans[s], vals[s], x_local, F, z, F, F, 1.f, s ? 1.f : 0.f, 0u, nullptr, nullptr, compute);
            if (rc) return rc;
        }
        return DG_OK;
    }
    if (comm->poisoned) return DG_ERR_STATE;
    DeviceGuard guard(comm->device);
    if ((rc = make_events(comm->ev_arrived, (size_t)nbuf, cudaEventDisableTiming))) return rc;
    if ((rc = make_events(comm->ev_free, (size_t)nbuf, cudaEventDisableTiming))) return rc;
    comm->timed_stages = 0;
    if (timed) {
        if ((rc = make_events(comm->t_comm, 2 * (size_t)n_groups, cudaEventDefault))) return rc;
        if ((rc = make_events(comm->t_spmm, 2 * (size_t)n_groups, cudaEventDefault))) return rc;
    }
    for (int g = 0; g < n_groups; ++g)                  // scratch growth (it allocates) happens before anything is enqueued
        if ((rc = dg_spmm_prepare(plans[g], F, compute))) return rc;
    IssueGuard issue(comm);
    if (timed) DG_CUDA(cudaEventRecord(comm->t_begin, compute));
    // Everything already queued on the compute stream (the producer of x_local, earlier readers of recv[]) comes first.
    DG_CUDA(cudaEventRecord(comm->ev_input, compute));
    DG_CUDA(cudaStreamWaitEvent(comm->side, comm->ev_input, 0));
    for (int g = 0; g < n_groups; ++g) {
        const int b = g % nbuf;
        const int s0 = g * group;
        const int in_group = n_stages - s0 < group ? n_stages - s0 : group;
        // a single-stage group rooted here is sent and read in place; wider groups gather every block (the root's
        // too) side by side in the receive buffer, so that one product covers the whole group
        const bool in_place = group == 1 && roots[s0] == comm->rank;
        float* landing = in_place ? const_cast<float*>(x_local) : recv[b];
        if (!in_place && g >= nbuf) DG_CUDA(cudaStreamWaitEvent(comm->side, comm->ev_free[b], 0));
        if (timed) DG_CUDA(cudaEventRecord(comm->t_comm[2 * g], comm->side));
        if (count) {
            NcclGroupScope scope;
            if (in_group > 1) DG_NCCL(scope.begin());
            for (int j = 0; j < in_group; ++j)
                DG_NCCL(ncclBroadcast(x_local, landing + (size_t)j * count, count, ncclFloat, roots[s0 + j], comm->comm, comm->side));
            if (in_group > 1) DG_NCCL(scope.end());
        }
        if (timed) DG_CUDA(cudaEventRecord(comm->t_comm[2 * g + 1], comm->side));
        DG_CUDA(cudaEventRecord(comm->ev_arrived[b], comm->side));
        DG_CUDA(cudaStreamWaitEvent(compute, comm->ev_arrived[b], 0));
        if (timed) DG_CUDA(cudaEventRecord(comm->t_spmm[2 * g], compute));
        rc = dg_spmm_csr(plans[g], vals[g], landing, F, z, F, F, 1.f, g ? 1.f : 0.f, 0u, nullptr, nullptr, compute);
        if (rc) return rc;
        if (timed) DG_CUDA(cudaEventRecord(comm->t_spmm[2 * g + 1], compute));
        DG_CUDA(cudaEventRecord(comm->ev_free[b], compute));
    }
    if (timed) {
        DG_CUDA(cudaEventRecord(comm->t_end, compute));
        comm->timed_stages = n_groups;
    }
    issue.done();
    return DG_OK;
}

}  // namespace

extern "C" int dg_comm_unique_id(char host_id_out[128])
{
    if (!host_id_out) return DG_ERR_NULL;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is expected to be 128 bytes");
    ncclUniqueId id;
    DG_NCCL(ncclGetUniqueId(&id));
    memcpy(host_id_out, &id, sizeof(id));
    return DG_OK;
}

extern "C" int dg_comm_create(const char host_id[128], int rank, int nranks, dg_comm** out)
{
    if (!host_id || !out) return DG_ERR_NULL;
    if (nranks < 1 || rank < 0 || rank >= nranks) return DG_ERR_DIMS;
    *out = nullptr;
    ncclUniqueId id;
    memcpy(&id, host_id, sizeof(id));
    ncclComm_t nc;
    DG_NCCL(ncclCommInitRank(&nc, nranks, id, rank));
    return finish_comm(nc, out);
}

extern "C" int dg_comm_split(dg_comm* parent, int color, int key, dg_comm** out)
{
    if (!parent || !out) return DG_ERR_NULL;
    *out = nullptr;
    DeviceGuard guard(parent->device);
    ncclComm_t nc = nullptr;
    DG_NCCL(ncclCommSplit(parent->comm, color < 0 ? NCCL_SPLIT_NOCOLOR : color, key, &nc, nullptr));
    if (!nc) return DG_OK;    // this rank asked to stay out
    return finish_comm(nc, out);
}

extern "C" int dg_comm_destroy(dg_comm* c)
{
    if (!c) return DG_OK;
    DeviceGuard guard(c->device);
    cudaStreamSynchronize(c->side);
    dg_comm_peer_destroy(c);
    ncclCommDestroy(c->comm);
    for (auto* v : {&c->ev_arrived, &c->ev_free, &c->ev_packed, &c->t_comm, &c->t_spmm})
        for (cudaEvent_t e : *v) cudaEventDestroy(e);
    cudaEventDestroy(c->ev_input);
    cudaEventDestroy(c->t_begin);
    cudaEventDestroy(c->t_end);
    cudaStreamDestroy(c->side);
    delete c;
    return DG_OK;
}

extern "C" int dg_comm_rank(const dg_comm* c, int* rank, int* nranks)
{
    if (!c) return DG_ERR_NULL;
    if (rank) *rank = c->rank;
    if (nranks) *nranks = c->nranks;
    return DG_OK;
}

extern "C" int dg_comm_allreduce_sum(dg_comm* c, float* buf, int64_t count, void* stream)
{
    if (!c || (!buf && count > 0)) return DG_ERR_NULL;
    if (count < 0) return DG_ERR_DIMS;
    if (count == 0 || c->nranks == 1) return DG_OK;
    DeviceGuard guard(c->device);
    DG_NCCL(ncclAllReduce(buf, buf, (size_t)count, ncclFloat, ncclSum, c->comm, (cudaStream_t)stream));
    return DG_OK;
}

extern "C" int dg_comm_broadcast(dg_comm* c, float* buf, int64_t count, int root, void* stream)
{
    if (!c || (!buf && count > 0)) return DG_ERR_NULL;
    if (count < 0 || root < 0 || root >= c->nranks) return DG_ERR_DIMS;
    if (count == 0 || c->nranks == 1) return DG_OK;
    DeviceGuard guard(c->device);
    DG_NCCL(ncclBroadcast(buf, buf, (size_t)count, ncclFloat, root, c->comm, (cudaStream_t)stream));
    return DG_OK;
}

extern "C" int dg_bcast_spmm_1d(dg_comm* comm, int32_t n_stages, const int32_t* roots, int32_t group,
                                const dg_plan* const* plans, const float* const* vals, const float* x_local, int32_t n,
                                int32_t F, float* const* recv, int32_t nbuf, float* z, int timed, void* compute_stream)
{
    return stage_loop(comm, n_stages, roots, group, plans, vals, x_local, n, F, recv, nbuf, z, timed, (cudaStream_t)compute_stream);
}

extern "C" int dg_bcast_spmm_15d(dg_comm* col_comm, dg_comm* row_comm, int32_t n_stages, const int32_t* roots,
                                 int32_t group, const dg_plan* const* plans, const float* const* vals,
                                 const float* x_local, int32_t n, int32_t F, float* const* recv, int32_t nbuf, float* z,
                                 int timed, void* compute_stream)
{
    int rc = stage_loop(col_comm, n_stages, roots, group, plans, vals, x_local, n, F, recv, nbuf, z, timed, (cudaStream_t)compute_stream);
    if (rc) return rc;
    if (row_comm) rc = dg_comm_allreduce_sum(row_comm, z, (int64_t)n * F, compute_stream);
    return rc;
}

// Stage loop with a receive area for every remote block: all broadcasts are queued back to back on the side stream
// (nothing ever waits for a buffer to be free), and the products run in the order the caller lists them - typically
// this rank's own block first, which needs no transfer at all, then the remote blocks as they arrive.
extern "C" int dg_bcast_spmm_ordered(dg_comm* comm, dg_comm* row_comm, int32_t n_stages, const int32_t* roots,
                                     int32_t bcast_group, float* const* landing, int32_t n_products, const dg_plan* const* plans,
                                     const float* const* vals, const float* const* operands, const int32_t* last_stage,
                                     const float* x_local, int32_t n, int32_t F, float* z, int timed, void* compute_stream)
{
    cudaStream_t compute = (cudaStream_t)compute_stream;
    if (!comm) return DG_ERR_NULL;
    if (n_stages < 0 || n_products < 0 || n < 0 || F < 0 || bcast_group < 1) return DG_ERR_DIMS;
    if ((n_stages > 0 && (!roots || !landing)) || (n_products > 0 && (!plans || !vals || !operands || !last_stage))) return DG_ERR_NULL;
    const size_t count = (size_t)n * (size_t)F;
    if (count && (!x_local || !z)) return DG_ERR_NULL;
    for (int s = 0; s < n_stages; ++s) {
        if (roots[s] < 0 || roots[s] >= comm->nranks) return DG_ERR_DIMS;
        if (count && roots[s] != comm->rank && !landing[s]) return DG_ERR_NULL;
    }
    int prev = -1;
    for (int p = 0; p < n_products; ++p) {      // products must consume the broadcasts in the order they are issued
        if (!plans[p] || (count && !operands[p])) return DG_ERR_NULL;
        if (plans[p]->m != n || last_stage[p] >= n_stages || (last_stage[p] >= 0 && last_stage[p] < prev)) return DG_ERR_DIMS;
        if (last_stage[p] > prev) prev = last_stage[p];
    }
    if (comm->poisoned) return DG_ERR_STATE;
    int rc;
    DeviceGuard guard(comm->device);
    if ((rc = make_events(comm->ev_arrived, (size_t)n_products, cudaEventDisableTiming))) return rc;
    if ((rc = make_events(comm->ev_free, 1, cudaEventDisableTiming))) return rc;
    comm->timed_stages = 0;
    if (timed) {
        if ((rc = make_events(comm->t_comm, 2 * (size_t)n_products, cudaEventDefault))) return rc;
        if ((rc = make_events(comm->t_spmm, 2 * (size_t)n_products, cudaEventDefault))) return rc;
    }
    for (int p = 0; p < n_products; ++p)                // scratch growth (it allocates) happens before anything is enqueued
        if ((rc = dg_spmm_prepare(plans[p], F, compute))) return rc;
    IssueGuard issue(comm);
    if (timed) DG_CUDA(cudaEventRecord(comm->t_begin, compute));
    if (n_products == 0 && count) DG_CUDA(cudaMemsetAsync(z, 0, count * sizeof(float), compute));
    // the producer of x_local and every earlier reader of the landing area are already queued on the compute stream
    DG_CUDA(cudaEventRecord(comm->ev_input, compute));
    DG_CUDA(cudaStreamWaitEvent(comm->side, comm->ev_input, 0));
    int issued = 0;                                 // broadcasts [0, issued) are on the side stream
    // Broadcasts go out in NCCL groups of bcast_group consecutive stages, cut at the same places on every rank.
    auto issue_until = [&](int until) -> int {
        while (issued < until) {
            const int end = issued + bcast_group < n_stages ? issued + bcast_group : n_stages;
            if (count && comm->nranks > 1) {
                NcclGroupScope scope;
                if (end - issued > 1) DG_NCCL(scope.begin());
                for (int s = issued; s < end; ++s) {
                    float* dst = roots[s] == comm->rank && !landing[s] ? const_cast<float*>(x_local) : landing[s];
                    DG_NCCL(ncclBroadcast(x_local, dst, count, ncclFloat, roots[s], comm->comm, comm->side));
                }
                if (end - issued > 1) DG_NCCL(scope.end());
            }
            issued = end;
        }
        return DG_OK;
    };
    for (int p = 0; p < n_products; ++p) {
        if (timed) DG_CUDA(cudaEventRecord(comm->t_comm[2 * p], comm->side));
        if (last_stage[p] >= issued && (rc = issue_until(last_stage[p] + 1))) return rc;
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
    if (issued < n_stages) {    // broadcasts no product of this rank reads (it only roots them): still its part of the collective
        if ((rc = issue_until(n_stages))) return rc;
        // later work on the compute stream may overwrite x_local: it has to wait until the send has read it
        DG_CUDA(cudaEventRecord(comm->ev_free[0], comm->side));
        DG_CUDA(cudaStreamWaitEvent(compute, comm->ev_free[0], 0));
    }
    if (row_comm) {
        rc = dg_comm_allreduce_sum(row_comm, z, (int64_t)n * F, compute_stream);
        if (rc) return rc;
    }
    if (timed) {
        DG_CUDA(cudaEventRecord(comm->t_end, compute));
        comm->timed_stages = n_products;
    }
    issue.done();
    return DG_OK;
}

// 1D distributed product pipelined along the FEATURE dimension instead of along the source rank: the operand is cut
// into column chunks; chunk c of every rank's block is all-gathered (one bandwidth-optimal collective) into a
// (P*n) x w_c area while the compute stream multiplies chunk c-1 with the rank's whole n x (P*n) row block.  Every
// product sees full-length rows (as on one GPU), z is written exactly once (no read-modify-write between stages), and
// inside a row the sum runs over ascending (source rank, column) - the order of the reference's stage loop.
extern "C" int dg_allgather_spmm(dg_comm* comm, const dg_plan* plan, const float* val, const float* x_local, int32_t n,
                                 int32_t F, int32_t n_chunks, const int32_t* chunk_widths, float* const* pack,
                                 float* const* area, float* z, int timed, void* compute_stream)
{
    cudaStream_t compute = (cudaStream_t)compute_stream;
    if (!comm || !plan) return DG_ERR_NULL;
    if (n < 0 || F < 0 || n_chunks < 1 || !chunk_widths) return DG_ERR_DIMS;
    if (plan->m != n || (int64_t)plan->k != (int64_t)n * comm->nranks) return DG_ERR_DIMS;
    int total = 0;
    for (int c = 0; c < n_chunks; ++c) {
        if (chunk_widths[c] <= 0) return DG_ERR_DIMS;
        total += chunk_widths[c];
    }
    if (total != F) return DG_ERR_DIMS;
    if ((int64_t)n * F == 0) return DG_OK;
    if (!x_local || !z || !area || !area[0] || !area[1] || (n_chunks > 1 && (!pack || !pack[0] || !pack[1]))) return DG_ERR_NULL;
    if (comm->poisoned) return DG_ERR_STATE;
    int rc;
    DeviceGuard guard(comm->device);
    if ((rc = make_events(comm->ev_arrived, 2, cudaEventDisableTiming))) return rc;
    if ((rc = make_events(comm->ev_free, 2, cudaEventDisableTiming))) return rc;
    if ((rc = make_events(comm->ev_packed, 2, cudaEventDisableTiming))) return rc;
    comm->timed_stages = 0;
    if (timed) {
        if ((rc = make_events(comm->t_comm, 2 * (size_t)n_chunks, cudaEventDefault))) return rc;
        if ((rc = make_events(comm->t_spmm, 2 * (size_t)n_chunks, cudaEventDefault))) return rc;
    }
    int widest = 0;
    for (int c = 0; c < n_chunks; ++c) widest = chunk_widths[c] > widest ? chunk_widths[c] : widest;
    if ((rc = dg_spmm_prepare(plan, widest, compute))) return rc;     // scratch growth before anything is enqueued
    IssueGuard issue(comm);
    if (timed) DG_CUDA(cudaEventRecord(comm->t_begin, compute));
    auto stage_in = [&](int c, int c0) -> int {      // pack chunk c on the compute stream, gather it on the side stream
        const int b = c & 1, w = chunk_widths[c];
        const float* send = x_local;
        if (n_chunks > 1) {
            DG_CUDA(cudaMemcpy2DAsync(pack[b], (size_t)w * 4, x_local + c0, (size_t)F * 4, (size_t)w * 4, (size_t)n,
                                      cudaMemcpyDeviceToDevice, compute));
            send = pack[b];
        }
        DG_CUDA(cudaEventRecord(comm->ev_packed[b], compute));
        DG_CUDA(cudaStreamWaitEvent(comm->side, comm->ev_packed[b], 0));
        if (c >= 2) DG_CUDA(cudaStreamWaitEvent(comm->side, comm->ev_free[b], 0));
        if (timed) DG_CUDA(cudaEventRecord(comm->t_comm[2 * c], comm->side));
        DG_NCCL(ncclAllGather(send, area[b], (size_t)n * w, ncclFloat, comm->comm, comm->side));
        if (timed) DG_CUDA(cudaEventRecord(comm->t_comm[2 * c + 1], comm->side));
        DG_CUDA(cudaEventRecord(comm->ev_arrived[b], comm->side));
        return DG_OK;
    };
    std::vector<int> first(n_chunks + 1, 0);
    for (int c = 0; c < n_chunks; ++c) first[c + 1] = first[c] + chunk_widths[c];
    if ((rc = stage_in(0, 0))) return rc;
    for (int c = 0; c < n_chunks; ++c) {
        const int b = c & 1, w = chunk_widths[c];
        if (c + 1 < n_chunks && (rc = stage_in(c + 1, first[c + 1]))) return rc;   // next chunk travels during this product
        DG_CUDA(cudaStreamWaitEvent(compute, comm->ev_arrived[b], 0));
        if (timed) DG_CUDA(cudaEventRecord(comm->t_spmm[2 * c], compute));
        rc = dg_spmm_csr(plan, val, area[b], w, z + first[c], F, w, 1.f, 0.f, 0u, nullptr, nullptr, compute);
        if (rc) return rc;
        if (timed) DG_CUDA(cudaEventRecord(comm->t_spmm[2 * c + 1], compute));
        DG_CUDA(cudaEventRecord(comm->ev_free[b], compute));
    }
    if (timed) {
        DG_CUDA(cudaEventRecord(comm->t_end, compute));
        comm->timed_stages = n_chunks;
    }
    issue.done();
    return DG_OK;
}

extern "C" int dg_comm_last_times(dg_comm* c, dg_stage_times* out)
{
    if (!c || !out) return DG_ERR_NULL;
    *out = dg_stage_times{0.f, 0.f, 0.f, 0};
    if (c->timed_stages == 0) return DG_OK;
    DeviceGuard guard(c->device);
    DG_CUDA(cudaEventSynchronize(c->t_end));
    DG_CUDA(cudaStreamSynchronize(c->side));
    for (int s = 0; s < c->timed_stages; ++s) {
        float ms = 0.f;
        DG_CUDA(cudaEventElapsedTime(&ms, c->t_comm[2 * s], c->t_comm[2 * s + 1]));
        out->comm_ms += ms;
        DG_CUDA(cudaEventElapsedTime(&ms, c->t_spmm[2 * s], c->t_spmm[2 * s + 1]));
        out->spmm_ms += ms;
    }
    DG_CUDA(cudaEventElapsedTime(&out->total_ms, c->t_begin, c->t_end));
    out->stages = c->timed_stages;
    return DG_OK;
}
