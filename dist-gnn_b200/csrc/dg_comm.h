// The communicator object shared by the stage loops (dg_pipeline.cu) and the peer-copy loop (dg_peer.cu).
#pragma once
#include <nccl.h>
#include <cstdint>
#include <vector>
#include "dg_internal.h"

#define DG_NCCL(expr)                                                  \
    do {                                                               \
        ncclResult_t _r = (expr);                                      \
        if (_r != ncclSuccess) return DG_NCCL_ERROR_BASE + (int)_r;    \
    } while (0)

struct dg_comm {
    ncclComm_t comm;
    int rank, nranks, device;
    cudaStream_t side;                       // transfers run here
    cudaEvent_t ev_input;                    // this rank's block is ready on the compute stream
    std::vector<cudaEvent_t> ev_arrived;     // per receive buffer: transfer into it finished
    std::vector<cudaEvent_t> ev_free;        // per receive buffer: the product that read it finished
    std::vector<cudaEvent_t> ev_packed;      // per pack buffer: the column chunk to send is ready
    std::vector<cudaEvent_t> t_comm, t_spmm; // timing pairs per stage (2 events each)
    cudaEvent_t t_begin, t_end;
    int timed_stages;
    // peer-copy loop: two send buffers exported over CUDA IPC, every rank's two buffers as mapped here ([2*r + b])
    float* peer_send[2] = {nullptr, nullptr};
    int64_t peer_floats = 0;
    std::vector<float*> peer_ptr;
    float* peer_token = nullptr;             // the one float of the meeting-point all-reduce
    cudaEvent_t ev_barrier = nullptr;
    uint64_t peer_loops = 0;
    std::vector<cudaStream_t> peer_lanes;    // extra copy streams: a block is cut into pieces that travel side by side
    std::vector<cudaEvent_t> ev_lane;
    // Set when a stage loop failed after it had started to enqueue: this rank's collectives or send-buffer parity may no
    // longer match its peers', so every later loop on this communicator is refused with DG_ERR_STATE instead of hanging.
    bool poisoned = false;
};

// Marks the communicator as poisoned unless the loop that created it ran to its end (call done()).
struct IssueGuard {
    dg_comm* c;
    bool finished = false;
    explicit IssueGuard(dg_comm* comm) : c(comm) {}
    void done() { finished = true; }
    ~IssueGuard() { if (!finished && c) c->poisoned = true; }
};

// ncclGroupStart / ncclGroupEnd as a scope: the group is closed on every path out of it, error returns included.
struct NcclGroupScope {
    bool open = false;
    ncclResult_t begin() { ncclResult_t r = ncclGroupStart(); open = (r == ncclSuccess); return r; }
    ncclResult_t end() { open = false; return ncclGroupEnd(); }
    ~NcclGroupScope() { if (open) ncclGroupEnd(); }
};

inline int make_events(std::vector<cudaEvent_t>& v, size_t count, unsigned flags)
{
    while (v.size() < count) {
        cudaEvent_t e;
        DG_CUDA(cudaEventCreateWithFlags(&e, flags));
        v.push_back(e);
    }
    return DG_OK;
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) { cudaGetDevice(&prev); if (prev != dev) cudaSetDevice(dev); else prev = -1; }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

int dg_comm_peer_destroy(dg_comm* c);        // dg_peer.cu: unmaps the peers' buffers and frees this rank's
