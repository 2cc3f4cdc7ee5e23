// dg_spmm_csr_static: the local product for callers that must not allocate device memory.
//
// Who needs it: a host program whose device memory is already fully reserved by its own pool (a cudaMalloc from a
// library would fail or fragment it), or a latency-critical loop that cannot afford the implicit device-wide
// synchronisation of cudaMalloc / cudaFree.  dg_spmm_csr grows a plan-owned scratch buffer with cudaMalloc the first
// time a plan is used at a wider F; this variant never allocates: the partial sums of split (heavy) rows go to a
// fixed array that is part of the library image, so every GPU that loads the library carries it until the process ends.
//
// Limit: DG_STATIC_SCRATCH_FLOATS floats (16 MiB).  A product needs heavy_chunks * F floats of scratch
// (dg_plan_get_stats gives heavy_chunks); a larger request is refused with DG_ERR_SCRATCH before anything is launched.
//
// Sharing: all calls on a device use the same array.  Nothing in it has to start at zero - every scratch row is fully
// written by the chunk kernel before the finishing kernel reads it - so no clearing is done between calls, but two
// calls that overlap in time on the GPU (different streams) race on it.  Serialise them on one stream.
//
// Set-up: the array's name below is a host-side handle, not a device address.  The address is looked up once per device
// with cudaGetSymbolAddress while that device is current, and cached.  With CUDA's lazy module loading that first lookup
// is also the moment the 16 MiB array is materialised on the device (it can fail for lack of memory, and may synchronise).
// dg_static_scratch_prepare() does the lookup on its own: call it once per device where an allocation is still acceptable
// (next to dg_plan_create, before the host's pool reserves the rest of the memory, before any stream capture); after it,
// dg_spmm_csr_static touches neither the allocator nor the module loader.  Without it the first product call on a device
// does the lookup.
//
// The entry always runs the row kernels (the streaming family sizes its scratch differently) and its products are not
// counted by dg_profile_begin / dg_profile_end.
#include <mutex>
#include "dg_internal.h"

#define DG_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)
#define DG_MAX_DEVICES 64

static __device__ __align__(256) float g_static_scratch[DG_STATIC_SCRATCH_FLOATS];

namespace {
std::mutex g_lookup_mutex;
float* g_scratch_address[DG_MAX_DEVICES] = {nullptr};

// Device address of g_static_scratch on `device`, which must be the current device.
int static_scratch_address(int device, float** out)
{
    if (device < 0 || device >= DG_MAX_DEVICES) return DG_ERR_STATE;
    std::lock_guard<std::mutex> lock(g_lookup_mutex);
    if (!g_scratch_address[device]) {
        float* ptr = nullptr;
        DG_CUDA(cudaGetSymbolAddress((void**)&ptr, g_static_scratch));
        if (!ptr) return DG_ERR_STATE;
        g_scratch_address[device] = ptr;
    }
    *out = g_scratch_address[device];
    return DG_OK;
}
}  // namespace

extern "C" int64_t dg_static_scratch_capacity(void) { return DG_STATIC_SCRATCH_FLOATS; }

extern "C" int dg_static_scratch_prepare(void)
{
    int device = -1;
    DG_CUDA(cudaGetDevice(&device));
    float* unused = nullptr;
    return static_scratch_address(device, &unused);
}

extern "C" int dg_spmm_csr_static(const dg_plan* plan, const float* val, const float* B, int64_t ldb, float* C,
                                  int64_t ldc, int32_t F, float alpha, float beta, uint32_t flags,
                                  const float* row_scale, const float* bias, void* stream)
{
    int rc = dg_check_spmm_args(plan, val, B, ldb, C, ldc, F, flags, row_scale, bias);   // also checks the current device
    if (rc) return rc;
    if ((int64_t)plan->n_chunks * F > DG_STATIC_SCRATCH_FLOATS) return DG_ERR_SCRATCH;
    float* scratch = nullptr;
    if ((rc = static_scratch_address(plan->device, &scratch))) return rc;
    return dg_spmm_launch_rows(plan, val, B, ldb, C, ldc, F, alpha, beta, flags, row_scale, bias, scratch, (cudaStream_t)stream);
}
