// CSR row block x dense fp32 operand for sm_100a:  C = epilogue(alpha * A * B + beta * C).
//
// Replaces cusparseSpMM(COO_ALG4) as called by the reference (light_dist_gnn/spmm_cpp/spmm.cpp:26-28).
//
// The product is a gather: every stored entry (i, j, a) pulls the F-float row j of B and adds a * B[j,:] into
// row i of C.  HBM / L2 bandwidth bounds it, tensor cores have nothing to do here.  Scheduling:
//   * light rows (<= heavy_threshold entries): one warp per row.  A CTA owns a contiguous range of rows and
//     its warps fetch the next row from a shared-memory counter, so a long row does not idle the other warps.
//   * heavy rows: cut into chunks of `chunk` entries at plan time; one warp per chunk writes a partial sum to
//     scratch, then one CTA per heavy row adds the partials in chunk order and applies the epilogue.  No float
//     atomics anywhere: the result is bit-reproducible.
// Inside a warp the 32 lanes are G groups of LPR lanes.  The lanes of a group hold TPL vectors (VEC floats each)
// of the output row at columns (t*LPR + lane)*VEC, so one gathered row of B is read with fully coalesced 64/128-bit
// loads.  The warp reads 32 (col, val) pairs with one coalesced load each and hands them out by shuffle; with
// G > 1 (narrow F) the groups take interleaved entries of the same row and are summed by shuffle at the end.
// U entries are in flight per group before the first FMA, which is what keeps the memory system busy.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <vector>
#include "dg_internal.h"

// Launch shapes, fixed after measurement on B200: 256-thread CTAs, 8 resident per SM (64 warps, <= 32 registers per thread),
// one gathered row in flight per warp (two or four were slower: 11.9 / 12.2 / 14.5 ms on the benchmark graph at F = 256).
#define DG_ROWS_MIN_BLOCKS 8
#define DG_V4_MIN_BLOCKS 8
#define DG_V4_UNROLL 1

namespace {

// ---- instrumentation: event pairs around products while a profile is open -------------------------------------------
struct ProfileState {
    std::mutex mu;
    bool open = false;
    std::vector<cudaEvent_t> events;     // pairs; reused between profiles
    size_t used = 0;
    double alg_bytes = 0, gather_bytes = 0, flops = 0;
    int64_t products = 0;
};
ProfileState g_profile;
std::atomic<int64_t> g_kernel_launches{0};

cudaEvent_t profile_event(cudaStream_t stream)   // caller holds the mutex
{
    if (g_profile.used == g_profile.events.size()) {
        cudaEvent_t e;
        if (cudaEventCreate(&e) != cudaSuccess) return nullptr;
        g_profile.events.push_back(e);
    }
    cudaEvent_t e = g_profile.events[g_profile.used++];
    cudaEventRecord(e, stream);
    return e;
}

struct SpmmArgs {
    const int64_t* rowptr;
    const int32_t* col;
    const float* val;
    const float* B;
    float* C;
    const float* row_scale;
    const float* bias;
    const dg_chunk* chunks;
    const dg_heavy_row* heavy;
    float* scratch;
    int64_t ldb, ldc;
    int32_t m, F, nvec;         // nvec = F / VEC
    int32_t heavy_threshold;
    int32_t n_chunks, n_heavy;
    int32_t rows_per_cta;
    float alpha, beta;
    uint32_t flags;
};

template <int VEC> struct VecT;
template <> struct VecT<1> { using type = float; };
template <> struct VecT<2> { using type = float2; };
template <> struct VecT<4> { using type = float4; };

template <int VEC> __device__ __forceinline__ void load_vec(const float* p, float (&out)[VEC])
{
    if constexpr (VEC == 4) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(p));
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    } else if constexpr (VEC == 2) {
        const float2 v = __ldg(reinterpret_cast<const float2*>(p));
        out[0] = v.x; out[1] = v.y;
    } else {
        out[0] = __ldg(p);
    }
}

template <int VEC> __device__ __forceinline__ void store_vec(float* p, const float (&v)[VEC])
{
    if constexpr (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    else if constexpr (VEC == 2) *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
    else *p = v[0];
}

// Adds sum_{e in [e0,e1)} val[e] * B[col[e], columns of this lane] into acc.  Warp-uniform e0, e1.
template <int VEC, int LPR, int TPL, int U>
__device__ __forceinline__ void gather_range(const SpmmArgs& a, int64_t e0, int64_t e1, const int (&coff)[TPL],
                                             const bool (&act)[TPL], int lane, float (&acc)[TPL][VEC])
{
    constexpr int G = 32 / LPR;
    const int grp = lane / LPR;
    for (int64_t e = e0; e < e1; e += 32) {
        const int cnt = (int)min((int64_t)32, e1 - e);
        int32_t c = 0;
        float v = 0.f;
        if (lane < cnt) {
            c = __ldcs(a.col + e + lane);       // streamed once: keep it from displacing B rows in cache
            v = __ldcs(a.val + e + lane);
        }
        for (int kk = 0; kk < cnt; kk += G * U) {
            float x[U][TPL][VEC];
            float w[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int k = kk + u * G + grp;
                const bool ok = k < cnt;
                const int32_t j = __shfl_sync(0xffffffffu, c, k & 31);
                const float wv = __shfl_sync(0xffffffffu, v, k & 31);
                w[u] = ok ? wv : 0.f;
                const float* brow = a.B + (size_t)j * (size_t)a.ldb;
#pragma unroll
                for (int t = 0; t < TPL; ++t) {
                    if (ok && act[t]) {
                        load_vec<VEC>(brow + coff[t], x[u][t]);
                    } else {
#pragma unroll
                        for (int q = 0; q < VEC; ++q) x[u][t][q] = 0.f;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int t = 0; t < TPL; ++t)
#pragma unroll
                    for (int q = 0; q < VEC; ++q) acc[t][q] = fmaf(w[u], x[u][t][q], acc[t][q]);
        }
    }
    if constexpr (G > 1) {
#pragma unroll
        for (int off = LPR; off < 32; off <<= 1)
#pragma unroll
            for (int t = 0; t < TPL; ++t)
#pragma unroll
                for (int q = 0; q < VEC; ++q) acc[t][q] += __shfl_xor_sync(0xffffffffu, acc[t][q], off);
    }
}

__device__ __forceinline__ float finish(const SpmmArgs& a, float sum, float cold, int32_t row, int32_t colidx)
{
    float out = a.alpha * sum;
    if (a.beta != 0.f) out = fmaf(a.beta, cold, out);
    if (a.flags & DG_EPI_ROW_SCALE) out *= __ldg(a.row_scale + row);
    if (a.flags & DG_EPI_BIAS) out += __ldg(a.bias + colidx);
    if (a.flags & DG_EPI_RELU) out = fmaxf(out, 0.f);
    return out;
}

template <int VEC, int LPR, int TPL>
__device__ __forceinline__ void lane_columns(const SpmmArgs& a, int lane, int (&coff)[TPL], bool (&act)[TPL])
{
    const int gl = lane % LPR;
    const int vec0 = blockIdx.y * (LPR * TPL);
#pragma unroll
    for (int t = 0; t < TPL; ++t) {
        const int v = vec0 + t * LPR + gl;
        act[t] = v < a.nvec;
        coff[t] = v * VEC;
    }
}

// Light rows.  grid.x = ceil(m / rows_per_cta), grid.y = column chunks of LPR*TPL vectors, 256 threads.
template <int VEC, int LPR, int TPL, int U>
__global__ void __launch_bounds__(256, DG_ROWS_MIN_BLOCKS) k_spmm_rows(const SpmmArgs a)
{
    __shared__ int next_row;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int coff[TPL];
    bool act[TPL];
    lane_columns<VEC, LPR, TPL>(a, lane, coff, act);
    const int64_t row0 = (int64_t)blockIdx.x * a.rows_per_cta;
    const int nrows = (int)min((int64_t)a.rows_per_cta, (int64_t)a.m - row0);
    if (threadIdx.x == 0) next_row = blockDim.x >> 5;
    __syncthreads();
    int r = warp;
    while (r < nrows) {
        const int32_t i = (int32_t)(row0 + r);
        const int64_t e0 = __ldg(a.rowptr + i), e1 = __ldg(a.rowptr + i + 1);
        if (e1 - e0 <= a.heavy_threshold) {
            float acc[TPL][VEC];
#pragma unroll
            for (int t = 0; t < TPL; ++t)
#pragma unroll
                for (int q = 0; q < VEC; ++q) acc[t][q] = 0.f;
            gather_range<VEC, LPR, TPL, U>(a, e0, e1, coff, act, lane, acc);
            if (lane < LPR) {
                float* crow = a.C + (size_t)i * (size_t)a.ldc;
#pragma unroll
                for (int t = 0; t < TPL; ++t) {
                    if (!act[t]) continue;
                    float old[VEC], outv[VEC];
                    if (a.beta != 0.f) {
                        if constexpr (VEC == 4) { const float4 o = *reinterpret_cast<const float4*>(crow + coff[t]); old[0] = o.x; old[1] = o.y; old[2] = o.z; old[3] = o.w; }
                        else if constexpr (VEC == 2) { const float2 o = *reinterpret_cast<const float2*>(crow + coff[t]); old[0] = o.x; old[1] = o.y; }
                        else old[0] = crow[coff[t]];
                    } else {
#pragma unroll
                        for (int q = 0; q < VEC; ++q) old[q] = 0.f;
                    }
#pragma unroll
                    for (int q = 0; q < VEC; ++q) outv[q] = finish(a, acc[t][q], old[q], i, coff[t] + q);
                    store_vec<VEC>(crow + coff[t], outv);
                }
            }
        }
        int nxt = 0;
        if (lane == 0) nxt = atomicAdd(&next_row, 1);
        r = __shfl_sync(0xffffffffu, nxt, 0);
    }
}

// Heavy rows, pass 1: one warp per chunk, partial sums (no alpha) to scratch[slot, 0..F).
template <int VEC, int LPR, int TPL, int U>
__global__ void __launch_bounds__(256, DG_ROWS_MIN_BLOCKS) k_spmm_chunks(const SpmmArgs a)
{
    const int lane = threadIdx.x & 31;
    const int chunk_id = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (chunk_id >= a.n_chunks) return;
    int coff[TPL];
    bool act[TPL];
    lane_columns<VEC, LPR, TPL>(a, lane, coff, act);
    const dg_chunk ch = a.chunks[chunk_id];
    float acc[TPL][VEC];
#pragma unroll
    for (int t = 0; t < TPL; ++t)
#pragma unroll
        for (int q = 0; q < VEC; ++q) acc[t][q] = 0.f;
    gather_range<VEC, LPR, TPL, U>(a, ch.e0, ch.e1, coff, act, lane, acc);
    if (lane < LPR) {
        float* srow = a.scratch + (size_t)ch.slot * (size_t)a.F;
#pragma unroll
        for (int t = 0; t < TPL; ++t)
            if (act[t]) {
#pragma unroll
                for (int q = 0; q < VEC; ++q) srow[coff[t] + q] = acc[t][q];
            }
    }
}

// Heavy rows, pass 2: one CTA per heavy row adds its partials in chunk order and applies the epilogue.
__global__ void __launch_bounds__(256) k_spmm_heavy_finish(const SpmmArgs a)
{
    const dg_heavy_row h = a.heavy[blockIdx.x];
    float* crow = a.C + (size_t)h.row * (size_t)a.ldc;
    for (int f = threadIdx.x; f < a.F; f += blockDim.x) {
        float sum = 0.f;
        for (int c = 0; c < h.nchunks; ++c) sum += a.scratch[(size_t)(h.slot0 + c) * (size_t)a.F + f];
        const float old = a.beta != 0.f ? crow[f] : 0.f;
        crow[f] = finish(a, sum, old, h.row, f);
    }
}

// ---- lean kernel for 16-byte aligned rows: float4 gathers, 32-bit offsets, one launch per product ---------------------
// Same scheduling and the same sum order as the generic kernels above, written to need few registers: on B200 the gather
// runs fastest at full occupancy (64 warps per SM, one gathered row per warp in flight).  A warp covers a column tile of
// 128 floats (every lane one float4; blockIdx.y walks the tiles, tile-major, so the CTAs resident at one time gather from
// the same 512-byte slice of B's rows), `on` masks the lanes of a partial last tile.  Row offsets col * (ldb / 4) are 32-bit
// (the host checks k * ldb / 4 < 2^31).  Measured on the 2,449,029-node benchmark graph (F = 256; whole graph / the eight
// 306 k-row stage blocks of one rank): two float4 per lane in separate row and chunk kernels 12.83 / 2.73 ms, this kernel
// 12.16 / 2.50 ms; F = 100: 6.15 / 1.82 -> 6.09 / 1.39 ms.
template <int U>
__device__ __forceinline__ void gather_v4(const float4* __restrict__ bl, int ld4, const int32_t* __restrict__ colp,
                                          const float* __restrict__ valp, int len, bool on, float4& acc)
{
    // colp / valp point at this lane's first entry (entry `lane` of the range); len = entries in the range (a light row or
    // one chunk of a split row, so it fits 32 bits with room to spare)
    for (int base = 0; base < len; base += 32) {
        const int cnt = min(32, len - base);
        int c = 0;
        float v = 0.f;
        if ((int)(threadIdx.x & 31) < cnt) {
            c = __ldcs(colp + base) * ld4;        // streamed once: keep it from displacing rows of B in cache
            v = __ldcs(valp + base);
        }
        for (int k = 0; k < cnt; k += U) {
            float4 x[U];
            float w[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int idx = __shfl_sync(0xffffffffu, c, (k + u) & 31);
                w[u] = __shfl_sync(0xffffffffu, v, (k + u) & 31);     // lanes >= cnt hold 0: a zero weight ...
                x[u] = k + u < cnt && on ? __ldg(bl + idx) : make_float4(0.f, 0.f, 0.f, 0.f);   // ... and nothing is loaded
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                acc.x = fmaf(w[u], x[u].x, acc.x); acc.y = fmaf(w[u], x[u].y, acc.y);
                acc.z = fmaf(w[u], x[u].z, acc.z); acc.w = fmaf(w[u], x[u].w, acc.w);
            }
        }
    }
}

// One launch for a whole product: the first `chunk_ctas` CTAs take the chunks of the split rows (one warp per chunk, partial
// sums to scratch), the others the light rows.  A chunk is a chain of `chunk` gathers walked by one warp, so on a small
// block the chunk work is a fixed latency that does not fill the GPU (385 CTAs for a 306 k-row stage block of the 8-rank
// partition: 0.09 ms on its own next to 0.25 ms of light rows); issued first in the same grid it runs underneath the light
// rows instead of after them.  k_spmm_heavy_finish follows as a second launch.
// PLAIN: alpha == 1 and no row scale, bias or ReLU - what the stage loops run; fmaf(beta, old, sum) with old = 0 is sum, so
// it gives the bits of the general epilogue.
template <int U, bool PLAIN>
__global__ void __launch_bounds__(256, DG_V4_MIN_BLOCKS) k_spmm_v4(const SpmmArgs a, const int chunk_ctas)
{
    __shared__ int next_row;
    const int lane = threadIdx.x & 31;
    const int vec0 = blockIdx.y * 32 + lane;                          // this lane's float4 of the row
    const bool on = vec0 < a.nvec;
    const float4* bl = reinterpret_cast<const float4*>(a.B) + vec0;
    const int ld4 = (int)(a.ldb >> 2);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if ((int)blockIdx.x < chunk_ctas) {
        const int chunk_id = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
        if (chunk_id >= a.n_chunks) return;
        const dg_chunk ch = a.chunks[chunk_id];
        gather_v4<U>(bl, ld4, a.col + ch.e0 + lane, a.val + ch.e0 + lane, (int)(ch.e1 - ch.e0), on, acc);
        if (on) __stcs(reinterpret_cast<float4*>(a.scratch + (size_t)ch.slot * (size_t)a.F) + vec0, acc);
        return;
    }
    const int32_t row0 = ((int)blockIdx.x - chunk_ctas) * a.rows_per_cta;     // m < 2^31
    const int nrows = min(a.rows_per_cta, a.m - row0);
    if (threadIdx.x == 0) next_row = blockDim.x >> 5;
    __syncthreads();
    int r = threadIdx.x >> 5;
    while (r < nrows) {
        const int32_t i = row0 + r;
        const int64_t e0 = __ldg(a.rowptr + i);
        const int64_t len = __ldg(a.rowptr + i + 1) - e0;
        if (len <= a.heavy_threshold) {
            float4* cp = reinterpret_cast<float4*>(a.C + (size_t)i * (size_t)a.ldc) + vec0;
            float4 old = make_float4(0.f, 0.f, 0.f, 0.f);
            if (on && a.beta != 0.f) old = __ldcs(cp);          // requested before the gather; streams through, must not displace rows of B in L2
            gather_v4<U>(bl, ld4, a.col + e0 + lane, a.val + e0 + lane, (int)len, on, acc);
            if (on) {
                if constexpr (PLAIN) {
                    __stcs(cp, make_float4(fmaf(a.beta, old.x, acc.x), fmaf(a.beta, old.y, acc.y), fmaf(a.beta, old.z, acc.z),
                                           fmaf(a.beta, old.w, acc.w)));
                } else {
                    const int c = vec0 * 4;
                    __stcs(cp, make_float4(finish(a, acc.x, old.x, i, c), finish(a, acc.y, old.y, i, c + 1),
                                           finish(a, acc.z, old.z, i, c + 2), finish(a, acc.w, old.w, i, c + 3)));
                }
            }
            acc = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        int nxt = 0;
        if (lane == 0) nxt = atomicAdd(&next_row, 1);
        r = __shfl_sync(0xffffffffu, nxt, 0);
    }
}

int launch_v4(const SpmmArgs& a, cudaStream_t stream)
{
    constexpr int U = DG_V4_UNROLL;
    const int col_tiles = (a.nvec + 31) / 32;
    const int chunk_ctas = (a.n_chunks + 7) / 8;
    const int64_t row_ctas = ((int64_t)a.m + a.rows_per_cta - 1) / a.rows_per_cta;
    if (chunk_ctas + row_ctas > 0) {
        dim3 grid((unsigned)(chunk_ctas + row_ctas), (unsigned)col_tiles);
        if (a.flags == 0u && a.alpha == 1.f) k_spmm_v4<U, true><<<grid, 256, 0, stream>>>(a, chunk_ctas);
        else k_spmm_v4<U, false><<<grid, 256, 0, stream>>>(a, chunk_ctas);
        g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
    }
    if (a.n_heavy > 0) {
        k_spmm_heavy_finish<<<(unsigned)a.n_heavy, 256, 0, stream>>>(a);
        g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
    }
    return (int)cudaGetLastError();
}

template <int VEC, int LPR, int TPL>
int launch_variant(const SpmmArgs& a, cudaStream_t stream)
{
    constexpr int U = (TPL * VEC >= 8) ? 1 : 2;          // gathers in flight per lane group before the first FMA
    const int col_chunks = (a.nvec + LPR * TPL - 1) / (LPR * TPL);
    if (a.m > 0) {
        dim3 grid((unsigned)(((int64_t)a.m + a.rows_per_cta - 1) / a.rows_per_cta), (unsigned)col_chunks);
        k_spmm_rows<VEC, LPR, TPL, U><<<grid, 256, 0, stream>>>(a);
        g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
    }
    if (a.n_chunks > 0) {
        dim3 grid((unsigned)((a.n_chunks + 7) / 8), (unsigned)col_chunks);
        k_spmm_chunks<VEC, LPR, TPL, U><<<grid, 256, 0, stream>>>(a);
        k_spmm_heavy_finish<<<(unsigned)a.n_heavy, 256, 0, stream>>>(a);
        g_kernel_launches.fetch_add(2, std::memory_order_relaxed);
    }
    return (int)cudaGetLastError();
}

template <int VEC>
int launch_vec(const SpmmArgs& a, cudaStream_t stream)
{
    const int nvec = a.nvec;
    if (nvec <= 4) return launch_variant<VEC, 4, 1>(a, stream);
    if (nvec <= 8) return launch_variant<VEC, 8, 1>(a, stream);
    if (nvec <= 16) return launch_variant<VEC, 16, 1>(a, stream);
    if (nvec <= 32) return launch_variant<VEC, 32, 1>(a, stream);
    if (nvec <= 64) return launch_variant<VEC, 32, 2>(a, stream);
    return launch_variant<VEC, 32, 4>(a, stream);       // wider rows take ceil(nvec/128) column chunks
}

bool aligned(const void* p, size_t bytes) { return (reinterpret_cast<uintptr_t>(p) % bytes) == 0; }

}  // namespace

int dg_check_spmm_args(const dg_plan* plan, const float* val, const float* B, int64_t ldb, const float* C, int64_t ldc,
                       int32_t F, uint32_t flags, const float* row_scale, const float* bias)
{
    if (!plan) return DG_ERR_NULL;
    if (F < 0 || ldb < F || ldc < F) return DG_ERR_DIMS;
    if (flags & ~(DG_EPI_ROW_SCALE | DG_EPI_BIAS | DG_EPI_RELU)) return DG_ERR_UNSUPPORTED;
    if (plan->m > 0 && F > 0 && !C) return DG_ERR_NULL;
    if (plan->nnz > 0 && F > 0 && (!val || !B)) return DG_ERR_NULL;
    if ((flags & DG_EPI_ROW_SCALE) && !row_scale) return DG_ERR_NULL;
    if ((flags & DG_EPI_BIAS) && !bias) return DG_ERR_NULL;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev != plan->device) return DG_ERR_STATE;
    return DG_OK;
}

int dg_spmm_launch_rows(const dg_plan* plan, const float* val, const float* B, int64_t ldb, float* C, int64_t ldc,
                        int32_t F, float alpha, float beta, uint32_t flags, const float* row_scale, const float* bias,
                        float* scratch, cudaStream_t stream)
{
    if (plan->m == 0 || F == 0) return DG_OK;
    SpmmArgs a{};
    a.rowptr = plan->rowptr; a.col = plan->col; a.val = val; a.B = B; a.C = C;
    a.row_scale = row_scale; a.bias = bias; a.chunks = plan->chunks; a.heavy = plan->heavy; a.scratch = scratch;
    a.ldb = ldb; a.ldc = ldc; a.m = plan->m; a.F = F;
    a.heavy_threshold = plan->heavy_threshold; a.n_chunks = plan->n_chunks; a.n_heavy = plan->n_heavy;
    a.rows_per_cta = 64;
    a.alpha = alpha; a.beta = beta; a.flags = flags;
    // widest vector the shapes and addresses allow (B may be NULL only when there is nothing to gather)
    int vec = 1;
    if (F % 4 == 0 && ldb % 4 == 0 && ldc % 4 == 0 && aligned(B, 16) && aligned(C, 16)) vec = 4;
    else if (F % 2 == 0 && ldb % 2 == 0 && ldc % 2 == 0 && aligned(B, 8) && aligned(C, 8)) vec = 2;
    a.nvec = F / vec;
    // The lean kernel takes rows of more than 64 floats, and narrower ones (36 to 64 floats) when the rows are short: there
    // (stage blocks of a partition, about 6 entries per row) it is 18 % faster than the generic kernel, which wins on long
    // rows by walking two entries per warp at a time (whole graph, F = 48: 4.1 against 4.9 ms).
    const bool narrow_ok = a.nvec > 8 && plan->nnz < (int64_t)16 * plan->m;
    if (vec == 4 && (a.nvec > 16 || narrow_ok) && (int64_t)plan->k * (ldb / 4) + a.nvec < (int64_t)INT32_MAX) return launch_v4(a, stream);
    switch (vec) {
        case 4: return launch_vec<4>(a, stream);
        case 2: return launch_vec<2>(a, stream);
        default: return launch_vec<1>(a, stream);
    }
}

// Picks the kernel family (streaming when the operands allow it, row kernels otherwise) and brackets the product with
// profile events while a profile is open.
int dg_spmm_launch(const dg_plan* plan, const float* val, const float* B, int64_t ldb, float* C, int64_t ldc,
                   int32_t F, float alpha, float beta, uint32_t flags, const float* row_scale, const float* bias,
                   float* scratch, cudaStream_t stream)
{
    if (plan->m == 0 || F == 0) return DG_OK;
    bool profiled = false;
    {
        std::lock_guard<std::mutex> lock(g_profile.mu);
        if (g_profile.open) {
            profiled = profile_event(stream) != nullptr;
            const double rw = 4.0 * F * plan->m * (beta != 0.f ? 2.0 : 1.0), csr = 8.0 * plan->nnz + 4.0 * (plan->m + 1.0);
            g_profile.alg_bytes += csr + 4.0 * F * plan->touched_columns + rw;
            g_profile.gather_bytes += csr + 4.0 * F * plan->nnz + rw;
            g_profile.flops += 2.0 * plan->nnz * F;
            g_profile.products += 1;
        }
    }
    int rc;
    if (dg_spmm_stream_eligible(plan, B, ldb, C, ldc, F)) {
        int launches = 0;
        rc = dg_spmm_stream_launch(plan, val, B, ldb, C, ldc, F, alpha, beta, flags, row_scale, bias, scratch, stream, &launches);
        g_kernel_launches.fetch_add(launches, std::memory_order_relaxed);
    } else {
        rc = dg_spmm_launch_rows(plan, val, B, ldb, C, ldc, F, alpha, beta, flags, row_scale, bias, scratch, stream);
    }
    if (profiled) {
        std::lock_guard<std::mutex> lock(g_profile.mu);
        profile_event(stream);
    }
    return rc;
}

extern "C" int dg_profile_begin(void)
{
    std::lock_guard<std::mutex> lock(g_profile.mu);
    g_profile.open = true;
    g_profile.used = 0;
    g_profile.alg_bytes = g_profile.gather_bytes = g_profile.flops = 0;
    g_profile.products = 0;
    g_kernel_launches.store(0);
    return DG_OK;
}

extern "C" int dg_profile_end(dg_profile* out)
{
    if (!out) return DG_ERR_NULL;
    std::lock_guard<std::mutex> lock(g_profile.mu);
    g_profile.open = false;
    DG_CUDA(cudaDeviceSynchronize());
    double ms = 0;
    for (size_t i = 0; i + 1 < g_profile.used; i += 2) {
        float t = 0.f;
        DG_CUDA(cudaEventElapsedTime(&t, g_profile.events[i], g_profile.events[i + 1]));
        ms += t;
    }
    *out = dg_profile{ms, g_profile.alg_bytes, g_profile.gather_bytes, g_profile.flops, g_profile.products,
                      g_kernel_launches.load()};
    g_profile.used = 0;
    return DG_OK;
}

// Grows the plan's scratch to what a product of width F may need (either kernel family); allocates and synchronises
// `stream` only when it has to grow.  The stage loops call it for every plan before they enqueue anything, so that an
// allocation failure cannot leave a loop half issued.
int dg_spmm_prepare(const dg_plan* plan, int32_t F, cudaStream_t stream)
{
    if (!plan) return DG_ERR_NULL;
    dg_plan* p = const_cast<dg_plan*>(plan);
    const int64_t need = dg_stream_selected() ? dg_scratch_floats(plan, F) : (int64_t)plan->n_chunks * F;
    if (need > p->scratch_floats) {
        DG_CUDA(cudaStreamSynchronize(stream));
        cudaFree(p->scratch);
        p->scratch = nullptr;
        p->scratch_floats = 0;
        DG_CUDA(cudaMalloc((void**)&p->scratch, (size_t)need * sizeof(float)));
        p->scratch_floats = need;
    }
    return DG_OK;
}

extern "C" int dg_spmm_csr(const dg_plan* plan, const float* val, const float* B, int64_t ldb, float* C, int64_t ldc,
                           int32_t F, float alpha, float beta, uint32_t flags, const float* row_scale,
                           const float* bias, void* stream)
{
    int rc = dg_check_spmm_args(plan, val, B, ldb, C, ldc, F, flags, row_scale, bias);
    if (rc) return rc;
    dg_plan* p = const_cast<dg_plan*>(plan);
    const int64_t need = dg_spmm_stream_eligible(plan, B, ldb, C, ldc, F) ? 2 * (int64_t)p->n_tasks * F : (int64_t)p->n_chunks * F;
    if (need > p->scratch_floats) {     // first use at this width: grow the plan's scratch (allocates, synchronises)
        DG_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
        cudaFree(p->scratch);
        p->scratch = nullptr;
        p->scratch_floats = 0;
        DG_CUDA(cudaMalloc((void**)&p->scratch, (size_t)need * sizeof(float)));
        p->scratch_floats = need;
    }
    return dg_spmm_launch(plan, val, B, ldb, C, ldc, F, alpha, beta, flags, row_scale, bias, p->scratch, (cudaStream_t)stream);
}

extern "C" int dg_spmm_coo(const int32_t* row, const int32_t* col, const float* val, int64_t nnz, int32_t m, int32_t k,
                           const float* B, float* C, int32_t F, float alpha, float beta, void* stream)
{
    dg_plan* plan = nullptr;
    int rc = dg_plan_build(row, col, nnz, m, k, 0, 0, /*lean=*/true, stream, &plan);
    if (rc) return rc;
    rc = dg_spmm_csr(plan, val, B, F, C, F, F, alpha, beta, 0u, nullptr, nullptr, stream);
    if (rc == DG_OK) rc = (int)cudaStreamSynchronize((cudaStream_t)stream);   // the plan's buffers die below
    dg_plan_destroy(plan);
    return rc;
}

extern "C" const char* dg_strerror(int code)
{
    switch (code) {
        case DG_OK: return "ok";
        case DG_ERR_NULL: return "a required pointer is NULL";
        case DG_ERR_DIMS: return "negative or inconsistent sizes";
        case DG_ERR_INDEX: return "sparse indices are not row-sorted or fall outside the matrix";
        case DG_ERR_UNSUPPORTED: return "unsupported request";
        case DG_ERR_STATE: return "object used in the wrong state or on the wrong device";
        case DG_ERR_SCRATCH: return "request exceeds the fixed scratch capacity";
        default: break;
    }
    if (code >= DG_NCCL_ERROR_BASE) return "NCCL error (code - 10000 is the ncclResult_t)";
    if (code > 0) return cudaGetErrorString((cudaError_t)code);
    return "unknown error";
}

extern "C" int dg_version(void) { return 100; }
