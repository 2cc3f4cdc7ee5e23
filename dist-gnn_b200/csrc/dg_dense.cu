// Dense transform of the GCN layer on the 5th-generation tensor cores:  C[M x N] = act(A[M x K] * Bt[N x K]^T), fp32 in
// and out, for the tall-skinny shapes either side of the SpMM (Z*W and AG*W^T: light_dist_gnn/models/gcn.py:41, :49;
// M = rows of the rank's block, K and N <= 256).
//
// fp32 accuracy from TF32 tensor cores: every operand is cut into a TF32-exact head (sign, exponent, top 10 mantissa
// bits) and its residual tail, and the accumulator (fp32, in tensor memory) receives
//     A_head*B_head + A_head*B_tail + A_tail*B_head
// (the dropped tail*tail term is 2^-22 relative).  The small matrix Bt is split once on the host side of the call
// (dg_dense_split); A is split inside the kernel, in shared memory, on its way from TMA to the MMA.  The tensor cores
// ignore the low 13 bits of a TF32 operand (verified: identical bits with and without a masked copy), so the tile as
// loaded serves as head and only the tail is written.
//
// k_dense_nt: one CTA per 128-row tile.  Warp 0 drives TMA (128B-swizzled boxes of 32 K-columns: A rows, Bt head, Bt tail)
// through a 2-stage ring; warps 2-5 split A and later drain the accumulator (tcgen05.ld) to global memory with the
// optional ReLU / ReLU-backward mask; one thread of warp 1 issues the tcgen05.mma instructions (kind::tf32, 128 x N x 8,
// operands described by shared-memory matrix descriptors, accumulator in TMEM columns) and commits them to the mbarriers
// that recycle the stages.  k_dense_nt_persistent: one CTA per SM walks the tiles with two accumulators and separate
// epilogue warps (used for results wider than 128 columns).  k_dense_tn (further down): the weight gradient X^T * G,
// both operands MN-major, split-K over the CTAs with periodic accumulator flushes.
// Every mbarrier wait is bounded; a role that gives up sets the status word and the CTA still frees its TMEM.
#include <cuda.h>
#include <cstdint>
#include <cstring>
#include "dg_internal.h"

namespace {

constexpr int BM = 128;             // rows per CTA tile (UMMA M)
constexpr int BK = 32;              // fp32 K-columns per stage = one 128-byte swizzle row
constexpr int STAGES = 2;
constexpr int kWaitLimit = 1 << 22;
constexpr int kThreads = 192;

struct DenseArgs {
    float* C;
    int64_t ldc;
    int64_t M;
    int32_t N, K, n_pad;            // n_pad = N rounded up to 16 (UMMA N)
    uint32_t relu;
    const float* mask;              // optional [M x N]: the result is zeroed where mask <= 0 (ReLU backward), else nullptr
    int64_t ldm;
    int32_t raw_head;               // persistent kernel: 0 = masked head copy; 1 = the fp32 tile itself serves as head;
                                    // 2 = as 1, and the two head passes of a slab are issued before its tail is ready
    int* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int limit = kWaitLimit)      // bounded
{
    for (int i = 0; i < limit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// Shared-memory matrix descriptor of a K-major tile stored as 128-byte rows with the 128B swizzle: 8-row groups are
// 1024 bytes apart (stride byte offset), the leading byte offset is unused for this layout, descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);            // start address, 16-byte units
    d |= (uint64_t)1 << 16;                                   // leading byte offset (ignored with swizzle), 16-byte units
    d |= (uint64_t)(1024 >> 4) << 32;                         // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                                   // descriptor version for sm_100
    d |= (uint64_t)2 << 61;                                   // layout type: SWIZZLE_128B
    return d;
}
// Instruction descriptor for kind::tf32: fp32 accumulator, TF32 A and B, both K-major, shape 128 x n_pad.
__device__ __forceinline__ uint32_t umma_idesc_tf32(int n_pad)
{
    uint32_t d = 0;
    d |= 1u << 4;                                             // accumulator format: F32
    d |= 2u << 7;                                             // A format: TF32
    d |= 2u << 10;                                            // B format: TF32
    d |= (uint32_t)(n_pad >> 3) << 17;                        // N / 8
    d |= (uint32_t)(BM >> 4) << 24;                           // M / 16
    return d;
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 16 consecutive accumulator columns of this warp's 32 tensor-memory lanes (no wait: pair with tcgen05.wait::ld).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

}  // namespace

namespace {

__global__ void __launch_bounds__(kThreads, 1)
k_dense_nt(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmBh,
           const __grid_constant__ CUtensorMap tmBt, const DenseArgs a)
{
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                 // swizzled tiles need 1024-byte alignment
    unsigned char* gbase = smem_raw + (base - raw);
    const int b_bytes = a.n_pad * 128;                            // one slab of Bt: n_pad rows x 128 bytes
    const int stage_bytes = 2 * BM * 128 + 2 * b_bytes;           // A head, A tail, Bt head, Bt tail
    const uint32_t bars = base + STAGES * stage_bytes;
    const uint32_t full0 = bars, ready0 = bars + 8 * STAGES, empty0 = bars + 16 * STAGES, acc_full = bars + 24 * STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gbase + STAGES * stage_bytes + 24 * STAGES + 8);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t m0 = (int64_t)blockIdx.x * BM;
    const int nslabs = (a.K + BK - 1) / BK;
    int tmem_cols = 32;
    while (tmem_cols < a.n_pad) tmem_cols <<= 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(ready0 + 8 * s, 128);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                                              // one warp allocates the accumulator columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {                                          // TMA producer
            for (int i = 0; i < nslabs && ok; ++i) {
                const int s = i % STAGES, u = i / STAGES;
                if (u > 0) ok = mbar_wait(empty0 + 8 * s, (u - 1) & 1);
                if (!ok) break;
                const uint32_t st = base + s * stage_bytes;
                mbar_expect_tx(full0 + 8 * s, BM * 128 + 2 * b_bytes);
                tma_load_2d(st, &tmA, i * BK, (int)m0, full0 + 8 * s);
                tma_load_2d(st + 2 * BM * 128, &tmBh, i * BK, 0, full0 + 8 * s);
                tma_load_2d(st + 2 * BM * 128 + b_bytes, &tmBt, i * BK, 0, full0 + 8 * s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                          // MMA issuer
            const uint32_t idesc = umma_idesc_tf32(a.n_pad);
            for (int i = 0; i < nslabs && ok; ++i) {
                const int s = i % STAGES, u = i / STAGES;
                ok = mbar_wait(ready0 + 8 * s, u & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t st = base + s * stage_bytes;
                const uint64_t a_head = umma_desc_sw128(st), a_tail = umma_desc_sw128(st + BM * 128);
                const uint64_t b_head = umma_desc_sw128(st + 2 * BM * 128), b_tail = umma_desc_sw128(st + 2 * BM * 128 + b_bytes);
#pragma unroll
                for (int k = 0; k < BK / 8; ++k) {               // 8 TF32 columns = 32 bytes per MMA: +2 in 16-byte units
                    umma_tf32(tmem, a_tail + 2 * k, b_head + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    umma_tf32(tmem, a_head + 2 * k, b_tail + 2 * k, idesc, 1u);
                    umma_tf32(tmem, a_head + 2 * k, b_head + 2 * k, idesc, 1u);
                }
                umma_commit(empty0 + 8 * s);                      // the stage is free once these MMAs have read it
            }
            if (ok) umma_commit(acc_full);
        }
    } else {
        const int t = threadIdx.x - 64;                           // 0..127: split A, then drain the accumulator
        for (int i = 0; i < nslabs && ok; ++i) {
            const int s = i % STAGES, u = i / STAGES;
            ok = mbar_wait(full0 + 8 * s, u & 1);
            if (!ok) break;
            float4* head = reinterpret_cast<float4*>(gbase + (size_t)s * stage_bytes);
            float4* tail = head + BM * 128 / 16;
#pragma unroll 4
            for (int j = t; j < BM * 128 / 16; j += 128) {
                const float4 x = head[j];
                float4 h;
                h.x = __uint_as_float(__float_as_uint(x.x) & 0xFFFFE000u); h.y = __uint_as_float(__float_as_uint(x.y) & 0xFFFFE000u);
                h.z = __uint_as_float(__float_as_uint(x.z) & 0xFFFFE000u); h.w = __uint_as_float(__float_as_uint(x.w) & 0xFFFFE000u);
                head[j] = h;
                tail[j] = make_float4(x.x - h.x, x.y - h.y, x.z - h.z, x.w - h.w);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(ready0 + 8 * s);
        }
        if (ok) ok = mbar_wait(acc_full, 0);
        ok = __all_sync(0xffffffffu, ok);                         // tcgen05.ld below is warp-collective: decide as a warp
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int q = warp & 3;                               // a warp may only read its own quarter of the TMEM lanes
            const int64_t row = m0 + q * 32 + lane;
            float* crow = a.C + row * a.ldc;
            const bool vec_ok = (a.ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.C) & 15) == 0);
            const bool mvec_ok = a.mask && (a.ldm % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.mask) & 15) == 0);
            const float* mrow = a.mask ? a.mask + row * a.ldm : nullptr;
            for (int c0 = 0; c0 < a.n_pad; c0 += 16) {
                float mk[16];
                if (mrow && row < a.M) {                          // issued before the accumulator read so that both are in flight
                    if (mvec_ok && c0 + 16 <= a.N) {
#pragma unroll
                        for (int j = 0; j < 16; j += 4) {
                            const float4 m4 = __ldg(reinterpret_cast<const float4*>(mrow + c0 + j));
                            mk[j] = m4.x; mk[j + 1] = m4.y; mk[j + 2] = m4.z; mk[j + 3] = m4.w;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) mk[j] = c0 + j < a.N ? __ldg(mrow + c0 + j) : 0.f;
                    }
                }
                uint32_t r[16];
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                      "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                    : "r"(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)c0));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < a.M) {
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        v[j] = __uint_as_float(r[j]);
                        if (a.relu) v[j] = fmaxf(v[j], 0.f);
                        if (mrow && !(mk[j] > 0.f)) v[j] = 0.f;
                    }
                    if (vec_ok && c0 + 16 <= a.N) {
#pragma unroll
                        for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4*>(crow + c0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c0 + j < a.N) crow[c0 + j] = v[j];
                    }
                }
            }
        }
    }
    if (!ok) atomicExch(a.status, 1);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
}

// The same product with one CTA per SM walking over the row tiles (tile, tile + grid, ...): two accumulators in tensor
// memory (columns 0 and 256) and separate warps for the operand split and for the epilogue, so that tile t is read out
// of tensor memory and stored while tile t+1 is already being loaded, split and multiplied.
// Warps: 0 TMA, 1 MMA issue + tensor-memory allocation, 2-5 split A, 6-9 epilogue (warp w reads lane quarter w % 4).
constexpr int kThreadsPersistent = 320;

__global__ void __launch_bounds__(kThreadsPersistent, 1)
k_dense_nt_persistent(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmBh,
                      const __grid_constant__ CUtensorMap tmBt, const DenseArgs a, const int n_tiles)
{
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* gbase = smem_raw + (base - raw);
    const int b_bytes = a.n_pad * 128;
    const int stage_bytes = 2 * BM * 128 + 2 * b_bytes;
    const uint32_t bars = base + STAGES * stage_bytes;
    const uint32_t full0 = bars, ready0 = bars + 8 * STAGES, empty0 = bars + 16 * STAGES;
    const uint32_t acc_full0 = bars + 24 * STAGES, acc_empty0 = acc_full0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gbase + STAGES * stage_bytes + 24 * STAGES + 32);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nslabs = (a.K + BK - 1) / BK;
    constexpr int kTmemCols = 512;                                // two accumulators of up to 256 columns

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(ready0 + 8 * s, 128);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, 128);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {                                          // TMA producer: one ring of stages across all tiles
            int it = 0;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                for (int i = 0; i < nslabs; ++i, ++it) {
                    const int s = it % STAGES, u = it / STAGES;
                    if (u > 0) ok = mbar_wait(empty0 + 8 * s, (u - 1) & 1);
                    if (!ok) break;
                    const uint32_t st = base + s * stage_bytes;
                    mbar_expect_tx(full0 + 8 * s, BM * 128 + 2 * b_bytes);
                    tma_load_2d(st, &tmA, i * BK, tile * BM, full0 + 8 * s);
                    tma_load_2d(st + 2 * BM * 128, &tmBh, i * BK, 0, full0 + 8 * s);
                    tma_load_2d(st + 2 * BM * 128 + b_bytes, &tmBt, i * BK, 0, full0 + 8 * s);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                          // MMA issuer
            const uint32_t idesc = umma_idesc_tf32(a.n_pad);
            int it = 0, lt = 0;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++lt) {
                const int b = lt & 1, v = lt >> 1;
                if (lt >= 2) ok = mbar_wait(acc_empty0 + 8 * b, (v - 1) & 1);     // the epilogue has drained this accumulator
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem + (uint32_t)(b * 256);
                for (int i = 0; i < nslabs; ++i, ++it) {
                    const int s = it % STAGES, u = it / STAGES;
                    const uint32_t st = base + s * stage_bytes;
                    const uint64_t a_head = umma_desc_sw128(st), a_tail = umma_desc_sw128(st + BM * 128);
                    const uint64_t b_head = umma_desc_sw128(st + 2 * BM * 128), b_tail = umma_desc_sw128(st + 2 * BM * 128 + b_bytes);
                    if (a.raw_head == 2) {
                        // The tensor cores read a TF32 operand from a 32-bit container and ignore its low 13 bits, so the
                        // tile as TMA delivered it IS the head: both head passes go out as soon as the data has landed,
                        // and only the tail pass waits for the split warps.
                        ok = mbar_wait(full0 + 8 * s, u & 1);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                        for (int k = 0; k < BK / 8; ++k) {
                            umma_tf32(acc, a_head + 2 * k, b_tail + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                            umma_tf32(acc, a_head + 2 * k, b_head + 2 * k, idesc, 1u);
                        }
                        ok = mbar_wait(ready0 + 8 * s, u & 1);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                        for (int k = 0; k < BK / 8; ++k) umma_tf32(acc, a_tail + 2 * k, b_head + 2 * k, idesc, 1u);
                        umma_commit(empty0 + 8 * s);
                        continue;
                    }
                    ok = mbar_wait(ready0 + 8 * s, u & 1);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int k = 0; k < BK / 8; ++k) {
                        umma_tf32(acc, a_tail + 2 * k, b_head + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                        umma_tf32(acc, a_head + 2 * k, b_tail + 2 * k, idesc, 1u);
                        umma_tf32(acc, a_head + 2 * k, b_head + 2 * k, idesc, 1u);
                    }
                    umma_commit(empty0 + 8 * s);
                }
                if (ok) umma_commit(acc_full0 + 8 * b);
            }
        }
    } else if (warp < 6) {
        const int t = threadIdx.x - 64;                           // 0..127: split the A slab of every stage
        int it = 0;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            for (int i = 0; i < nslabs; ++i, ++it) {
                const int s = it % STAGES, u = it / STAGES;
                ok = mbar_wait(full0 + 8 * s, u & 1);
                if (!ok) break;
                float4* head = reinterpret_cast<float4*>(gbase + (size_t)s * stage_bytes);
                float4* tail = head + BM * 128 / 16;
#pragma unroll 4
                for (int j = t; j < BM * 128 / 16; j += 128) {
                    const float4 x = head[j];
                    float4 h;
                    h.x = __uint_as_float(__float_as_uint(x.x) & 0xFFFFE000u); h.y = __uint_as_float(__float_as_uint(x.y) & 0xFFFFE000u);
                    h.z = __uint_as_float(__float_as_uint(x.z) & 0xFFFFE000u); h.w = __uint_as_float(__float_as_uint(x.w) & 0xFFFFE000u);
                    if (!a.raw_head) head[j] = h;
                    tail[j] = make_float4(x.x - h.x, x.y - h.y, x.z - h.z, x.w - h.w);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(ready0 + 8 * s);
            }
        }
    } else {
        const int q = warp & 3;                                   // a warp may only read its own quarter of the TMEM lanes
        const bool vec_ok = (a.ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.C) & 15) == 0);
        const bool mvec_ok = a.mask && (a.ldm % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.mask) & 15) == 0);
        int lt = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++lt) {
            const int b = lt & 1, v = lt >> 1;
            ok = __all_sync(0xffffffffu, mbar_wait(acc_full0 + 8 * b, v & 1));     // tcgen05.ld is warp-collective
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int64_t row = (int64_t)tile * BM + q * 32 + lane;
            float* crow = a.C + row * a.ldc;
            const float* mrow = a.mask ? a.mask + row * a.ldm : nullptr;
            for (int c0 = 0; c0 < a.n_pad; c0 += 16) {
                float mk[16];
                if (mrow && row < a.M) {
                    if (mvec_ok && c0 + 16 <= a.N) {
#pragma unroll
                        for (int j = 0; j < 16; j += 4) {
                            const float4 m4 = __ldg(reinterpret_cast<const float4*>(mrow + c0 + j));
                            mk[j] = m4.x; mk[j + 1] = m4.y; mk[j + 2] = m4.z; mk[j + 3] = m4.w;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) mk[j] = c0 + j < a.N ? __ldg(mrow + c0 + j) : 0.f;
                    }
                }
                uint32_t r[16];
                tmem_ld16(tmem + (uint32_t)(b * 256) + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < a.M) {
                    float v16[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        v16[j] = __uint_as_float(r[j]);
                        if (a.relu) v16[j] = fmaxf(v16[j], 0.f);
                        if (mrow && !(mk[j] > 0.f)) v16[j] = 0.f;
                    }
                    if (vec_ok && c0 + 16 <= a.N) {
#pragma unroll
                        for (int j = 0; j < 16; j += 4)
                            __stcs(reinterpret_cast<float4*>(crow + c0 + j), make_float4(v16[j], v16[j + 1], v16[j + 2], v16[j + 3]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c0 + j < a.N) crow[c0 + j] = v16[j];
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(acc_empty0 + 8 * b);
        }
    }
    if (!ok) atomicExch(a.status, 1);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
}

__global__ void k_tf32_split(const float* __restrict__ src, float* __restrict__ head, float* __restrict__ tail, int64_t count)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float x = src[i];
    const float h = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
    head[i] = h;
    tail[i] = x - h;
}

}  // namespace

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled()
{
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// 2-D fp32 row-major matrix [rows x cols] with leading dimension ld, boxes of 32 columns x box_rows rows, 128B swizzle,
// out-of-range elements read as zero.
int make_map(CUtensorMap* map, const float* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows)
{
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return DG_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? DG_OK : DG_ERR_UNSUPPORTED;
}

int* dense_status_word()
{
    static int* word[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!word[dev]) {
        if (cudaMalloc((void**)&word[dev], sizeof(int)) != cudaSuccess) return nullptr;
        cudaMemset(word[dev], 0, sizeof(int));
    }
    return word[dev];
}

}  // namespace

extern "C" int dg_dense_split(const float* src, float* head, float* tail, int64_t count, void* stream)
{
    if (count < 0) return DG_ERR_DIMS;
    if (count == 0) return DG_OK;
    if (!src || !head || !tail) return DG_ERR_NULL;
    k_tf32_split<<<(unsigned)((count + 255) / 256), 256, 0, (cudaStream_t)stream>>>(src, head, tail, count);
    return (int)cudaGetLastError();
}

extern "C" int dg_dense_supported(int64_t M, int32_t N, int32_t K, int64_t lda, int64_t ldb, const void* A, const void* Bh, const void* Bt)
{
    if (M <= 0 || N <= 0 || K <= 0 || M >= ((int64_t)1 << 31)) return 0;
    if (lda % 4 || ldb % 4 || lda < K || ldb < K) return 0;                       // TMA strides are multiples of 16 bytes
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(Bh) | reinterpret_cast<uintptr_t>(Bt)) & 15) return 0;
    return encode_tiled() != nullptr;
}

extern "C" int dg_dense_nt(const float* A, int64_t lda, const float* Bt_head, const float* Bt_tail, int64_t ldb, float* C,
                           int64_t ldc, int64_t M, int32_t N, int32_t K, int32_t relu, void* stream)
{
    return dg_dense_nt_masked(A, lda, Bt_head, Bt_tail, ldb, C, ldc, M, N, K, relu, nullptr, 0, stream);
}

extern "C" int dg_dense_nt_masked(const float* A, int64_t lda, const float* Bt_head, const float* Bt_tail, int64_t ldb, float* C,
                                  int64_t ldc, int64_t M, int32_t N, int32_t K, int32_t relu, const float* mask, int64_t ldm,
                                  void* stream)
{
    if (!A || !Bt_head || !Bt_tail || !C) return DG_ERR_NULL;
    if (ldc < N || (mask && ldm < N)) return DG_ERR_DIMS;
    if (!dg_dense_supported(M, N, K, lda, ldb, A, Bt_head, Bt_tail)) return DG_ERR_UNSUPPORTED;
    if (N > 256) {      // a result wider than one accumulator: panels of 256 columns, A is streamed once per panel
        for (int32_t n0 = 0; n0 < N; n0 += 256) {
            const int rc = dg_dense_nt_masked(A, lda, Bt_head + (int64_t)n0 * ldb, Bt_tail + (int64_t)n0 * ldb, ldb, C + n0, ldc, M,
                                              N - n0 < 256 ? N - n0 : 256, K, relu, mask ? mask + n0 : nullptr, ldm, stream);
            if (rc) return rc;
        }
        return DG_OK;
    }
    DenseArgs a{};
    a.C = C; a.ldc = ldc; a.M = M; a.N = N; a.K = K; a.n_pad = (N + 15) / 16 * 16; a.relu = relu ? 1u : 0u;
    a.mask = mask; a.ldm = ldm;
    // Measured: the tensor cores ignore the low 13 bits of a TF32 operand (results with and without the masked head copy are
    // bit-identical), so the tile as loaded serves as head; issuing the head passes before the split is 4 % faster.
    a.raw_head = 2;
    a.status = dense_status_word();
    if (!a.status) return DG_ERR_STATE;
    CUtensorMap tmA, tmBh, tmBt;
    int rc;
    if ((rc = make_map(&tmA, A, M, K, lda, BM)) || (rc = make_map(&tmBh, Bt_head, N, K, ldb, a.n_pad)) ||
        (rc = make_map(&tmBt, Bt_tail, N, K, ldb, a.n_pad)))
        return rc;
    const size_t smem = (size_t)STAGES * (2 * BM * 128 + 2 * a.n_pad * 128) + 24 * STAGES + 48 + 1024;
    const int n_tiles = (int)((M + BM - 1) / BM);
    // two kernels: one tile per CTA, or one persistent CTA per SM walking the tiles
    // Narrow results leave room for two one-tile CTAs per SM, which overlap each other's load latency better than the
    // persistent CTA's two stages do (2,449,029 x 256 -> 47: 1.09 ms against 1.28 ms; -> 256: 2.16 against 1.88).
    const bool per_tile = a.n_pad <= 128;
    if (per_tile) {
        DG_CUDA(cudaFuncSetAttribute(k_dense_nt, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k_dense_nt<<<(unsigned)n_tiles, kThreads, smem, (cudaStream_t)stream>>>(tmA, tmBh, tmBt, a);
        return (int)cudaGetLastError();
    }
    int dev = 0, sms = 0;
    DG_CUDA(cudaGetDevice(&dev));
    DG_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    DG_CUDA(cudaFuncSetAttribute(k_dense_nt_persistent, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_dense_nt_persistent<<<(unsigned)(n_tiles < sms ? n_tiles : sms), kThreadsPersistent, smem, (cudaStream_t)stream>>>(tmA, tmBh, tmBt, a, n_tiles);
    return (int)cudaGetLastError();
}

extern "C" int dg_dense_status(int* host_status, void* stream)
{
    if (!host_status) return DG_ERR_NULL;
    int* w = dense_status_word();
    if (!w) return DG_ERR_STATE;
    DG_CUDA(cudaMemcpyAsync(host_status, w, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    DG_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return DG_OK;
}

extern "C" int dg_dense_status_reset(void* stream)
{
    int* w = dense_status_word();
    if (!w) return DG_ERR_STATE;
    DG_CUDA(cudaMemsetAsync(w, 0, sizeof(int), (cudaStream_t)stream));
    return DG_OK;
}

// Self-test of the give-up path every dense kernel shares: a CTA allocates tensor-memory columns as the kernels do, then
// waits - with a limit of a few thousand polls - on an mbarrier that nothing ever arrives at.  The wait runs out, the
// thread records it in `flag`, the CTA frees its tensor memory and the kernel returns normally.  Nothing traps or spins
// without bound; the context stays usable, which the caller can check by running a product afterwards.
namespace {
__global__ void __launch_bounds__(64, 1) k_dense_wait_selftest(int* flag, int limit)
{
    __shared__ __align__(8) unsigned long long bar_storage;
    __shared__ uint32_t tmem_slot;
    const uint32_t bar = smem_u32(&bar_storage);
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(32) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    if (threadIdx.x == 0 && !mbar_wait(bar, 0, limit)) atomicExch(flag, 1);      // nobody arrives: the wait must give up
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(32) : "memory");
}
}  // namespace

extern "C" int dg_dense_wait_selftest(int* host_gave_up, void* stream)
{
    if (!host_gave_up) return DG_ERR_NULL;
    int* flag = nullptr;
    DG_CUDA(cudaMalloc((void**)&flag, sizeof(int)));
    cudaError_t e = cudaMemsetAsync(flag, 0, sizeof(int), (cudaStream_t)stream);
    if (e == cudaSuccess) {
        k_dense_wait_selftest<<<1, 64, 0, (cudaStream_t)stream>>>(flag, 4096);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(host_gave_up, flag, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    cudaFree(flag);
    return (int)e;
}

// ---- weight-gradient product  D[Km x Nn] = X[n x Km]^T * G[n x Nn]  (models/gcn.py:50) -------------------------------------
// The reduction runs over the n rows of the block, so both operands are read "MN-major": a TMA box of 32 columns x 16
// rows lands as 16 rows of 128 bytes in the 32-byte-atom variant of the 128B swizzle, which is the one layout the tensor
// cores accept for 32-bit MN-major operands (the plain 128B swizzle makes them read zeros); the boxes of one operand lie
// 2048 bytes apart (leading byte offset), 4-row groups 512 bytes.  Each CTA streams a contiguous range
// of rows through a 3-stage ring, splits BOTH operands into TF32 head and tail in shared memory, accumulates the three
// passes into one or two 128 x Nn fp32 accumulators in tensor memory, and writes its partial D to scratch; a second
// kernel adds the partials of all CTAs in CTA order (deterministic).
namespace {

constexpr int TN_ROWS = 16;                     // rows of X / G per stage (two MMA k-steps of 8)
constexpr int TN_STAGES = 3;
constexpr int TN_BOX_BYTES = TN_ROWS * 128;     // one 32-column box

struct DenseTnArgs {
    float* partial;                             // [gridDim.x][m_halves][n_pad / 16][4][128][4], see tn_partial_index
    int64_t n;                                  // rows to reduce over
    int64_t rows_per_cta;                       // multiple of TN_ROWS
    int32_t Km, Nn, n_pad, m_halves;            // n_pad: Nn rounded up to 16; m_halves: 1 (Km <= 128) or 2
    int32_t flush_slabs;                        // slabs accumulated in tensor memory between two flushes
    int32_t raw_head;                           // as DenseArgs::raw_head
    int* status;
};

// Where element (m, c) of a CTA's partial D lives: the 128 rows of an accumulator half are the fastest index above a
// float4 of columns, so that a warp that holds 32 rows of tensor memory moves 512 contiguous bytes per access.
__host__ __device__ __forceinline__ int64_t tn_partial_index(int m, int c, int n_pad)
{
    return ((((int64_t)(m >> 7) * (n_pad >> 4) + (c >> 4)) * 4 + ((c & 15) >> 2)) * 128 + (m & 127)) * 4 + (c & 3);
}

// MN-major tile of 32-bit elements.  The tensor cores read such operands only in the "128B swizzle with 32-byte atoms"
// layout (32-byte chunks of a 128-byte row XOR-ed with the row index modulo 4), which TMA writes in its
// SWIZZLE_128B_ATOM_32B mode: 4-row groups are 512 bytes apart (stride byte offset), the 32-column boxes 2048 bytes
// (leading byte offset).
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(TN_BOX_BYTES >> 4) << 16;                 // leading byte offset: next 32 columns of M / N
    d |= (uint64_t)(512 >> 4) << 32;                          // stride byte offset: next 4 rows of K
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;                                   // layout type: SWIZZLE_128B_BASE32B
    return d;
}
__device__ __forceinline__ uint32_t umma_idesc_tf32_mn(int n_pad)
{
    return umma_idesc_tf32(n_pad) | (1u << 15) | (1u << 16);  // A and B are MN-major
}

__global__ void __launch_bounds__(kThreads, 1)
k_dense_tn(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmG, const DenseTnArgs a)
{
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* gbase = smem_raw + (base - raw);
    const int x_boxes = a.m_halves * 4;                           // 32-column boxes covering the (padded) Km
    const int g_boxes = (a.n_pad + 31) / 32;
    const int x_bytes = x_boxes * TN_BOX_BYTES, g_bytes = g_boxes * TN_BOX_BYTES;
    const int stage_bytes = 2 * x_bytes + 2 * g_bytes;            // X head, X tail, G head, G tail
    const uint32_t bars = base + TN_STAGES * stage_bytes;
    const uint32_t full0 = bars, ready0 = bars + 8 * TN_STAGES, empty0 = bars + 16 * TN_STAGES, acc_full = bars + 24 * TN_STAGES;
    const uint32_t acc_empty = acc_full + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gbase + TN_STAGES * stage_bytes + 24 * TN_STAGES + 16);
    const int T = a.flush_slabs;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r_begin = (int64_t)blockIdx.x * a.rows_per_cta;
    const int64_t r_end = min(r_begin + a.rows_per_cta, a.n);
    const int nslabs = r_end > r_begin ? (int)((r_end - r_begin + TN_ROWS - 1) / TN_ROWS) : 0;
    int tmem_cols = 32;
    while (tmem_cols < (a.m_halves == 2 ? 256 + a.n_pad : a.n_pad)) tmem_cols <<= 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TN_STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(ready0 + 8 * s, 128);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 128);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {                                          // TMA producer
            for (int i = 0; i < nslabs && ok; ++i) {
                const int s = i % TN_STAGES, u = i / TN_STAGES;
                if (u > 0) ok = mbar_wait(empty0 + 8 * s, (u - 1) & 1);
                if (!ok) break;
                const uint32_t st = base + s * stage_bytes;
                const int r0 = (int)(r_begin + (int64_t)i * TN_ROWS);
                mbar_expect_tx(full0 + 8 * s, x_bytes + g_bytes);
                for (int j = 0; j < x_boxes; ++j) tma_load_2d(st + j * TN_BOX_BYTES, &tmX, 32 * j, r0, full0 + 8 * s);
                for (int j = 0; j < g_boxes; ++j) tma_load_2d(st + 2 * x_bytes + j * TN_BOX_BYTES, &tmG, 32 * j, r0, full0 + 8 * s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                          // MMA issuer
            const uint32_t idesc = umma_idesc_tf32_mn(a.n_pad);
            for (int i = 0; i < nslabs && ok; ++i) {
                const int s = i % TN_STAGES, u = i / TN_STAGES;
                const int grp = i / T, in_grp = i % T;            // the accumulators restart with every flush group
                if (in_grp == 0 && grp > 0) ok = mbar_wait(acc_empty, (grp - 1) & 1);
                if (!ok) break;
                const uint32_t st = base + s * stage_bytes;
                const uint64_t g_head = umma_desc_mn_sw128(st + 2 * x_bytes), g_tail = umma_desc_mn_sw128(st + 2 * x_bytes + g_bytes);
                if (a.raw_head == 2) {
                    // the tiles as TMA delivered them serve as heads (the low 13 bits of a TF32 operand are ignored): the
                    // head x head pass does not wait for the split
                    ok = mbar_wait(full0 + 8 * s, u & 1);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    for (int h = 0; h < a.m_halves; ++h) {
                        const uint64_t x_head = umma_desc_mn_sw128(st + h * 4 * TN_BOX_BYTES);
#pragma unroll
                        for (int k = 0; k < TN_ROWS / 8; ++k)
                            umma_tf32(tmem + (uint32_t)(h * 256), x_head + (uint64_t)(k * (1024 >> 4)), g_head + (uint64_t)(k * (1024 >> 4)), idesc,
                                      (in_grp > 0 || k > 0) ? 1u : 0u);
                    }
                    ok = mbar_wait(ready0 + 8 * s, u & 1);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    for (int h = 0; h < a.m_halves; ++h) {
                        const uint64_t x_head = umma_desc_mn_sw128(st + h * 4 * TN_BOX_BYTES);
                        const uint64_t x_tail = umma_desc_mn_sw128(st + x_bytes + h * 4 * TN_BOX_BYTES);
#pragma unroll
                        for (int k = 0; k < TN_ROWS / 8; ++k) {
                            const uint64_t adv = (uint64_t)(k * (1024 >> 4));
                            umma_tf32(tmem + (uint32_t)(h * 256), x_tail + adv, g_head + adv, idesc, 1u);
                            umma_tf32(tmem + (uint32_t)(h * 256), x_head + adv, g_tail + adv, idesc, 1u);
                        }
                    }
                    umma_commit(empty0 + 8 * s);
                    if (in_grp == T - 1 || i == nslabs - 1) umma_commit(acc_full);
                    continue;
                }
                ok = mbar_wait(ready0 + 8 * s, u & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int h = 0; h < a.m_halves; ++h) {
                    const uint64_t x_head = umma_desc_mn_sw128(st + h * 4 * TN_BOX_BYTES);
                    const uint64_t x_tail = umma_desc_mn_sw128(st + x_bytes + h * 4 * TN_BOX_BYTES);
                    const uint32_t acc = tmem + (uint32_t)(h * 256);
#pragma unroll
                    for (int k = 0; k < TN_ROWS / 8; ++k) {       // one 8-row group (1024 bytes) per MMA
                        const uint64_t adv = (uint64_t)(k * (1024 >> 4));
                        umma_tf32(acc, x_tail + adv, g_head + adv, idesc, (in_grp > 0 || k > 0) ? 1u : 0u);
                        umma_tf32(acc, x_head + adv, g_tail + adv, idesc, 1u);
                        umma_tf32(acc, x_head + adv, g_head + adv, idesc, 1u);
                    }
                }
                umma_commit(empty0 + 8 * s);
                if (in_grp == T - 1 || i == nslabs - 1) umma_commit(acc_full);
            }
        }
    } else {
        const int t = threadIdx.x - 64;
        const int q = warp & 3;                                   // the quarter of the tensor-memory lanes this warp may read
        float4* part4 = reinterpret_cast<float4*>(a.partial + (size_t)blockIdx.x * a.m_halves * 128 * a.n_pad) + q * 32 + lane;
        for (int i = 0; i < nslabs && ok; ++i) {
            const int s = i % TN_STAGES, u = i / TN_STAGES;
            ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, u & 1));        // warp-uniform: tcgen05.ld below is .aligned
            if (!ok) break;
            unsigned char* st = gbase + (size_t)s * stage_bytes;
            for (int part = 0; part < 2; ++part) {                // X then G: head in place, tail behind it
                float4* head = reinterpret_cast<float4*>(st + (part ? 2 * x_bytes : 0));
                const int count = (part ? g_bytes : x_bytes) / 16;
                float4* tail = head + count;
                for (int j = t; j < count; j += 128) {
                    const float4 x = head[j];
                    float4 h;
                    h.x = __uint_as_float(__float_as_uint(x.x) & 0xFFFFE000u); h.y = __uint_as_float(__float_as_uint(x.y) & 0xFFFFE000u);
                    h.z = __uint_as_float(__float_as_uint(x.z) & 0xFFFFE000u); h.w = __uint_as_float(__float_as_uint(x.w) & 0xFFFFE000u);
                    if (!a.raw_head) head[j] = h;
                    tail[j] = make_float4(x.x - h.x, x.y - h.y, x.z - h.z, x.w - h.w);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(ready0 + 8 * s);
            if (i % T != T - 1 && i != nslabs - 1) continue;
            // Flush: the tensor cores add into their accumulator with truncation, an error that grows with the length
            // of the chain, so after T slabs the accumulators are added - rounded to nearest - into this CTA's partial
            // result (which stays in L2) and restart from zero.
            const int grp = i / T;
            ok = __all_sync(0xffffffffu, mbar_wait(acc_full, grp & 1));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int h = 0; h < a.m_halves; ++h) {
                for (int c0 = 0; c0 < a.n_pad; c0 += 32) {        // two 16-column reads in flight per wait
                    const int two = c0 + 16 < a.n_pad;            // warp-uniform
                    uint32_t r[32];
                    tmem_ld16(tmem + (uint32_t)(h * 256) + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
                    if (two) tmem_ld16(tmem + (uint32_t)(h * 256) + ((uint32_t)(q * 32) << 16) + (uint32_t)(c0 + 16), r + 16);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    float4* p = part4 + (size_t)(h * (a.n_pad >> 4) + (c0 >> 4)) * 4 * 128;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (j >= 4 && !two) break;
                        // Only this thread ever touches these 16 bytes, in program order, so the sum order is fixed; the
                        // reduction is sent to L2 and not waited for.
                        if (grp == 0)
                            __stcg(p + j * 128, make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                            __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
                        else
                            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p + j * 128), "f"(__uint_as_float(r[4 * j])),
                                         "f"(__uint_as_float(r[4 * j + 1])), "f"(__uint_as_float(r[4 * j + 2])), "f"(__uint_as_float(r[4 * j + 3]))
                                         : "memory");
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(acc_empty);
        }
        if (nslabs == 0) {                                        // a CTA without rows contributes zeros
            for (int j = 0; j < a.m_halves * a.n_pad / 4; ++j) __stcg(part4 + (size_t)j * 128, make_float4(0.f, 0.f, 0.f, 0.f));
        }
    }
    if (!ok) atomicExch(a.status, 1);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
}

// One thread per slot of the partial layout (coalesced over the CTAs' partials); slots of the padding are skipped.
__global__ void k_dense_tn_reduce(const float* __restrict__ partial, int n_parts, int64_t slots, float* __restrict__ D, int64_t ldd,
                                  int32_t Km, int32_t Nn, int32_t n_pad)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= slots) return;
    const int e = (int)(i & 3), r = (int)((i >> 2) & 127);
    const int64_t blk = i >> 9;                                   // (half, 16-column group, float4 within the group)
    const int j4 = (int)(blk & 3), c16 = (int)((blk >> 2) % (n_pad >> 4)), h = (int)((blk >> 2) / (n_pad >> 4));
    const int m = h * 128 + r, c = c16 * 16 + j4 * 4 + e;
    if (m >= Km || c >= Nn) return;
    float sum = 0.f;
    for (int p = 0; p < n_parts; ++p) sum += partial[(size_t)p * slots + i];
    D[(int64_t)m * ldd + c] = sum;
}

int make_map_box(CUtensorMap* map, const float* ptr, int64_t rows, int64_t cols, int64_t ld, int box_cols, int box_rows)
{
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return DG_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? DG_OK : DG_ERR_UNSUPPORTED;
}

}  // namespace

extern "C" int dg_dense_tn_supported(int64_t n, int32_t Km, int32_t Nn, int64_t ldx, int64_t ldg, const void* X, const void* G)
{
    if (n <= 0 || Km <= 0 || Nn <= 0 || n >= ((int64_t)1 << 31)) return 0;
    if (ldx % 4 || ldg % 4 || ldx < Km || ldg < Nn) return 0;
    if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(G)) & 15) return 0;
    return encode_tiled() != nullptr;
}

extern "C" int dg_dense_tn(const float* X, int64_t ldx, const float* G, int64_t ldg, float* D, int64_t ldd, int64_t n,
                           int32_t Km, int32_t Nn, float* scratch, int64_t scratch_floats, int32_t max_ctas, void* stream)
{
    if (!X || !G || !D || !scratch) return DG_ERR_NULL;
    if (ldd < Nn || max_ctas < 1 || (reinterpret_cast<uintptr_t>(scratch) & 15)) return DG_ERR_DIMS;
    if (!dg_dense_tn_supported(n, Km, Nn, ldx, ldg, X, G)) return DG_ERR_UNSUPPORTED;
    if (Km > 256 || Nn > 256) {     // wider than two accumulators: 256 x 256 panels of D, one after the other on the stream
        for (int32_t m0 = 0; m0 < Km; m0 += 256)                  // (they share `scratch`; the operands are streamed once per panel)
            for (int32_t c0 = 0; c0 < Nn; c0 += 256) {
                const int rc = dg_dense_tn(X + m0, ldx, G + c0, ldg, D + (int64_t)m0 * ldd + c0, ldd, n, Km - m0 < 256 ? Km - m0 : 256,
                                           Nn - c0 < 256 ? Nn - c0 : 256, scratch, scratch_floats, max_ctas, stream);
                if (rc) return rc;
            }
        return DG_OK;
    }
    DenseTnArgs a{};
    a.n = n; a.Km = Km; a.Nn = Nn; a.n_pad = (Nn + 15) / 16 * 16; a.m_halves = Km > 128 ? 2 : 1;
    const int64_t slabs = (n + TN_ROWS - 1) / TN_ROWS;
    const int ctas = (int)std::min<int64_t>(max_ctas, slabs);
    a.rows_per_cta = (slabs + ctas - 1) / ctas * TN_ROWS;
    const int64_t slots = (int64_t)a.m_halves * 128 * a.n_pad;    // one CTA's partial, padding included
    if (ctas * slots > scratch_floats) return DG_ERR_SCRATCH;
    a.raw_head = 1;     // no masked head copies (bit-identical results, fewer shared-memory writes); issuing head x head before the split is not faster here
    a.flush_slabs = 16;                                           // 256 rows = 96 tensor-core accumulations per chain
    a.partial = scratch;
    a.status = dense_status_word();
    if (!a.status) return DG_ERR_STATE;
    CUtensorMap tmX, tmG;
    int rc;
    if ((rc = make_map_box(&tmX, X, n, Km, ldx, 32, TN_ROWS)) || (rc = make_map_box(&tmG, G, n, Nn, ldg, 32, TN_ROWS))) return rc;
    const int x_bytes = a.m_halves * 4 * TN_BOX_BYTES, g_bytes = (a.n_pad + 31) / 32 * TN_BOX_BYTES;
    const size_t smem = (size_t)TN_STAGES * (2 * x_bytes + 2 * g_bytes) + 24 * TN_STAGES + 24 + 1024;
    DG_CUDA(cudaFuncSetAttribute(k_dense_tn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_dense_tn<<<ctas, kThreads, smem, (cudaStream_t)stream>>>(tmX, tmG, a);
    k_dense_tn_reduce<<<(unsigned)((slots + 255) / 256), 256, 0, (cudaStream_t)stream>>>(scratch, ctas, slots, D, ldd, Km, Nn, a.n_pad);
    return (int)cudaGetLastError();
}
