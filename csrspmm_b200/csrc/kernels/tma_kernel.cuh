// Merge-path kernel with B rows staged through shared memory by bulk asynchronous copies.
//
// Serves the reference's shared-memory entry points
// (src/device/csrspmm_warp_per_row_smem.cu:11-62, csrspmm_warp_per_row_smem_fp4.cu:11-84) and any
// wide dense operand.  The reference stages a whole row's (val, col) pairs per warp, which ties
// its shared-memory need to max_row_nnz and stops it launching beyond 1536 non-zeros per row
// (src/host/spmm_launcher.cu:112-120).  Here the merge-path tile bounds the staged (val, col)
// slice, and what flows through shared memory is the expensive operand: the gathered rows of B.
//
// Work split, shared-memory slice of A and the handling of split rows are those of the merge
// kernel.  The difference is the gather: every warp owns a ring of SLOTS row buffers.  One
// elected lane issues, per non-zero, one bulk copy global -> shared of the whole B row
// (Nd * 4 bytes, 16-byte aligned) that signals the slot's mbarrier with its byte count; all
// lanes wait on the barrier, read their float4 columns from the slot and multiply-add; the
// slot is re-armed for the non-zero SLOTS positions ahead.  SLOTS rows stay in flight per warp
// without holding them in registers.  Copies are plain CTA-local bulk copies (one destination
// CTA).  Every wait is bounded: when it gives up the warp stops issuing, reports
// kStatusWaitTimeout and drains what it had in flight with a second bounded wait.
#pragma once

#include "merge_kernel.cuh"

namespace csrspmm_b200 {

constexpr int kTmaWarps = kMergeThreads / 32;

__device__ __forceinline__ unsigned smem_u32(const void* p)
{
    return static_cast<unsigned>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity)
{
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// false when the limit was reached
__device__ __forceinline__ bool mbar_wait_bounded(unsigned bar, unsigned parity, unsigned limit = kWaitSpinLimit)
{
    for (unsigned spin = 0; spin < limit; ++spin)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// One row of B (bytes % 16 == 0, both addresses 16-byte aligned) into this CTA's shared memory.
__device__ __forceinline__ void bulk_copy_g2s(unsigned dst, const void* src, unsigned bytes, unsigned bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Static part of the shared memory.  The ring is dynamic: kTmaWarps * ring_stride bytes with
// ring_stride = max(SLOTS * slot_bytes, 512 * NV), so that a warp's ring can also hold the
// 32 * NV float4 of its partial sums once its copies have all been consumed.
template <int NV, int TG, int SLOTS>
struct TmaSmem {
    static constexpr int GROUPS = kTmaWarps;
    static constexpr int TILE = GROUPS * TG;
    static constexpr int ROWW = 32 * NV * 4;
    int rowend[TILE + 1];
    alignas(8) int2 cv[TILE];  // (column index, value bits) of each staged non-zero
    int coord[4];
    int tail_row[GROUPS];
    float* tail_ptr[GROUPS];  // each warp's partial-sum row lives in its own (by then idle) ring
    alignas(8) unsigned long long bar[GROUPS][SLOTS];
    __device__ __forceinline__ float* tail_of(int g) { return tail_ptr[g]; }
};

// NV float4 per lane cover the whole row (Nd <= 128 * NV), so there is a single column pass.
template <int NV, int TG, int SLOTS, int FMT>
__global__ void __launch_bounds__(kMergeThreads, CSRSPMM_TUNE_TMA_MINB) spmm_tma_kernel(const SpmmParams p, unsigned slot_bytes,
                                                                                         unsigned ring_stride)
{
    constexpr int G = 32, VW = 4;
    using Smem = TmaSmem<NV, TG, SLOTS>;
    __shared__ Smem s;
    extern __shared__ __align__(128) unsigned char ring[];

    const int g = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    unsigned char* my_ring = ring + (size_t)g * ring_stride;
    if (lane == 0) {
        s.tail_ptr[g] = reinterpret_cast<float*>(my_ring);
#pragma unroll
        for (int k = 0; k < SLOTS; ++k) mbar_init(smem_u32(&s.bar[g][k]), 1);
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    // the __syncthreads inside merge_tile_setup make the initialised barriers visible

    TileRange r;
    if (!merge_tile_setup<Smem, G, TG, FMT>(p, s, r)) return;

    const unsigned row_bytes = (unsigned)p.Nd * 4u;
    const unsigned ring_base = smem_u32(my_ring);
    const unsigned bar_base = smem_u32(&s.bar[g][0]);

    Vec<VW> acc[NV];
    Vec<VW> head[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        acc[v].zero();
        head[v].zero();
    }
    int i = r.il0;
    bool dirty = false;
    bool failed = false;

    auto finish_row = [&]() {
        if (i == r.il0) {
#pragma unroll
            for (int v = 0; v < NV; ++v) head[v] = acc[v];
        } else {
            store_row<G, NV, VW>(p, r.i0 + i, 0, lane, acc);
        }
#pragma unroll
        for (int v = 0; v < NV; ++v) acc[v].zero();
        dirty = false;
        ++i;
    };

    const int n = r.jl1 - r.jl0;
    int issued = 0;  // copies started (same value in every lane)
    if (lane == 0) {
        for (int k = 0; k < min(SLOTS, n); ++k) {
            const unsigned bar = bar_base + k * 8u;
            mbar_expect_tx(bar, row_bytes);
            bulk_copy_g2s(ring_base + k * slot_bytes, p.B + (long long)s.cv[r.jl0 + k].x * p.ldb, row_bytes, bar);
        }
    }
    issued = min(SLOTS, n);

    int k = 0;
    for (; k < n; ++k) {
        const int slot = k % SLOTS;
        const unsigned parity = (unsigned)(k / SLOTS) & 1u;
        // the vote keeps the warp together should the limit be hit by some lanes only
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar_base + slot * 8u, parity, p.wait_limit))) {
            failed = true;
            break;
        }
        const int jj = r.jl0 + k;
        while (jj >= s.rowend[i]) finish_row();
        const float a = __int_as_float(s.cv[jj].y);
        const float* srow = reinterpret_cast<const float*>(my_ring + (size_t)slot * slot_bytes);
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const int cv = lane + v * G;
            if (cv < p.ncolv) {
                Vec<VW> b;
                b.load(srow + cv * VW);
                acc[v].fma(a, b);
            }
        }
        dirty = true;
        __syncwarp();  // every lane has read the slot before it is overwritten
        if (k + SLOTS < n) {
            if (lane == 0) {
                fence_proxy_async_smem();
                const unsigned bar = bar_base + slot * 8u;
                mbar_expect_tx(bar, row_bytes);
                bulk_copy_g2s(ring_base + slot * slot_bytes,
                              p.B + (long long)s.cv[r.jl0 + k + SLOTS].x * p.ldb, row_bytes, bar);
            }
            ++issued;
        }
    }
    failed = __any_sync(0xffffffffu, failed);
    if (failed) {
        // drain: copies k .. issued-1 may still be landing in this CTA's shared memory; this wait keeps
        // the full limit whatever p.wait_limit is, so that no copy can arrive after the CTA has gone
        if (lane == 0) report_status(p, kStatusWaitTimeout);
        for (int q = k; q < issued; ++q) mbar_wait_bounded(bar_base + (q % SLOTS) * 8u, (unsigned)(q / SLOTS) & 1u);
        dirty = false;  // publish nothing from a failed range: no carry, and the held-back first row stays unwritten
    } else {
        while (i < r.il1) finish_row();
    }

    merge_tile_finish<Smem, G, NV, VW>(p, s, r, 0, g, lane, acc, head, dirty, failed);
}

}  // namespace csrspmm_b200
