// Row kernel: one lane group per row of A.
//
// Serves the reference's whole-row kernels (src/device/csrspmm_naive.cu:11-39,
// csrspmm_warp_per_row.cu:13-48, csrspmm_warp_per_row_fp4.cu:9-65) on matrices whose rows are
// short and even.  A group of G lanes owns one row (G = 8/16 puts 4/2 rows in a warp when the
// dense width is small); each lane keeps NV column vectors, so the row's (col, val) pairs are
// walked once per G*NV*VW columns instead of once per 32 columns.  The group loads G pairs
// with one coalesced access, then broadcasts them lane to lane and keeps U B-row loads in
// flight before the dependent FMAs.  Each output still accumulates its products one after the
// other in stored order, so results equal the sequential fp32 oracle bit for bit.
#pragma once

#include <cooperative_groups.h>

#include "common.cuh"

namespace csrspmm_b200 {

namespace cg = cooperative_groups;

constexpr int kRowThreads = 256;

template <int G, int NV, int VW, int U, int FMT>
__global__ void __launch_bounds__(kRowThreads) spmm_row_kernel(const SpmmParams p)
{
    constexpr int GROUPS = kRowThreads / G;
    const cg::thread_block_tile<G> tile = cg::tiled_partition<G>(cg::this_thread_block());
    const int lane = tile.thread_rank();
    const long long row_ll = (long long)blockIdx.x * GROUPS + (threadIdx.x / G);
    if (row_ll >= p.M) return;
    const int row = (int)row_ll;

    // clamped so that a malformed row_ptr cannot index outside col_idx/values
    const int rs = max(__ldg(p.row_ptr + row), 0);
    const int re = min(__ldg(p.row_ptr + row + 1), p.nnz);

    for (int cb = 0; cb < p.ncolv; cb += G * NV) {
        Vec<VW> acc[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) acc[v].zero();

        for (int base = rs; base < re; base += G) {
            const int jj = base + lane;
            int c_l = 0;
            float a_l = 0.f;
            if (jj < re) {
                c_l = __ldcs(p.col_idx + jj);
                a_l = load_value<FMT>(p.values, jj, p.value_scale);
                if ((unsigned)c_l >= (unsigned)p.Kd) {  // never fault on a bad index
                    c_l = min(max(c_l, 0), p.Kd - 1);
                    report_status(p, kStatusColClamped);
                }
            }
            const int n = min(G, re - base);
            for (int t = 0; t < n; t += U) {
                Vec<VW> bq[U][NV];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (t + u < n) {
                        const int c = tile.shfl(c_l, t + u);
                        const float* brow = p.B + (long long)c * p.ldb;
#pragma unroll
                        for (int v = 0; v < NV; ++v) {
                            const int cv = cb + lane + v * G;
                            if (cv < p.ncolv) bq[u][v].load_nc(brow + (long long)cv * VW);
                            else bq[u][v].zero();
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (t + u < n) {
                        const float a = tile.shfl(a_l, t + u);
#pragma unroll
                        for (int v = 0; v < NV; ++v) acc[v].fma(a, bq[u][v]);
                    }
                }
            }
        }
        store_row<G, NV, VW>(p, row, cb, lane, acc);
    }
}

}  // namespace csrspmm_b200
