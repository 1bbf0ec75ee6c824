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
#include "tuning.h"

namespace csrspmm_b200 {

namespace cg = cooperative_groups;

constexpr int kRowThreads = CSRSPMM_TUNE_ROW_THREADS;

// FULL: one pass covers the row exactly (G * NV == ncolv), so no column guard is compiled in.
// MINB: resident CTAs per SM asked of the compiler (caps the registers).
template <int G, int NV, int VW, int U, int FMT, bool FULL, int MINB>
__global__ void __launch_bounds__(kRowThreads, MINB) spmm_row_kernel(const SpmmParams p)
{
    constexpr int GROUPS = kRowThreads / G;
    const cg::thread_block_tile<G> tile = cg::tiled_partition<G>(cg::this_thread_block());
    const int lane = tile.thread_rank();
    // rows are dealt to the groups of the grid round-robin; with one CTA per GROUPS rows (the
    // default grid) every group gets exactly one row
    const long long group_stride = (long long)gridDim.x * GROUPS;
    for (long long row_ll = (long long)blockIdx.x * GROUPS + (threadIdx.x / G); row_ll < p.M; row_ll += group_stride) {
    const int row = (int)row_ll;

    // clamped so that a malformed row_ptr cannot index outside col_idx/values
    const int rs = max(__ldg(p.row_ptr + row) - p.rp_base, 0);
    const int re = min(__ldg(p.row_ptr + row + 1) - p.rp_base, p.nnz);
    const char* const b_lane = reinterpret_cast<const char*>(p.B) + (size_t)lane * (VW * 4);
    const unsigned long long b_policy = make_b_policy();
#if CSRSPMM_TUNE_ROW_STAGE_SMEM
    __shared__ int2 s_cv[kRowThreads];  // each group's current chunk of (col, val bits)
    int2* const my_cv = s_cv + (threadIdx.x / G) * G;
#endif

    for (int cb = 0; cb < p.ncolv; cb += G * NV) {
        const char* const b_pass = b_lane + (size_t)cb * (VW * 4);
        bool col_ok[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) col_ok[v] = FULL || (cb + lane + v * G < p.ncolv);
        Vec<VW> acc[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) acc[v].zero();

        auto load_b = [&](Vec<VW> (&dst)[NV], int col) {
            const char* brow = b_pass + (unsigned long long)(unsigned)col * p.ldb_bytes;
#pragma unroll
            for (int v = 0; v < NV; ++v) {
                if (col_ok[v]) dst[v].load_b(reinterpret_cast<const float*>(brow + v * (G * VW * 4)), b_policy);
                else dst[v].zero();
            }
        };

        // (col, val) of the row, G at a time: the next chunk is requested before the current one is
        // consumed, so its latency overlaps the multiply-adds
        auto load_pair = [&](int jj, int& c, float& a) {
            c = 0;
            a = 0.f;
            if (jj < re) {
                c = __ldcs(p.col_idx + jj);
                a = load_value<FMT>(p.values, jj, p.value_scale);
                if ((unsigned)c >= (unsigned)p.Kd) {  // never fault on a bad index
                    c = min(max(c, 0), p.Kd - 1);
                    report_status(p, kStatusColClamped);
                }
            }
        };
        int c_next;
        float a_next;
        load_pair(rs + lane, c_next, a_next);
        for (int base = rs; base < re; base += G) {
#if CSRSPMM_TUNE_ROW_STAGE_SMEM
            tile.sync();  // the previous chunk has been consumed by every lane of the group
            my_cv[lane] = make_int2(c_next, __float_as_int(a_next));
            tile.sync();
#define ROW_COL(k) (my_cv[(k)].x)
#define ROW_VAL(k) (__int_as_float(my_cv[(k)].y))
#else
            const int c_l = c_next;
            const float a_l = a_next;
#define ROW_COL(k) (tile.shfl(c_l, (k)))
#define ROW_VAL(k) (tile.shfl(a_l, (k)))
#endif
            load_pair(base + G + lane, c_next, a_next);
            const int n = min(G, re - base);
            int t = 0;
            for (; t + U <= n; t += U) {  // whole batches: no per-element test
                Vec<VW> bq[U][NV];
#pragma unroll
                for (int u = 0; u < U; ++u) load_b(bq[u], ROW_COL(t + u));
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const float a = ROW_VAL(t + u);
#pragma unroll
                    for (int v = 0; v < NV; ++v) acc[v].fma(a, bq[u][v]);
                }
            }
            if (t < n) {  // the last, partial batch
                Vec<VW> bq[U][NV];
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (t + u < n) load_b(bq[u], ROW_COL(t + u));
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (t + u < n) {
                        const float a = ROW_VAL(t + u);
#pragma unroll
                        for (int v = 0; v < NV; ++v) acc[v].fma(a, bq[u][v]);
                    }
                }
            }
#undef ROW_COL
#undef ROW_VAL
        }
        store_row<G, NV, VW>(p, row, cb, lane, acc);
    }
    }
}

}  // namespace csrspmm_b200
