// Column-panel pass of the tiled SpMM: the whole-row kernel restricted to one slab of B.
//
// No counterpart in the reference, whose kernels walk each row once over all of B
// (src/device/csrspmm_warp_per_row.cu:24-43).  When B is much larger than L2 and the rows are long,
// almost every one of those nnz row reads comes from HBM.  The tiled product instead goes through
// the columns of A in panels whose slab of B fits in L2: pass t handles, for every row, the stored
// entries from where pass t-1 stopped up to the first entry with col >= limit_t, so the slab is
// read from HBM once and from L2 for every further non-zero that names it.
//
// Nothing is re-ordered and nothing is searched for.  A per-row cursor (one int32) remembers where
// the previous pass stopped; a pass walks on from there in stored order and stops at the first
// column index that is not below its limit (the last pass has no limit).  With ascending columns
// each pass gets exactly its panel; with unsorted columns an entry is simply taken by the first
// pass that reaches it, so the product is right either way and only the locality suffers.  The
// running sums are carried between passes as raw fp32 accumulators (in C itself when beta == 0,
// in caller scratch otherwise, so that C_old survives to the end) and every output element still
// accumulates its products one by one in stored order: the result equals the whole-row kernel's,
// and the sequential oracle's, bit for bit.  A row with no entry in a middle panel is skipped
// without touching C.
#pragma once

#include <cooperative_groups.h>
#include <limits.h>

#include "common.cuh"
#include "row_kernel.cuh"
#include "tuning.h"

namespace csrspmm_b200 {

struct PanelPass {
    int* cursor;        // per row: first stored entry not consumed yet (written by every pass but the last)
    int col_limit;      // this pass stops a row at the first entry with col >= col_limit (INT_MAX: none)
    int first;          // no earlier pass: start at the row's beginning with zero sums
    int last;           // no later pass: apply alpha / beta and write C
    float* partial;     // raw running sums between passes
    long long ldp;
};

template <int G, int NV, int VW, int U, int FMT, int MINB>
__global__ void __launch_bounds__(kRowThreads, MINB) spmm_panel_kernel(const SpmmParams p, const PanelPass pp)
{
    constexpr int GROUPS = kRowThreads / G;
    constexpr unsigned kGroupMask = G == 32 ? 0xffffffffu : ((1u << G) - 1u);
    const cg::thread_block_tile<G> tile = cg::tiled_partition<G>(cg::this_thread_block());
    const int lane = tile.thread_rank();
    __shared__ int2 s_cv[kRowThreads];  // each group's current chunk of (col, val bits)
    int2* const my_cv = s_cv + (threadIdx.x / G) * G;
    const char* const b_lane = reinterpret_cast<const char*>(p.B) + (size_t)lane * (VW * 4);
    const unsigned long long b_policy = make_b_policy();

    const long long group_stride = (long long)gridDim.x * GROUPS;
    for (long long row_ll = (long long)blockIdx.x * GROUPS + (threadIdx.x / G); row_ll < p.M; row_ll += group_stride) {
        const int row = (int)row_ll;
        // clamped so that a malformed row_ptr or cursor cannot index outside col_idx/values
        const int row_lo = max(__ldg(p.row_ptr + row) - p.rp_base, 0);
        const int re = min(__ldg(p.row_ptr + row + 1) - p.rp_base, p.nnz);
        int rs = row_lo;
        if (!pp.first) rs = max(pp.cursor[row], row_lo);

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
        // how many entries at the head of the chunk that starts at `base` belong to this pass
        auto leading = [&](int base, int c) -> int {
            const bool mine = (base + lane < re) && (c < pp.col_limit);
            const unsigned stop = ~tile.ballot(mine) & kGroupMask;
            return stop ? (__ffs(stop) - 1) : G;
        };

        int c_first;
        float a_first;
        load_pair(rs + lane, c_first, a_first);
        const int n_first = leading(rs, c_first);
        if (n_first == 0 && !pp.first && !pp.last) continue;  // nothing of this row in the panel

        int end = rs;
        for (int cb = 0; cb < p.ncolv; cb += G * NV) {
            const char* const b_pass = b_lane + (size_t)cb * (VW * 4);
            bool col_ok[NV];
#pragma unroll
            for (int v = 0; v < NV; ++v) col_ok[v] = cb + lane + v * G < p.ncolv;
            Vec<VW> acc[NV];
#pragma unroll
            for (int v = 0; v < NV; ++v) {
                acc[v].zero();
                if (!pp.first && col_ok[v])
                    acc[v].load(pp.partial + (long long)row * pp.ldp + (long long)(cb + lane + v * G) * VW);
            }

            auto load_b = [&](Vec<VW> (&dst)[NV], int col) {
                const char* brow = b_pass + (unsigned long long)(unsigned)col * p.ldb_bytes;
#pragma unroll
                for (int v = 0; v < NV; ++v) {
                    if (col_ok[v]) dst[v].load_b(reinterpret_cast<const float*>(brow + v * (G * VW * 4)), b_policy);
                    else dst[v].zero();
                }
            };

            int base = rs;
            int c_cur = c_first;
            float a_cur = a_first;
            int n = n_first;  // a further column pass walks the same entries again
            while (n > 0) {
                tile.sync();  // the previous chunk has been consumed by every lane of the group
                my_cv[lane] = make_int2(c_cur, __float_as_int(a_cur));
                tile.sync();
                int c_nx = 0;
                float a_nx = 0.f;
                if (n == G) load_pair(base + G + lane, c_nx, a_nx);  // requested ahead; needed if this chunk is taken whole
                int t = 0;
                for (; t + U <= n; t += U) {  // whole batches: no per-element test
                    Vec<VW> bq[U][NV];
#pragma unroll
                    for (int u = 0; u < U; ++u) load_b(bq[u], my_cv[t + u].x);
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const float a = __int_as_float(my_cv[t + u].y);
#pragma unroll
                        for (int v = 0; v < NV; ++v) acc[v].fma(a, bq[u][v]);
                    }
                }
                if (t < n) {  // the last, partial batch
                    Vec<VW> bq[U][NV];
#pragma unroll
                    for (int u = 0; u < U; ++u)
                        if (t + u < n) load_b(bq[u], my_cv[t + u].x);
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        if (t + u < n) {
                            const float a = __int_as_float(my_cv[t + u].y);
#pragma unroll
                            for (int v = 0; v < NV; ++v) acc[v].fma(a, bq[u][v]);
                        }
                    }
                }
                base += n;
                if (n < G) break;
                c_cur = c_nx;
                a_cur = a_nx;
                n = leading(base, c_cur);
            }
            end = base;

            if (pp.last) {
                store_row<G, NV, VW>(p, row, cb, lane, acc);
            } else {
#pragma unroll
                for (int v = 0; v < NV; ++v)
                    if (col_ok[v])
                        acc[v].store(pp.partial + (long long)row * pp.ldp + (long long)(cb + lane + v * G) * VW);
            }
        }
        if (!pp.last && lane == 0) pp.cursor[row] = end;
    }
}

}  // namespace csrspmm_b200
