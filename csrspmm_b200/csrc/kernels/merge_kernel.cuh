// Merge-path kernel: equal shares of (rows + non-zeros) per CTA and per lane group.
//
// Serves every entry point of the reference on matrices whose rows are long or uneven, where a
// whole-row mapping (src/device/csrspmm_warp_per_row.cu:24-43: one warp walks one row from start
// to end) leaves most of the chip waiting for the longest row.
//
// The list of row ends (row_ptr[1..M]) is merged with the list of non-zero positions
// (0..nnz-1); consuming a row end means "row finished, write it", consuming a position means
// "one multiply-add per output column".  Diagonal d of that merge is found by binary search,
// so CTA t owns items [t*TILE, (t+1)*TILE) and lane group g of the CTA owns TG of them, whatever
// the row lengths are.
//
//   1. two warps search the CTA's two diagonals in row_ptr (32 probes per step);
//   2. the CTA copies its slice of row ends, column indices and (decoded) values to shared
//      memory with coalesced loads;
//   3. each group finds its own sub-range in shared memory and walks it: U B-row loads in
//      flight per lane, FMAs in stored order, a row written when its end is passed;
//   4. a row that several groups of the CTA worked on is summed through shared memory (the
//      group that passes its end holds the write back until the others have published their
//      partial sums), so rows inside one CTA never touch global scratch;
//   5. the one row a CTA leaves unfinished goes to carry_row/carry_val[blockIdx.x]; the fix-up
//      kernel adds those to C in tile order.  No atomics: the result is the same on every run.
//
// A row that lies inside one group's range is accumulated sequentially and matches the oracle
// bit for bit; a split row is a fixed-order sum of sequential partial sums.
#pragma once

#include <limits.h>

#include "common.cuh"
#include "tuning.h"

namespace csrspmm_b200 {

constexpr int kMergeThreads = CSRSPMM_TUNE_MERGE_THREADS;

// First i in [max(0, d-nnz), min(d, M)] with row_end[i] > d - i - 1; then j = d - i positions
// precede the diagonal.  Cooperative over one full warp: 32 probes per round.
__device__ __forceinline__ int merge_search_warp(long long d, const int* __restrict__ row_end, int rp_base,
                                                 int M, int nnz, int lane)
{
    int lo = (int)max(0LL, d - (long long)nnz);
    int hi = (int)min(d, (long long)M);
    while (lo < hi) {
        const int span = hi - lo;
        const int step = (span + 31) / 32;
        const long long mid = (long long)lo + (long long)lane * step;
        bool pred = false;
        if (mid < hi) pred = ((long long)__ldg(row_end + mid) - rp_base <= d - mid - 1);
        const int t = __popc(__ballot_sync(0xffffffffu, pred));
        if (t == 0) {
            hi = lo;
        } else {
            const long long first_false = (long long)lo + (long long)t * step;
            lo = lo + (t - 1) * step + 1;
            hi = (int)min((long long)hi, first_false);
            if (hi < lo) hi = lo;  // only reachable when row_ptr is not monotone
        }
    }
    return lo;
}

// Same search inside the CTA's shared-memory slice (local coordinates).
__device__ __forceinline__ int merge_search_local(int d, const int* s_rowend, int nrows, int nnzt)
{
    int lo = max(0, d - nnzt);
    int hi = min(d, nrows);
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (s_rowend[mid] <= d - mid - 1) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}

template <int G, int NV, int VW, int TG>
struct MergeSmem {
    static constexpr int GROUPS = kMergeThreads / G;
    static constexpr int TILE = GROUPS * TG;
    static constexpr int ROWW = G * NV * VW;  // floats one group holds per pass
    int rowend[TILE + 1];
    alignas(8) int2 cv[TILE];  // (column index, value bits) of each staged non-zero
    int coord[4];
    int tail_row[GROUPS];
    unsigned longbits[TILE / 32 + 1];  // SKIP only: bit k = local row k is left to the scheduled pieces
    alignas(16) float tail[GROUPS][ROWW];
    __device__ __forceinline__ float* tail_of(int g) { return tail[g]; }
    __device__ __forceinline__ bool is_long(int k) const { return (longbits[k >> 5] >> (k & 31)) & 1u; }
};

// Where a lane group's share of the tile starts and ends, in tile-local coordinates.
struct TileRange {
    int i0, j0;      // global row / non-zero position where the tile starts
    int nrows;       // row ends inside the tile
    int nnzt;        // non-zeros inside the tile
    int il0, jl0;    // the group's start (local row, local non-zero)
    int il1, jl1;    // the group's end
};

// Steps 1-3.  Returns false (for every thread of the CTA) when there is nothing for the CTA to do: row_ptr
// is inconsistent, or (SKIP) the tile lies inside one scheduled row.
// SKIP: rows of p.skip_len entries or more belong to the scheduled pieces; they are marked in
// s.longbits and 32-entry runs that lie wholly inside such a row are not fetched.
template <class Smem, int G, int TG, int FMT, bool SKIP = false>
__device__ __forceinline__ bool merge_tile_setup(const SpmmParams& p, Smem& s, TileRange& r)
{
    constexpr int TILE = Smem::TILE;
    constexpr int SB = CSRSPMM_TUNE_MERGE_STAGE_BATCH;
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int* __restrict__ row_end = p.row_ptr + 1;

    // ---- 1. the CTA's two diagonals --------------------------------------------------------
    const long long d0 = (long long)blockIdx.x * TILE;
    const long long d1 = min(d0 + (long long)TILE, p.num_items);
    if (warp < 2) {
        const long long d = warp == 0 ? d0 : d1;
        const int i = merge_search_warp(d, row_end, p.rp_base, p.M, p.nnz, tid & 31);
        if ((tid & 31) == 0) {
            s.coord[warp * 2] = i;
            s.coord[warp * 2 + 1] = (int)(d - i);
        }
    }
    __syncthreads();
    r.i0 = s.coord[0];
    r.j0 = s.coord[1];
    r.nrows = s.coord[2] - r.i0;
    r.nnzt = s.coord[3] - r.j0;
    if (r.nrows < 0 || r.nnzt < 0 || r.nrows + r.nnzt > TILE) {  // malformed row_ptr: touch nothing
        if (tid == 0) {
            report_status(p, kStatusBadTile);
            p.carry_row[blockIdx.x] = -1;
        }
        return false;
    }

    // ---- 2. stage the slice ----------------------------------------------------------------
    // SB global loads in flight per thread and list, then the stores to shared memory: a load-store
    // pair per iteration would make the staging a chain of TILE / kMergeThreads round trips to memory.
    auto clamp_col = [&](int c) {
        if ((unsigned)c >= (unsigned)p.Kd) {  // never fault on a bad index
            c = min(max(c, 0), p.Kd - 1);
            report_status(p, kStatusColClamped);
        }
        return c;
    };
    if constexpr (SKIP) {
        for (int k0 = warp * 32; k0 <= r.nrows; k0 += kMergeThreads * SB) {  // whole warps: one flag word each
            int end[SB], beg[SB];
#pragma unroll
            for (int b = 0; b < SB; ++b) {
                const long long gi = (long long)r.i0 + k0 + b * kMergeThreads + (tid & 31);
                const bool live = k0 + b * kMergeThreads + (tid & 31) <= r.nrows && gi < p.M;
                end[b] = live ? __ldg(row_end + gi) : 0;
                beg[b] = live ? __ldg(p.row_ptr + gi) : 0;
            }
#pragma unroll
            for (int b = 0; b < SB; ++b) {
                const int kw = k0 + b * kMergeThreads;  // the same for the whole warp
                if (kw <= r.nrows) {
                    const int k = kw + (tid & 31);
                    if (k <= r.nrows) s.rowend[k] = (k < r.nrows) ? (end[b] - p.rp_base - r.j0) : INT_MAX;
                    const unsigned bits = __ballot_sync(0xffffffffu, end[b] - beg[b] >= p.skip_len);
                    if ((tid & 31) == 0) s.longbits[kw >> 5] = bits;
                }
            }
        }
        __syncthreads();
        if (r.nrows == 0 && s.is_long(0)) {  // the whole tile lies inside one scheduled row: nothing to do here
            if (tid == 0) p.carry_row[blockIdx.x] = -1;
            return false;
        }
        for (int k0 = tid; k0 < r.nnzt; k0 += kMergeThreads * SB) {
            int c[SB];
            float a[SB];
            bool fetch[SB];
#pragma unroll
            for (int b = 0; b < SB; ++b) {
                const int k = k0 + b * kMergeThreads;
                fetch[b] = k < r.nnzt;
                if (fetch[b]) {
                    // the row that holds the first entry of this warp's run of 32
                    const int run = k & ~31;
                    int lo = 0, hi = r.nrows;
                    while (lo < hi) {
                        const int mid = (lo + hi) >> 1;
                        if (s.rowend[mid] <= run) lo = mid + 1;
                        else hi = mid;
                    }
                    if (s.is_long(lo) && s.rowend[lo] >= min(run + 32, r.nnzt)) {
                        s.cv[k] = make_int2(0, 0);  // never read as data, but a batch may gather row 0 of B for it
                        fetch[b] = false;
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < SB; ++b) {
                if (fetch[b]) {
                    const int k = k0 + b * kMergeThreads;
                    c[b] = __ldcs(p.col_idx + r.j0 + k);
                    a[b] = load_value<FMT>(p.values, r.j0 + k, p.value_scale);
                }
            }
#pragma unroll
            for (int b = 0; b < SB; ++b)
                if (fetch[b]) s.cv[k0 + b * kMergeThreads] = make_int2(clamp_col(c[b]), __float_as_int(a[b]));
        }
    } else {
        // row ends and entries are independent lists: both requested before either is stored
        for (int k0 = tid; k0 <= r.nrows || k0 < r.nnzt; k0 += kMergeThreads * SB) {
            int end[SB], c[SB];
            float a[SB];
#pragma unroll
            for (int b = 0; b < SB; ++b) {
                const int k = k0 + b * kMergeThreads;
                if (k < r.nrows) end[b] = __ldg(row_end + r.i0 + k);
                if (k < r.nnzt) {
                    c[b] = __ldcs(p.col_idx + r.j0 + k);
                    a[b] = load_value<FMT>(p.values, r.j0 + k, p.value_scale);
                }
            }
#pragma unroll
            for (int b = 0; b < SB; ++b) {
                const int k = k0 + b * kMergeThreads;
                if (k <= r.nrows) s.rowend[k] = (k < r.nrows) ? (end[b] - p.rp_base - r.j0) : INT_MAX;
                if (k < r.nnzt) s.cv[k] = make_int2(clamp_col(c[b]), __float_as_int(a[b]));
            }
        }
    }
    __syncthreads();

    // ---- 3. the group's own range ----------------------------------------------------------
    const int g = tid / G;
    const int total = r.nrows + r.nnzt;
    const int dl0 = min(g * TG, total);
    const int dl1 = min(dl0 + TG, total);
    r.il0 = merge_search_local(dl0, s.rowend, r.nrows, r.nnzt);
    r.jl0 = dl0 - r.il0;
    r.il1 = merge_search_local(dl1, s.rowend, r.nrows, r.nnzt);
    r.jl1 = dl1 - r.il1;
    return true;
}

// Step 5 for CTAs of many small lane groups (more than 32 of them): a tile inside a long row leaves
// one partial sum per group, and one thread adding them all is the longest chain of the tile.  The
// CTA's last warp does it: it finds the run of groups that stopped inside the open row 32 groups
// per vote, cuts the run into 32 / (G * NV) contiguous chunks, every lane adds one chunk for one
// column vector in group order, and the chunk sums are added in chunk order.  A fixed order, so the
// carry is the same on every run.
template <class Smem, int G, int NV, int VW>
__device__ __forceinline__ void merge_carry_by_warp(const SpmmParams& p, Smem& s, const TileRange& r, int cb)
{
    constexpr int GROUPS = Smem::GROUPS;
    constexpr int POS = G * NV;       // column vectors one group holds per pass
    constexpr int CHUNKS = 32 / POS;
    static_assert(GROUPS % 32 == 0 && POS <= 32 && 32 % POS == 0, "merge_carry_by_warp: lane groups must tile a warp");
    const int wl = threadIdx.x & 31;

    int gs = 0;
    for (int base = GROUPS - 32; base >= 0; base -= 32) {
        const unsigned open = __ballot_sync(0xffffffffu, s.tail_row[base + wl] == r.nrows);
        const int lead = __clz((int)~open);  // groups at the top of these 32 that belong to the run
        if (lead < 32) {
            gs = base + 32 - lead;
            break;
        }
    }
    if (wl == 0 && cb == 0) p.carry_row[blockIdx.x] = (gs < GROUPS) ? (r.i0 + r.nrows) : -1;
    if (gs >= GROUPS) return;

    const int pos = wl % POS;
    const int chunk = wl / POS;
    const int per = (GROUPS - gs + CHUNKS - 1) / CHUNKS;
    const int q0 = gs + chunk * per;
    const int q1 = min(q0 + per, GROUPS);
    Vec<VW> sum;
    sum.zero();
    if (q0 < q1) {
        sum.load(s.tail_of(q0) + pos * VW);
        for (int q = q0 + 1; q < q1; ++q) {
            Vec<VW> t;
            t.load(s.tail_of(q) + pos * VW);
            sum.add(t);
        }
    }
    Vec<VW> total = sum;  // chunk 0 is never empty
    for (int c = 1; c < CHUNKS; ++c) {
        const Vec<VW> t = sum.shuffle(c * POS + pos);
        if (gs + c * per < GROUPS) total.add(t);
    }
    const int cv = cb + pos;
    if (chunk == 0 && cv < p.ncolv) total.store(p.carry_val + (long long)blockIdx.x * p.carry_ld + (long long)cv * VW);
}

// Steps 4-5 for one column pass.  acc = the group's unfinished partial sum (valid when dirty),
// head = its held-back first finished row (valid when il1 > il0).  Contains one __syncthreads.
// head_skip: the group's first finished row belongs to the scheduled pieces and is not written.
template <class Smem, int G, int NV, int VW>
__device__ __forceinline__ void merge_tile_finish(const SpmmParams& p, Smem& s, const TileRange& r,
                                                  int cb, int g, int lane, const Vec<VW> (&acc)[NV],
                                                  Vec<VW> (&head)[NV], bool dirty, bool head_skip = false)
{
    constexpr int GROUPS = Smem::GROUPS;
    // ---- 4. rows shared between groups of this CTA -------------------------------------------
    if (lane == 0) s.tail_row[g] = dirty ? r.il1 : -1;
    if (dirty) {
#pragma unroll
        for (int v = 0; v < NV; ++v) acc[v].store(s.tail_of(g) + (lane + v * G) * VW);
    }
    __syncthreads();

    if (r.il1 > r.il0 && !head_skip) {
        // earlier groups' partial sums of my first row, oldest first, then my own part
        int gs = g;
        while (gs > 0 && s.tail_row[gs - 1] == r.il0) --gs;
        if (gs < g) {
            Vec<VW> sum[NV];
#pragma unroll
            for (int v = 0; v < NV; ++v) sum[v].load(s.tail_of(gs) + (lane + v * G) * VW);
            for (int q = gs + 1; q < g; ++q) {
#pragma unroll
                for (int v = 0; v < NV; ++v) {
                    Vec<VW> t;
                    t.load(s.tail_of(q) + (lane + v * G) * VW);
                    sum[v].add(t);
                }
            }
#pragma unroll
            for (int v = 0; v < NV; ++v) {
                sum[v].add(head[v]);
                head[v] = sum[v];
            }
        }
        store_row<G, NV, VW>(p, r.i0 + r.il0, cb, lane, head);
    }

    // ---- 5. the row this CTA leaves unfinished ------------------------------------------------
    if constexpr (GROUPS > 32) {
        if (threadIdx.x >= kMergeThreads - 32) merge_carry_by_warp<Smem, G, NV, VW>(p, s, r, cb);
    } else if (g == GROUPS - 1) {
        int gs = GROUPS;
        while (gs > 0 && s.tail_row[gs - 1] == r.nrows) --gs;
        if (lane == 0 && cb == 0) p.carry_row[blockIdx.x] = (gs < GROUPS) ? (r.i0 + r.nrows) : -1;
        if (gs < GROUPS) {
            float* crow = p.carry_val + (long long)blockIdx.x * p.carry_ld;
#pragma unroll
            for (int v = 0; v < NV; ++v) {
                const int cv = cb + lane + v * G;
                if (cv < p.ncolv) {
                    Vec<VW> sum;
                    sum.load(s.tail_of(gs) + (lane + v * G) * VW);
                    for (int q = gs + 1; q < GROUPS; ++q) {
                        Vec<VW> t;
                        t.load(s.tail_of(q) + (lane + v * G) * VW);
                        sum.add(t);
                    }
                    sum.store(crow + (long long)cv * VW);
                }
            }
        }
    }
}

// FULL: one pass covers the row exactly (G * NV == ncolv), so no column guard is compiled in.
// SKIP: the product runs under a schedule; rows of p.skip_len entries or more are summed by the
// scheduled pieces (sliced_kernel.cuh) and this kernel neither reads their entries nor writes
// their rows of C.  The tiles still count those rows' items, so a tile inside a hub row is a
// search and an exit.
template <int G, int NV, int VW, int TG, int U, int FMT, bool FULL, bool SKIP = false>
__global__ void __launch_bounds__(kMergeThreads, merge_min_blocks(NV)) spmm_merge_kernel(const SpmmParams p)
{
    using Smem = MergeSmem<G, NV, VW, TG>;
    __shared__ Smem s;

    TileRange r;
    if (!merge_tile_setup<Smem, G, TG, FMT, SKIP>(p, s, r)) return;
    const int g = threadIdx.x / G;
    const int lane = threadIdx.x % G;
    const char* const b_lane = reinterpret_cast<const char*>(p.B) + (size_t)lane * (VW * 4);
    const unsigned long long b_policy = make_b_policy();

    for (int cb = 0; cb < p.ncolv; cb += G * NV) {
        const char* const b_pass = b_lane + (size_t)cb * (VW * 4);
        bool col_ok[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) col_ok[v] = FULL || (cb + lane + v * G < p.ncolv);

        Vec<VW> acc[NV];
        Vec<VW> head[NV];  // the first row this group finishes is held back until step 4
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            acc[v].zero();
            head[v].zero();
        }
        int i = r.il0;
        int next_end = s.rowend[i];  // local position where row i ends (INT_MAX past the tile's rows)
        bool dirty = false;
        bool skip = false;       // SKIP: row i belongs to the scheduled pieces
        bool head_skip = false;  // SKIP: so did the first row this group finished
        if constexpr (SKIP) skip = s.is_long(i);

        auto finish_row = [&]() {
            if (SKIP && skip) {
                if (i == r.il0) head_skip = true;
            } else if (i == r.il0) {
#pragma unroll
                for (int v = 0; v < NV; ++v) head[v] = acc[v];
            } else {
                store_row<G, NV, VW>(p, r.i0 + i, cb, lane, acc);
            }
#pragma unroll
            for (int v = 0; v < NV; ++v) acc[v].zero();
            dirty = false;
            ++i;
            next_end = s.rowend[i];
            if constexpr (SKIP) skip = s.is_long(i);
        };

        // B row of staged non-zero e: one 32x32->64 multiply-add gives the address
        auto load_b = [&](Vec<VW> (&dst)[NV], int col) {
            const char* brow = b_pass + (unsigned long long)(unsigned)col * p.ldb_bytes;
#pragma unroll
            for (int v = 0; v < NV; ++v) {
                if (col_ok[v]) dst[v].load_b(reinterpret_cast<const float*>(brow + v * (G * VW * 4)), b_policy);
                else dst[v].zero();
            }
        };

        int base = r.jl0;
        if constexpr (SKIP || CSRSPMM_TUNE_MERGE_ONE_LOOP) {
            // as below, but a scheduled row is jumped over: to its end when that lies in this
            // group's range (rows before il1 end at or before jl1), else to the end of the range
            while (base < r.jl1) {
                while (base >= next_end) finish_row();  // an entry exists at `base`, so these ends are mine
                if (SKIP && skip) {
                    if (i < r.il1) {
                        base = next_end;
                        finish_row();
                    } else {
                        base = r.jl1;
                    }
                    continue;
                }
                const int n = min(U, r.jl1 - base);
                int2 e[U];
                Vec<VW> bq[U][NV];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (u < n) {
                        e[u] = s.cv[base + u];
                        load_b(bq[u], e[u].x);
                    }
                }
                if (n == U && base + U <= next_end) {
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const float a = __int_as_float(e[u].y);
#pragma unroll
                        for (int v = 0; v < NV; ++v) acc[v].fma(a, bq[u][v]);
                    }
                    dirty = true;
                } else {
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        if (u < n) {
                            while (base + u >= next_end) finish_row();
                            if (!(SKIP && skip)) {
                                const float a = __int_as_float(e[u].y);
#pragma unroll
                                for (int v = 0; v < NV; ++v) acc[v].fma(a, bq[u][v]);
                                dirty = true;
                            }
                        }
                    }
                }
                base += n;
            }
        } else {
        // whole batches of U non-zeros: loads first (they do not depend on the row structure),
        // then the multiply-adds, without any per-element test when no row ends inside the batch
        for (; base + U <= r.jl1; base += U) {
            int2 e[U];
            Vec<VW> bq[U][NV];
#pragma unroll
            for (int u = 0; u < U; ++u) e[u] = s.cv[base + u];
#pragma unroll
            for (int u = 0; u < U; ++u) load_b(bq[u], e[u].x);
            if (base + U <= next_end) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const float a = __int_as_float(e[u].y);
#pragma unroll
                    for (int v = 0; v < NV; ++v) acc[v].fma(a, bq[u][v]);
                }
                dirty = true;
            } else {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    while (base + u >= next_end) finish_row();  // rowend[nrows] = INT_MAX stops it
                    const float a = __int_as_float(e[u].y);
#pragma unroll
                    for (int v = 0; v < NV; ++v) acc[v].fma(a, bq[u][v]);
                    dirty = true;
                }
            }
        }
        // the last, partial batch
        if (base < r.jl1) {
            const int n = r.jl1 - base;
            int2 e[U];
            Vec<VW> bq[U][NV];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (u < n) {
                    e[u] = s.cv[base + u];
                    load_b(bq[u], e[u].x);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (u < n) {
                    while (base + u >= next_end) finish_row();
                    const float a = __int_as_float(e[u].y);
#pragma unroll
                    for (int v = 0; v < NV; ++v) acc[v].fma(a, bq[u][v]);
                    dirty = true;
                }
            }
        }
        }  // !SKIP
        while (i < r.il1) finish_row();

        merge_tile_finish<Smem, G, NV, VW>(p, s, r, cb, g, lane, acc, head, dirty, head_skip);
        if (cb + G * NV < p.ncolv) __syncthreads();  // tails are rewritten by the next pass
    }
}

// Adds the carries to C: the first tile of each run of equal carry_row sums the run in tile
// order and does C[row] += alpha * sum.  One warp per tile, lanes over column vectors.
template <int VW>
__global__ void __launch_bounds__(256) spmm_fixup_kernel(const SpmmParams p, int num_tiles)
{
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (t >= num_tiles) return;
    const int row = __ldg(p.carry_row + t);
    if (row < 0 || row >= p.M) return;
    if (t > 0 && __ldg(p.carry_row + t - 1) == row) return;
    // end of the run of tiles that carry this row: 32 tiles examined per step, so that a row
    // spread over thousands of tiles (a hub row) is not a chain of dependent loads
    int e = t + 1;
    for (;;) {
        const int idx = e + lane;
        const bool same = idx < num_tiles && __ldg(p.carry_row + idx) == row;
        const unsigned m = __ballot_sync(0xffffffffu, same);
        if (m == 0xffffffffu) {
            e += 32;
            continue;
        }
        e += __ffs(~m) - 1;
        break;
    }

    float* crow = p.C + (long long)row * p.ldc;
    for (int cv = lane; cv < p.ncolv; cv += 32) {
        const float* src = p.carry_val + (long long)cv * VW;
        Vec<VW> sum;
        sum.load(src + (long long)t * p.carry_ld);
        int q = t + 1;
        for (; q + 8 <= e; q += 8) {  // eight loads in flight, added in tile order
            Vec<VW> x[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) x[k].load(src + (long long)(q + k) * p.carry_ld);
#pragma unroll
            for (int k = 0; k < 8; ++k) sum.add(x[k]);
        }
        for (; q < e; ++q) {
            Vec<VW> x;
            x.load(src + (long long)q * p.carry_ld);
            sum.add(x);
        }
        Vec<VW> old;
        old.load(crow + (long long)cv * VW);
        sum.add_scaled_to(p.alpha, old).store(crow + (long long)cv * VW);
    }
}

}  // namespace csrspmm_b200
