// Scheduled pieces of long rows: the part of a product that a csrspmm_b200_schedule orders by
// slab of B.
//
// The reference has one mapping, a warp per row (src/device/csrspmm_warp_per_row.cu:24-43), and an
// auto-selection stub that looks at nothing (src/csrspmm.cpp:34-40).  When B is several times
// larger than L2, almost every gathered row of B comes from HBM; but a row with several entries
// per L2-sized slab of B can take them from L2 if every long row's entries of one slab are
// processed at about the same time.  The schedule (abi/schedule.cu) cuts each long row at the slab
// boundaries, cuts every part again into pieces of bounded length and lists the pieces slab by
// slab.  Here:
//
//   spmm_sliced_kernel   a persistent grid; every warp draws runs of consecutive pieces from the list
//                        (one ticket counter, the next ticket requested while the current run is
//                        summed), its lane groups sum a few pieces each: a sequential fp32 sum over
//                        the piece's entries, the rows of B pipelined through a ring in shared
//                        memory, written raw (no alpha/beta) to the piece's own slot of scratch.
//                        Drawing in list order keeps every SM on the same one or two slabs at any
//                        time; which warp sums a piece does not change the sum.
//   spmm_slot_reduce_kernel   one thread per long row and column vector: the row's slots added in stored order,
//                        then C[row] = alpha * sum + beta * C[row].  No atomics anywhere, so the
//                        result is the same on every run; a row that fits one piece is the
//                        sequential sum of the oracle bit for bit.
//
// Pieces hold offsets into col_idx/values; they are clamped to [0, nnz] and column indices to
// [0, Kd), so a schedule that does not belong to the matrix gives wrong numbers, never a fault.
#pragma once

#include <cooperative_groups.h>

#include "common.cuh"
#include "tuning.h"

namespace csrspmm_b200 {

namespace cg = cooperative_groups;

constexpr int kSlicedThreads = 256;

struct SlicedParams {
    const int4* pieces;    // {first entry, end entry, slot, slab}, slab-major
    int num_pieces;
    int pieces_per_group;  // consecutive pieces one lane group sums
    int piece_cap;         // no piece is longer than this (the schedule's piece_nnz)
    float* slots;          // num_pieces rows of slot_ld floats
    long long slot_ld;     // multiple of 4
    const int4* long_rows; // {row, first slot, slot count, unused}
    int num_long_rows;
    int evict_last;        // B loads carry an evict_last policy (the slab should outlive the streams)
    unsigned* tickets;     // one counter, zero at launch: runs of pieces handed out in list order
};

// Shared memory of one CTA of spmm_sliced_kernel, in bytes: the ring of gathered B rows, the staged
// (col, val) pairs and the piece tables of every lane group.
__host__ __device__ constexpr size_t sliced_smem_bytes(int G, int NV, int VW, int D, int ppg, int cap)
{
    const size_t groups = kSlicedThreads / G;
    return groups * D * (size_t)(G * NV * VW) * 4 + groups * (size_t)ppg * cap * 8 + groups * (size_t)(2 * ppg + 2) * 4;
}

// A warp takes a run of (32 / G) * pieces_per_group consecutive pieces; each of its lane groups sums
// `pieces_per_group` of them.  The group first copies their (col, val) pairs to shared memory
// (coalesced, several requests in flight), then runs one pipeline over all of them: the rows of B
// for entries f + D .. f + D + 3 are requested (asynchronous copies into the group's ring, each
// lane its own 16 bytes of a row, so no lane ever reads what another lane copied) while entries
// f .. f + 3 are multiplied.  D rows per group stay in flight whatever the piece boundaries are, and
// a slow row (a miss in L2) delays the group only when it reaches the head of the ring.
template <int G, int NV, int VW, int D, int FMT, bool FULL, int MINB>
__global__ void __launch_bounds__(kSlicedThreads, MINB) spmm_sliced_kernel(const SpmmParams p, const SlicedParams q)
{
    constexpr int GROUPS = kSlicedThreads / G;
    constexpr int ROWW = G * NV * VW;  // floats per ring slot
    constexpr int NB = D / 4;  // completion groups in flight
    constexpr int SB = 4;      // (col, val) loads in flight per lane while a piece is staged
    static_assert(D % 4 == 0 && (D & (D - 1)) == 0, "ring depth must be a power of two and a multiple of 4");
    extern __shared__ __align__(16) unsigned char sliced_smem[];
    const cg::thread_block_tile<G> tile = cg::tiled_partition<G>(cg::this_thread_block());
    const int lane = tile.thread_rank();
    const int g = threadIdx.x / G;
    const int wl = threadIdx.x & 31;
    const int ppg = q.pieces_per_group;
    const int cap = ppg * q.piece_cap;
    const int run = (32 / G) * ppg;  // pieces per ticket

    float* const ring = reinterpret_cast<float*>(sliced_smem) + (size_t)g * D * ROWW;
    int2* const cvbuf = reinterpret_cast<int2*>(sliced_smem + (size_t)GROUPS * D * ROWW * 4) + (size_t)g * cap;
    int* const tab = reinterpret_cast<int*>(sliced_smem + (size_t)GROUPS * D * ROWW * 4 + (size_t)GROUPS * cap * 8) +
                     (size_t)g * (2 * ppg + 2);
    int* const off = tab;             // off[k] = first flat position of piece k, off[np] = total
    int* const slot_of = tab + ppg + 1;

    const char* const b_lane = reinterpret_cast<const char*>(p.B) + (size_t)lane * (VW * 4);
    const unsigned ring_lane = smem_addr(ring) + (unsigned)lane * (VW * 4);
    unsigned long long policy = 0;
    if (q.evict_last) asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
    const bool hinted = q.evict_last != 0;

    // ---- runs of pieces, handed out in list order ---------------------------------------------------------
    auto fetch = [&]() -> unsigned { return wl == 0 ? atomicAdd(q.tickets, 1u) : 0u; };
    // ticket -> first piece and end of the run (the same in every lane); first < 0: the list is used up
    auto resolve = [&](unsigned ticket, int& first, int& last) {
        const unsigned t = __shfl_sync(0xffffffffu, ticket, 0);
        if ((long long)t * run < (long long)q.num_pieces) {
            first = (int)t * run;
            last = min(first + run, q.num_pieces);
        } else {
            first = -1;
            last = 0;
        }
    };

    int run_first, run_last;
    resolve(fetch(), run_first, run_last);
    while (run_first >= 0) {
        const unsigned next_ticket = fetch();  // on its way while this run is summed; looked at only after it

        // ---- the group's pieces and their (col, val) pairs ------------------------------------------------
        const int it0 = run_first + (wl / G) * ppg;
        int total = 0, np = 0;
        for (int k = 0; k < ppg; ++k) {
            if (it0 + k >= run_last) break;
            const int4 d = __ldg(q.pieces + it0 + k);
            const int rs = min(max(d.x, 0), p.nnz);
            const int re = min(max(d.y, rs), min(p.nnz, rs + q.piece_cap));
            if (lane == 0) {
                off[k] = total;
                slot_of[k] = d.z;
            }
            for (int j0 = rs + lane; j0 < re; j0 += G * SB) {  // SB loads in flight per lane, then the stores
                int c[SB];
                float a[SB];
#pragma unroll
                for (int b = 0; b < SB; ++b) {
                    const int j = j0 + b * G;
                    if (j < re) {
                        c[b] = __ldcs(p.col_idx + j);
                        a[b] = load_value<FMT>(p.values, j, p.value_scale);
                    }
                }
#pragma unroll
                for (int b = 0; b < SB; ++b) {
                    const int j = j0 + b * G;
                    if (j < re) {
                        if ((unsigned)c[b] >= (unsigned)p.Kd) {  // never fault on a bad index
                            c[b] = min(max(c[b], 0), p.Kd - 1);
                            report_status(p, kStatusColClamped);
                        }
                        cvbuf[total + (j - rs)] = make_int2(c[b], __float_as_int(a[b]));
                    }
                }
            }
            total += re - rs;
            ++np;
        }
        if (lane == 0) off[np] = total;
        tile.sync();

        for (int cb = 0; np > 0 && cb < p.ncolv; cb += G * NV) {
            const char* const b_pass = b_lane + (size_t)cb * (VW * 4);
            bool col_ok[NV];
#pragma unroll
            for (int v = 0; v < NV; ++v) col_ok[v] = FULL || (cb + lane + v * G < p.ncolv);

            auto issue = [&](int f) {
                const char* brow = b_pass + (unsigned long long)(unsigned)cvbuf[f].x * p.ldb_bytes;
                const unsigned dst = ring_lane + (unsigned)(f & (D - 1)) * (ROWW * 4);
#pragma unroll
                for (int v = 0; v < NV; ++v) {
                    if (col_ok[v]) {
                        if (hinted) async_copy_vec_hint<VW>(dst + v * (G * VW * 4), brow + v * (G * VW * 4), policy);
                        else async_copy_vec<VW>(dst + v * (G * VW * 4), brow + v * (G * VW * 4));
                    }
                }
            };
            auto store_piece = [&](int k, const Vec<VW> (&acc)[NV]) {
                float* slot = q.slots + (long long)slot_of[k] * q.slot_ld;
#pragma unroll
                for (int v = 0; v < NV; ++v) {
                    const int cv = cb + lane + v * G;
                    if (FULL || cv < p.ncolv) {
                        if (CSRSPMM_TUNE_SLICED_STREAM_SLOTS) acc[v].store_streaming(slot + (long long)cv * VW);
                        else acc[v].store(slot + (long long)cv * VW);
                    }
                }
            };

            auto multiply = [&](int f, Vec<VW> (&acc)[NV]) {
                const float a = __int_as_float(cvbuf[f].y);
                const float* src = ring + (size_t)(f & (D - 1)) * ROWW + lane * VW;
#pragma unroll
                for (int v = 0; v < NV; ++v) {
                    if (col_ok[v]) {
                        Vec<VW> b;
                        b.load(src + v * (G * VW));
                        acc[v].fma(a, b);
                    }
                }
            };
            // requests go out four at a time, one completion group per four: the group of entries
            // f .. f+3 is always the NB-th youngest when they are multiplied
            auto request_four = [&](int f) {
                if (f + 4 <= total) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) issue(f + u);
                } else {
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (f + u < total) issue(f + u);
                }
                async_commit();
            };
#pragma unroll
            for (int b = 0; b < NB; ++b) request_four(b * 4);
            Vec<VW> acc[NV];
#pragma unroll
            for (int v = 0; v < NV; ++v) acc[v].zero();
            int k = 0;
            int next_off = off[1];
            for (int f = 0; f < total; f += 4) {
                async_wait<NB - 1>();
                if (f + 4 <= next_off) {  // inside one piece (f < next_off <= total)
#pragma unroll
                    for (int u = 0; u < 4; ++u) multiply(f + u, acc);
                } else {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (f + u < total) {
                            while (f + u >= next_off) {  // an empty piece writes zeros
                                store_piece(k, acc);
#pragma unroll
                                for (int v = 0; v < NV; ++v) acc[v].zero();
                                ++k;
                                next_off = off[k + 1];
                            }
                            multiply(f + u, acc);
                        }
                    }
                }
                request_four(f + D);
            }
            for (; k < np; ++k) {  // the last piece, and empty ones after it
                store_piece(k, acc);
#pragma unroll
                for (int v = 0; v < NV; ++v) acc[v].zero();
            }
            async_wait<0>();
        }
        tile.sync();  // the group's tables and ring are rewritten for the next run
        resolve(next_ticket, run_first, run_last);
    }
}

// One thread per (long row, column vector), consecutive threads on consecutive vectors: the row's
// slots added in stored order, sixteen loads in flight, then C[row] = alpha * sum + beta * C[row].
template <int VW>
__global__ void __launch_bounds__(256) spmm_slot_reduce_kernel(const SpmmParams p, const SlicedParams q)
{
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int h = (int)(t / p.ncolv);
    const int cv = (int)(t % p.ncolv);
    if (h >= q.num_long_rows) return;
    const int4 d = __ldg(q.long_rows + h);
    const int row = d.x;
    if (row < 0 || row >= p.M) return;
    const int n = d.z;
    const float* src = q.slots + (long long)d.y * q.slot_ld + (long long)cv * VW;
    Vec<VW> sum;
    sum.zero();
    int k = 0;
    if (n > 0) {
        sum.load(src);
        k = 1;
    }
    for (; k + 16 <= n; k += 16) {
        Vec<VW> x[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) x[u].load(src + (long long)(k + u) * q.slot_ld);
#pragma unroll
        for (int u = 0; u < 16; ++u) sum.add(x[u]);
    }
    for (; k < n; ++k) {
        Vec<VW> x;
        x.load(src + (long long)k * q.slot_ld);
        sum.add(x);
    }
    float* cp = p.C + (long long)row * p.ldc + (long long)cv * VW;
    if (p.beta != 0.0f) {
        Vec<VW> old;
        old.load(cp);
        sum.epilogue(p.alpha, p.beta, old).store(cp);
    } else {
        sum.epilogue0(p.alpha).store(cp);
    }
}

// ---- building a schedule ---------------------------------------------------------------------------

// counters[0] = long rows, [2..3] = their entries (one 64-bit count), [4] = 1 when a long row has
// unsorted columns, [5] = slots handed out
constexpr int kSchedCounters = 8;

// Lists the rows of `threshold` entries or more (any order: the list only decides which CTA sums
// which piece, never a result).
__global__ void sched_list_long_rows_kernel(int M, const int* __restrict__ row_ptr, int threshold, int* long_rows,
                                            int capacity, unsigned* counters)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long r0 = (long long)blockIdx.x * blockDim.x; r0 < M; r0 += stride) {
        const long long r = r0 + threadIdx.x;
        int len = 0;
        if (r < M) len = __ldg(row_ptr + r + 1) - __ldg(row_ptr + r);
        const bool is_long = r < M && len >= threshold;
        const unsigned m = __ballot_sync(0xffffffffu, is_long);
        if (m == 0) continue;
        const int lane = threadIdx.x & 31;
        unsigned base = 0;
        unsigned long long sum = is_long ? (unsigned long long)len : 0ull;
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) {
            base = atomicAdd(counters + 0, (unsigned)__popc(m));
            atomicAdd(reinterpret_cast<unsigned long long*>(counters + 2), sum);  // 8-byte aligned pair [2], [3]
        }
        base = __shfl_sync(0xffffffffu, base, 0);
        if (is_long) {
            const unsigned pos = base + __popc(m & ((1u << lane) - 1u));
            if (long_rows != nullptr && pos < (unsigned)capacity) long_rows[pos] = (int)r;
        }
    }
}

// One warp per long row.  Walks the row's columns once: checks that they ascend and records where
// each slab starts, bounds[h * (S + 1) + s] = first entry of the row whose column is >= s * slab_rows
// (bounds[.][S] = the row's end).  Then counts the row's pieces per slab into slab_count[s] and
// reserves its slots.
__global__ void sched_cut_rows_kernel(int num_long, const int* __restrict__ long_rows, const int* __restrict__ row_ptr,
                                      const int* __restrict__ col_idx, int nnz, int slab_rows, int num_slabs,
                                      int piece_nnz, int* bounds, unsigned* slab_count, int4* long_desc,
                                      unsigned* counters)
{
    const int warps_per_cta = blockDim.x >> 5;
    const int h = blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (h >= num_long) return;
    const int row = __ldg(long_rows + h);
    const int rs = min(max(__ldg(row_ptr + row), 0), nnz);
    const int re = min(max(__ldg(row_ptr + row + 1), rs), nnz);
    int* b = bounds + (long long)h * (num_slabs + 1);
    bool unsorted = false;
    // entry j starts every slab in (slab(j-1), slab(j)]; the first entry also starts slabs 0..slab(rs)
    for (int j = rs + lane; j < re; j += 32) {
        const int c = __ldg(col_idx + j);
        const int sj = min(max(c, 0) / slab_rows, num_slabs - 1);
        int sp = -1;
        if (j > rs) {
            const int cp = __ldg(col_idx + j - 1);
            if (cp >= c) unsorted = true;
            sp = min(max(cp, 0) / slab_rows, num_slabs - 1);
        }
        for (int s = sp + 1; s <= sj; ++s) b[s] = j;
    }
    // slabs after the last entry's are empty
    int s_last = -1;
    if (re > rs) s_last = min(max(__ldg(col_idx + re - 1), 0) / slab_rows, num_slabs - 1);
    for (int s = s_last + 1 + lane; s <= num_slabs; s += 32) b[s] = re;
    if (__any_sync(0xffffffffu, unsorted)) {
        if (lane == 0) atomicOr(counters + 4, 1u);
    }
    __syncwarp();
    __threadfence_block();
    // pieces per slab
    int mine = 0;
    for (int s = lane; s < num_slabs; s += 32) {
        const int len = b[s + 1] - b[s];
        if (len > 0) {
            const int cnt = (len + piece_nnz - 1) / piece_nnz;
            atomicAdd(slab_count + s, (unsigned)cnt);
            mine += cnt;
        }
    }
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if (lane == 0) {
        const unsigned s0 = atomicAdd(counters + 5, (unsigned)mine);
        long_desc[h] = make_int4(row, (int)s0, mine, 0);
    }
}

// One thread per long row: writes the row's pieces into the slab-major list.  slab_fill[s] starts
// at the first list position of slab s and is advanced by each row's piece count.
__global__ void sched_emit_pieces_kernel(int num_long, int num_slabs, int piece_nnz, const int* __restrict__ bounds,
                                         unsigned* slab_fill, const int4* __restrict__ long_desc, int4* pieces,
                                         int num_pieces)
{
    const int h = blockIdx.x * blockDim.x + threadIdx.x;
    if (h >= num_long) return;
    const int* b = bounds + (long long)h * (num_slabs + 1);
    int slot = long_desc[h].y;
    for (int s = 0; s < num_slabs; ++s) {
        const int lo = b[s], len = b[s + 1] - lo;
        if (len <= 0) continue;
        const int cnt = (len + piece_nnz - 1) / piece_nnz;
        const int each = (len + cnt - 1) / cnt;  // equal pieces rather than full ones and a stub
        const unsigned pos = atomicAdd(slab_fill + s, (unsigned)cnt);
        for (int k = 0; k < cnt; ++k) {
            const int a = lo + k * each;
            const int e = min(a + each, lo + len);
            if (pos + k < (unsigned)num_pieces) pieces[pos + k] = make_int4(a, e, slot, s);
            ++slot;
        }
    }
}

}  // namespace csrspmm_b200
