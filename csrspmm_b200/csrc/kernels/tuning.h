// Compile-time tuning constants of the SpMM kernels.  Every value can be overridden on the
// compiler command line (-DCSRSPMM_TUNE_...=n) to build an experimental variant of the library;
// the defaults are the measured best on B200.
#pragma once

// B-row loads kept in flight per lane, by number of column vectors per lane (NV) -- merge kernel
#ifndef CSRSPMM_TUNE_MERGE_U_NV1
#define CSRSPMM_TUNE_MERGE_U_NV1 6
#endif
#ifndef CSRSPMM_TUNE_MERGE_U_NV2
#define CSRSPMM_TUNE_MERGE_U_NV2 4
#endif
#ifndef CSRSPMM_TUNE_MERGE_U_NV4
#define CSRSPMM_TUNE_MERGE_U_NV4 3
#endif
// ... and row kernel
#ifndef CSRSPMM_TUNE_ROW_U_NV1
#define CSRSPMM_TUNE_ROW_U_NV1 4
#endif
#ifndef CSRSPMM_TUNE_ROW_U_NV2
#define CSRSPMM_TUNE_ROW_U_NV2 2
#endif
#ifndef CSRSPMM_TUNE_ROW_U_NV4
#define CSRSPMM_TUNE_ROW_U_NV4 4
#endif

// scheduled pieces (sliced_kernel.cuh): consecutive pieces per lane group
#ifndef CSRSPMM_TUNE_SLICED_PIECES_PER_GROUP
#define CSRSPMM_TUNE_SLICED_PIECES_PER_GROUP 1
#endif
// scheduled pieces: resident CTAs per SM asked of the compiler (caps the registers)
#ifndef CSRSPMM_TUNE_SLICED_MINB
#define CSRSPMM_TUNE_SLICED_MINB 2
#endif
// scheduled pieces load B with an evict_last policy (1) or plainly (0)
#ifndef CSRSPMM_TUNE_SLICED_EVICT_LAST
#define CSRSPMM_TUNE_SLICED_EVICT_LAST 0
#endif
// scheduled pieces write their slots with streaming stores (1) or plain ones (0): the slots are read
// back by another kernel and should not push the slab of B out of L2
#ifndef CSRSPMM_TUNE_SLICED_STREAM_SLOTS
#define CSRSPMM_TUNE_SLICED_STREAM_SLOTS 0
#endif

// Scheduled pieces (sliced_kernel.cuh): the gather is pipelined through shared memory, no gathered
// row is held in registers, so a lane can own more column vectors and a warp more pieces.  Per dense
// width class k: lanes per group G, vectors per lane NV, rows of B in flight per group D (a multiple
// of 4 and a power of two; G*NV*16*D*(256/G) = 64 KB of ring per CTA at every width).
#ifndef CSRSPMM_TUNE_P0_G
#define CSRSPMM_TUNE_P0_G 8
#endif
#ifndef CSRSPMM_TUNE_P0_NV
#define CSRSPMM_TUNE_P0_NV 1
#endif
#ifndef CSRSPMM_TUNE_P0_D
#define CSRSPMM_TUNE_P0_D 16
#endif
#ifndef CSRSPMM_TUNE_P1_G
#define CSRSPMM_TUNE_P1_G 8
#endif
#ifndef CSRSPMM_TUNE_P1_NV
#define CSRSPMM_TUNE_P1_NV 2
#endif
#ifndef CSRSPMM_TUNE_P1_D
#define CSRSPMM_TUNE_P1_D 8
#endif
#ifndef CSRSPMM_TUNE_P2_G
#define CSRSPMM_TUNE_P2_G 16
#endif
#ifndef CSRSPMM_TUNE_P2_NV
#define CSRSPMM_TUNE_P2_NV 2
#endif
#ifndef CSRSPMM_TUNE_P2_D
#define CSRSPMM_TUNE_P2_D 8
#endif
#ifndef CSRSPMM_TUNE_P3_G
#define CSRSPMM_TUNE_P3_G 32
#endif
#ifndef CSRSPMM_TUNE_P3_NV
#define CSRSPMM_TUNE_P3_NV 2
#endif
#ifndef CSRSPMM_TUNE_P3_D
#define CSRSPMM_TUNE_P3_D 8
#endif
#ifndef CSRSPMM_TUNE_P4_G
#define CSRSPMM_TUNE_P4_G 32
#endif
#ifndef CSRSPMM_TUNE_P4_NV
#define CSRSPMM_TUNE_P4_NV 4
#endif
#ifndef CSRSPMM_TUNE_P4_D
#define CSRSPMM_TUNE_P4_D 4
#endif

// merge-path kernel: walk a lane group's range with one loop (loads predicated on the batch length)
// instead of a loop of whole batches followed by the partial one
#ifndef CSRSPMM_TUNE_MERGE_ONE_LOOP
#define CSRSPMM_TUNE_MERGE_ONE_LOOP 0
#endif

// threads per CTA of the merge-path kernels (merge, bulk-copy): lane groups per CTA = this / G
// merge-path tile staging: global loads in flight per thread before the stores to shared memory
#ifndef CSRSPMM_TUNE_MERGE_STAGE_BATCH
#define CSRSPMM_TUNE_MERGE_STAGE_BATCH 6
#endif
#ifndef CSRSPMM_TUNE_MERGE_THREADS
#define CSRSPMM_TUNE_MERGE_THREADS 256
#endif

// L2 residency hints: rows of B loaded with an evict_last policy applied to this percentage of
// the lines, C written with streaming stores.  Both are OFF by default: on B200 neither helped
// (config 3, B = 2.1 x L2: 685 us without hints, 687-714 us with any combination of them).
#ifndef CSRSPMM_TUNE_B_EVICT_LAST_PCT
#define CSRSPMM_TUNE_B_EVICT_LAST_PCT 0
#endif
#ifndef CSRSPMM_TUNE_C_STREAMING
#define CSRSPMM_TUNE_C_STREAMING 0
#endif

// shared-memory row buffers per warp in the TMA kernel (bulk copies in flight per warp)
#ifndef CSRSPMM_TUNE_TMA_SLOTS
#define CSRSPMM_TUNE_TMA_SLOTS 4
#endif
// merge-path items per warp in the TMA kernel, and its requested CTAs per SM
#ifndef CSRSPMM_TUNE_TMA_TG
#define CSRSPMM_TUNE_TMA_TG 128
#endif
#ifndef CSRSPMM_TUNE_TMA_MINB
#define CSRSPMM_TUNE_TMA_MINB 2
#endif

// row kernel: how a group hands its G loaded (col, val) pairs to all its lanes: 1 = through a
// shared-memory slice (broadcast reads), 0 = lane to lane by shuffle
#ifndef CSRSPMM_TUNE_ROW_STAGE_SMEM
#define CSRSPMM_TUNE_ROW_STAGE_SMEM 1
#endif

// row kernel on short rows (mean of 64 non-zeros or fewer): at most this many CTAs per SM, each
// looping over rows, instead of one short-lived CTA per 128/G rows (0 = never)
#ifndef CSRSPMM_TUNE_ROW_PERSISTENT
#define CSRSPMM_TUNE_ROW_PERSISTENT 8
#endif

// ... for matrices whose mean row length is at most this
#ifndef CSRSPMM_TUNE_ROW_PERSISTENT_MAX_MEAN
#define CSRSPMM_TUNE_ROW_PERSISTENT_MAX_MEAN 64
#endif

// threads per CTA of the row kernel (128: 4 rows per CTA at G = 32; small CTAs keep the tail short
// when there are only a few thousand rows -- 4096 rows in 256-thread CTAs left a 15 % imbalance)
#ifndef CSRSPMM_TUNE_ROW_THREADS
#define CSRSPMM_TUNE_ROW_THREADS 128
#endif

// row kernel, few rows (fewer warps of work than 8 per SM): registers are plentiful and latency is
// everything, so many more loads are kept in flight per lane
#ifndef CSRSPMM_TUNE_ROW_ULOW_NV1
#define CSRSPMM_TUNE_ROW_ULOW_NV1 16
#endif
#ifndef CSRSPMM_TUNE_ROW_ULOW_NV2
#define CSRSPMM_TUNE_ROW_ULOW_NV2 8
#endif
#ifndef CSRSPMM_TUNE_ROW_ULOW_NV4
#define CSRSPMM_TUNE_ROW_ULOW_NV4 4
#endif

// minimum resident CTAs per SM requested from the compiler (caps registers per thread)
#ifndef CSRSPMM_TUNE_MERGE_MINB_NV1
#define CSRSPMM_TUNE_MERGE_MINB_NV1 4
#endif
#ifndef CSRSPMM_TUNE_MERGE_MINB_NV2
#define CSRSPMM_TUNE_MERGE_MINB_NV2 3
#endif
#ifndef CSRSPMM_TUNE_MERGE_MINB_NV4
#define CSRSPMM_TUNE_MERGE_MINB_NV4 2
#endif
#ifndef CSRSPMM_TUNE_ROW_MINB_NV1
#define CSRSPMM_TUNE_ROW_MINB_NV1 8
#endif
#ifndef CSRSPMM_TUNE_ROW_MINB_NV2
#define CSRSPMM_TUNE_ROW_MINB_NV2 8
#endif
#ifndef CSRSPMM_TUNE_ROW_MINB_NV4
#define CSRSPMM_TUNE_ROW_MINB_NV4 4
#endif

// lane-group shapes by dense width class k (column vectors per row <= 8, 16, 32, 64, more):
// lanes per group G, vectors per lane NV, merge-path items per group TG.  TG = 192 against 128:
// fewer, longer-lived CTAs (one search, one staging round and one carry row each) -- config 3
// 686 -> 654 us, the same matrix at Nd = 128 1361 -> 1285 us, config 5 at a quarter of its rows
// 10.26 -> 10.04 ms; 224-256 gained nothing more and TG = 256 at G = 16 no longer fits the 48 KB
// of static shared memory
#ifndef CSRSPMM_TUNE_S0_G
#define CSRSPMM_TUNE_S0_G 8
#endif
#ifndef CSRSPMM_TUNE_S0_NV
#define CSRSPMM_TUNE_S0_NV 1
#endif
#ifndef CSRSPMM_TUNE_S0_TG
#define CSRSPMM_TUNE_S0_TG 64
#endif
#ifndef CSRSPMM_TUNE_S1_G
#define CSRSPMM_TUNE_S1_G 16
#endif
#ifndef CSRSPMM_TUNE_S1_NV
#define CSRSPMM_TUNE_S1_NV 1
#endif
#ifndef CSRSPMM_TUNE_S1_TG
#define CSRSPMM_TUNE_S1_TG 192
#endif
#ifndef CSRSPMM_TUNE_S2_G
#define CSRSPMM_TUNE_S2_G 32
#endif
#ifndef CSRSPMM_TUNE_S2_NV
#define CSRSPMM_TUNE_S2_NV 1
#endif
#ifndef CSRSPMM_TUNE_S2_TG
#define CSRSPMM_TUNE_S2_TG 192
#endif
#ifndef CSRSPMM_TUNE_S3_G
#define CSRSPMM_TUNE_S3_G 32
#endif
#ifndef CSRSPMM_TUNE_S3_NV
#define CSRSPMM_TUNE_S3_NV 2
#endif
#ifndef CSRSPMM_TUNE_S3_TG
#define CSRSPMM_TUNE_S3_TG 192
#endif
#ifndef CSRSPMM_TUNE_S4_G
#define CSRSPMM_TUNE_S4_G 32
#endif
#ifndef CSRSPMM_TUNE_S4_NV
#define CSRSPMM_TUNE_S4_NV 4
#endif
#ifndef CSRSPMM_TUNE_S4_TG
#define CSRSPMM_TUNE_S4_TG 192
#endif

namespace csrspmm_b200 {

// merge kernel on small problems: when the regular tiles would give fewer than this many CTAs
// per SM, lane groups take CSRSPMM_TUNE_MERGE_TG_SMALL items instead, so that the chip still fills
#ifndef CSRSPMM_TUNE_MERGE_TG_SMALL
#define CSRSPMM_TUNE_MERGE_TG_SMALL 64
#endif
#ifndef CSRSPMM_TUNE_MERGE_SMALL_BELOW_CTAS_PER_SM
#define CSRSPMM_TUNE_MERGE_SMALL_BELOW_CTAS_PER_SM 2
#endif

struct ShapeDesc {
    int G, NV, TG;
};
// Merge-path kernel on very narrow dense operands (1, 2 or 4 column vectors: Nd <= 4, 8, 16 with the
// 16-byte layout): a lane group of eight would leave seven, six or four of its lanes without a column,
// so the groups shrink to 1, 2 or 4 lanes -- at G = 1 every lane walks its own run of non-zeros
// (lanes over non-zeros instead of lanes over columns) and the rows cut between lanes are summed in
// lane order through shared memory like any other split row.  3072 merge-path items per CTA as for
// the wider shapes.
#ifndef CSRSPMM_TUNE_MERGE_NARROW
#define CSRSPMM_TUNE_MERGE_NARROW 1
#endif
constexpr int kNumNarrowShapes = 3;
constexpr ShapeDesc kNarrowShapes[kNumNarrowShapes] = {{1, 1, 12}, {2, 1, 24}, {4, 1, 48}};
struct PieceShapeDesc {
    int G, NV, D;
};
constexpr PieceShapeDesc kPieceShapes[5] = {
    {CSRSPMM_TUNE_P0_G, CSRSPMM_TUNE_P0_NV, CSRSPMM_TUNE_P0_D}, {CSRSPMM_TUNE_P1_G, CSRSPMM_TUNE_P1_NV, CSRSPMM_TUNE_P1_D},
    {CSRSPMM_TUNE_P2_G, CSRSPMM_TUNE_P2_NV, CSRSPMM_TUNE_P2_D}, {CSRSPMM_TUNE_P3_G, CSRSPMM_TUNE_P3_NV, CSRSPMM_TUNE_P3_D},
    {CSRSPMM_TUNE_P4_G, CSRSPMM_TUNE_P4_NV, CSRSPMM_TUNE_P4_D}};
constexpr int kNumShapes = 5;
constexpr ShapeDesc kShapes[kNumShapes] = {
    {CSRSPMM_TUNE_S0_G, CSRSPMM_TUNE_S0_NV, CSRSPMM_TUNE_S0_TG}, {CSRSPMM_TUNE_S1_G, CSRSPMM_TUNE_S1_NV, CSRSPMM_TUNE_S1_TG},
    {CSRSPMM_TUNE_S2_G, CSRSPMM_TUNE_S2_NV, CSRSPMM_TUNE_S2_TG}, {CSRSPMM_TUNE_S3_G, CSRSPMM_TUNE_S3_NV, CSRSPMM_TUNE_S3_TG},
    {CSRSPMM_TUNE_S4_G, CSRSPMM_TUNE_S4_NV, CSRSPMM_TUNE_S4_TG}};

constexpr int merge_unroll(int nv) { return nv == 1 ? CSRSPMM_TUNE_MERGE_U_NV1 : (nv == 2 ? CSRSPMM_TUNE_MERGE_U_NV2 : CSRSPMM_TUNE_MERGE_U_NV4); }
constexpr int row_unroll(int nv) { return nv == 1 ? CSRSPMM_TUNE_ROW_U_NV1 : (nv == 2 ? CSRSPMM_TUNE_ROW_U_NV2 : CSRSPMM_TUNE_ROW_U_NV4); }
constexpr int row_unroll_low(int nv) { return nv == 1 ? CSRSPMM_TUNE_ROW_ULOW_NV1 : (nv == 2 ? CSRSPMM_TUNE_ROW_ULOW_NV2 : CSRSPMM_TUNE_ROW_ULOW_NV4); }
constexpr int row_min_blocks(int nv) { return nv == 1 ? CSRSPMM_TUNE_ROW_MINB_NV1 : (nv == 2 ? CSRSPMM_TUNE_ROW_MINB_NV2 : CSRSPMM_TUNE_ROW_MINB_NV4); }
constexpr int merge_min_blocks(int nv) { return nv == 1 ? CSRSPMM_TUNE_MERGE_MINB_NV1 : (nv == 2 ? CSRSPMM_TUNE_MERGE_MINB_NV2 : CSRSPMM_TUNE_MERGE_MINB_NV4); }

}  // namespace csrspmm_b200
