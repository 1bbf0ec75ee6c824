// Host-only launch planning for the SpMM entry point: which kernel, which lane-group shape,
// how many tiles, how much scratch.  Pure C++ (no CUDA call), so it can be unit-tested on a
// machine without a GPU.  Replaces the fixed geometry of the reference's launchers
// (src/host/spmm_launcher.cu:17-19, 63-66, 112-120) and the stub auto-selection of
// src/csrspmm.cpp:34-40.
#pragma once

#include <cstddef>
#include <cstdint>

#include "../kernels/tuning.h"
#include "csrspmm_b200.h"

namespace csrspmm_b200 {

struct Plan {
    int kernel = CSRSPMM_B200_KERNEL_ROW;  // resolved, never AUTO
    int shape = 0;                         // index into kShapes (tuning.h)
    bool low_occupancy = false;            // row kernel: fewer than 8 warps of rows per SM
    bool full = false;                     // one pass covers the row exactly: G*NV == ncolv
    bool small_tile = false;               // merge kernel: the small-problem tile (fewer items per lane group)
    int narrow = 0;                        // merge kernel: 1 + index into kNarrowShapes when the dense operand has at
                                           // most four column vectors (lane groups of 1, 2 or 4 lanes), else 0
    int G = 8, NV = 1, VW = 4;             // lanes per group, vectors per lane, vector width
    int ncolv = 0;                         // ceil(Nd / VW)
    int tile = 0;                          // merge-path items per CTA (split kernels)
    long long num_items = 0;               // M + nnz
    long long num_tiles = 0;               // CTAs of the split kernels
    long long grid = 0;                    // CTAs of the main kernel
    long long carry_ld = 0;                // floats per carry row
    size_t carry_row_bytes = 0;            // 256-byte aligned
    size_t workspace_bytes = 0;            // carry_row_bytes + carry values
    size_t dynamic_smem = 0;               // TMA kernel only: 8 warps x ring_stride
    size_t tma_slot_bytes = 0;             // TMA kernel only: one row of B rounded up to 128 bytes
};

// Checks the argument block (sizes, enums, pointers) without touching memory.
int check_args(const csrspmm_b200_args* a, bool need_pointers);

// True when every row of B and C, and both base pointers, allow 16-byte vector access.
bool vector_layout_ok(const csrspmm_b200_args* a);

// Resolves AUTO (and the CSRSPMM_FORCE_KERNEL override) and fills the launch geometry.
// Returns CSRSPMM_B200_OK or an error status.
int make_plan(const csrspmm_b200_args* a, Plan* plan, bool allow_narrow = true);

// Merge-path items per CTA of the merge kernel for lane-group shape `shape` on a problem of
// `num_items` = M + nnz items (*small says whether the small-problem tile was chosen).
int merge_tile_for(int shape, long long num_items, bool* small);

// Workspace of the split kernels for a given plan-independent worst case: what
// csrspmm_b200_workspace_bytes reports (the larger of the MERGE and TMA needs).  any_row_block:
// also enough for any contiguous block of the matrix's rows multiplied on its own.
size_t worst_case_workspace(const csrspmm_b200_args* a, bool any_row_block = false);

void set_last_error(const char* fmt, ...);
const char* get_last_error();

}  // namespace csrspmm_b200
