// Host-only launch planning (see plan.h).
#include "plan.h"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace csrspmm_b200 {

namespace {
thread_local char g_last_error[512] = "";

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
}  // namespace

void set_last_error(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

const char* get_last_error() { return g_last_error; }

int check_args(const csrspmm_b200_args* a, bool need_pointers)
{
    if (a == nullptr) {
        set_last_error("args is null");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (a->struct_size != sizeof(csrspmm_b200_args)) {
        set_last_error("args.struct_size is %u, this library expects %zu", a->struct_size,
                       sizeof(csrspmm_b200_args));
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (a->M < 0 || a->Kd < 0 || a->Nd < 0 || a->nnz < 0 || a->nnz > 0x7fffffffLL) {
        set_last_error("negative or oversized dimension (M=%d Kd=%d Nd=%d nnz=%lld)", a->M, a->Kd,
                       a->Nd, (long long)a->nnz);
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (a->row_ptr_base < 0) {
        set_last_error("negative row_ptr_base %d", a->row_ptr_base);
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (a->row_ptr_base != 0 && a->value_format == CSRSPMM_B200_VALUES_E2M1 && (a->row_ptr_base & 1)) {
        set_last_error("row_ptr_base must be even for packed e2m1 values (two codes per byte)");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (a->nnz > 0 && a->Kd == 0) {
        set_last_error("nnz > 0 with Kd == 0");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (a->ldb >= (1LL << 30) || a->ldc >= (1LL << 30)) {
        set_last_error("leading dimension of 2^30 elements or more (ldb=%lld ldc=%lld)", (long long)a->ldb,
                       (long long)a->ldc);
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (a->ldb < a->Nd || a->ldc < a->Nd) {
        set_last_error("leading dimension smaller than Nd (ldb=%lld ldc=%lld Nd=%d)",
                       (long long)a->ldb, (long long)a->ldc, a->Nd);
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (a->value_format != CSRSPMM_B200_VALUES_F32 && a->value_format != CSRSPMM_B200_VALUES_E2M1) {
        set_last_error("unknown value_format %d", a->value_format);
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (a->entry < CSRSPMM_B200_ENTRY_NAIVE || a->entry > CSRSPMM_B200_ENTRY_WARP_PER_ROW_SMEM_FP4) {
        set_last_error("unknown entry %d", a->entry);
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (a->kernel < CSRSPMM_B200_KERNEL_AUTO || a->kernel > CSRSPMM_B200_KERNEL_TMA) {
        set_last_error("unknown kernel %d", a->kernel);
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (need_pointers && a->M > 0 && a->Nd > 0) {
        if (a->row_ptr == nullptr || a->C == nullptr ||
            (a->nnz > 0 && (a->col_idx == nullptr || a->values == nullptr || a->B == nullptr))) {
            set_last_error("null matrix pointer");
            return CSRSPMM_B200_ERR_BAD_ARG;
        }
    }
    return CSRSPMM_B200_OK;
}

bool vector_layout_ok(const csrspmm_b200_args* a)
{
    return a->Nd % 4 == 0 && a->ldb % 4 == 0 && a->ldc % 4 == 0 &&
           (reinterpret_cast<uintptr_t>(a->B) & 15u) == 0 &&
           (reinterpret_cast<uintptr_t>(a->C) & 15u) == 0;
}

static int shape_for(int ncolv)
{
    if (ncolv <= 8) return 0;
    if (ncolv <= 16) return 1;
    if (ncolv <= 32) return 2;
    if (ncolv <= 64) return 3;
    return 4;
}

static bool tma_can_run(const csrspmm_b200_args* a)
{
    return vector_layout_ok(a) && a->Nd >= 4 && a->Nd <= 512;
}

static int forced_kernel_from_env()
{
    const char* e = std::getenv("CSRSPMM_FORCE_KERNEL");
    if (e == nullptr || *e == 0) return CSRSPMM_B200_KERNEL_AUTO;
    if (!std::strcmp(e, "row")) return CSRSPMM_B200_KERNEL_ROW;
    if (!std::strcmp(e, "merge")) return CSRSPMM_B200_KERNEL_MERGE;
    if (!std::strcmp(e, "tma")) return CSRSPMM_B200_KERNEL_TMA;
    return CSRSPMM_B200_KERNEL_AUTO;
}

int merge_tile_for(int shape, long long num_items, bool* small)
{
    const int groups = CSRSPMM_TUNE_MERGE_THREADS / kShapes[shape].G;
    const int big = groups * kShapes[shape].TG;
    const bool use_small = CSRSPMM_TUNE_MERGE_TG_SMALL < kShapes[shape].TG &&
                           num_items < (long long)big * 148 * CSRSPMM_TUNE_MERGE_SMALL_BELOW_CTAS_PER_SM;
    if (small != nullptr) *small = use_small;
    return use_small ? groups * CSRSPMM_TUNE_MERGE_TG_SMALL : big;
}

static void fill_split_geometry(const csrspmm_b200_args* a, Plan* plan, int tile)
{
    plan->tile = tile;
    plan->num_items = (long long)a->M + a->nnz;
    plan->num_tiles = (plan->num_items + tile - 1) / tile;
    plan->grid = plan->num_tiles;
    plan->carry_ld = ((long long)a->Nd + 3) / 4 * 4;
    plan->carry_row_bytes = align_up((size_t)plan->num_tiles * sizeof(int32_t), 256);
    plan->workspace_bytes =
        plan->carry_row_bytes + (size_t)plan->num_tiles * (size_t)plan->carry_ld * sizeof(float);
}

int make_plan(const csrspmm_b200_args* a, Plan* plan, bool allow_narrow)
{
    int st = check_args(a, false);
    if (st != CSRSPMM_B200_OK) return st;
    *plan = Plan();
    const bool vec = vector_layout_ok(a);
    plan->VW = vec ? 4 : 1;
    plan->ncolv = vec ? a->Nd / 4 : a->Nd;
    plan->num_items = (long long)a->M + a->nnz;

    int kernel = a->kernel;
    bool forced = kernel != CSRSPMM_B200_KERNEL_AUTO;
    if (!forced) {
        kernel = forced_kernel_from_env();
        // an environment override that cannot run this layout falls back to AUTO
        if (kernel == CSRSPMM_B200_KERNEL_TMA && !tma_can_run(a)) kernel = CSRSPMM_B200_KERNEL_AUTO;
    }
    if (kernel == CSRSPMM_B200_KERNEL_AUTO) {
        // Measured on B200: the bulk-copy path completes about one row copy per 80
        // cycles per SM, so it only keeps HBM busy when a row of B is 2 KB (384 < Nd <= 512),
        // where it is 3-4 % ahead of the merge kernel -- provided B is far larger than L2, since
        // an L2-resident B is served faster through the load/store units.  Whole-row mapping
        // wins when the longest row is known and close to the mean; everything else (unknown
        // or skewed row lengths) takes the merge-path kernel.  The entry point asked for does
        // not change the choice.
        const double avg = a->M > 0 ? (double)a->nnz / (double)a->M : 0.0;
        const double row_limit = avg * 4.0 > 64.0 ? avg * 4.0 : 64.0;
        const double b_bytes = (double)a->Kd * (double)a->Nd * 4.0;
        const bool rows_even = a->max_row_nnz > 0 && (double)a->max_row_nnz <= row_limit;
        if (tma_can_run(a) && a->Nd > 384 && b_bytes >= 1073741824.0 && !rows_even)
            kernel = CSRSPMM_B200_KERNEL_TMA;
        else if (rows_even)
            kernel = CSRSPMM_B200_KERNEL_ROW;
        else
            kernel = CSRSPMM_B200_KERNEL_MERGE;
    }
    if (kernel == CSRSPMM_B200_KERNEL_TMA && !tma_can_run(a)) {
        set_last_error("the TMA kernel needs Nd %% 4 == 0, Nd <= 512, ldb/ldc %% 4 == 0 and "
                       "16-byte aligned B and C (Nd=%d ldb=%lld ldc=%lld)",
                       a->Nd, (long long)a->ldb, (long long)a->ldc);
        return CSRSPMM_B200_ERR_UNSUPPORTED;
    }
    plan->kernel = kernel;

    if (kernel == CSRSPMM_B200_KERNEL_TMA) {
        plan->G = 32;
        plan->NV = plan->ncolv <= 32 ? 1 : (plan->ncolv <= 64 ? 2 : 4);
        plan->shape = plan->NV == 1 ? 2 : (plan->NV == 2 ? 3 : 4);
        fill_split_geometry(a, plan, (CSRSPMM_TUNE_MERGE_THREADS / 32) * CSRSPMM_TUNE_TMA_TG);
        const size_t slot = align_up((size_t)a->Nd * 4, 128);
        size_t ring = (size_t)CSRSPMM_TUNE_TMA_SLOTS * slot;          // per warp
        if (ring < (size_t)512 * plan->NV) ring = (size_t)512 * plan->NV;  // must also hold the partial sums
        plan->tma_slot_bytes = slot;
        plan->dynamic_smem = (CSRSPMM_TUNE_MERGE_THREADS / 32) /*warps*/ * ring;
    } else {
        plan->shape = shape_for(plan->ncolv);
        plan->G = kShapes[plan->shape].G;
        plan->NV = kShapes[plan->shape].NV;
        plan->full = plan->VW == 4 && plan->G * plan->NV == plan->ncolv;
        if (CSRSPMM_TUNE_MERGE_NARROW && kernel == CSRSPMM_B200_KERNEL_MERGE && allow_narrow && plan->ncolv >= 1 && plan->ncolv <= 4) {
            // one, two or four column vectors: lane groups of that many lanes (kNarrowShapes)
            plan->narrow = plan->ncolv == 1 ? 1 : (plan->ncolv == 2 ? 2 : 3);
            const ShapeDesc& ns = kNarrowShapes[plan->narrow - 1];
            plan->G = ns.G;
            plan->NV = ns.NV;
            plan->full = plan->VW == 4 && plan->G * plan->NV == plan->ncolv;
            fill_split_geometry(a, plan, (CSRSPMM_TUNE_MERGE_THREADS / ns.G) * ns.TG);
        } else if (kernel == CSRSPMM_B200_KERNEL_MERGE) {
            fill_split_geometry(a, plan, merge_tile_for(plan->shape, plan->num_items, &plan->small_tile));
        } else {
            const int groups = CSRSPMM_TUNE_ROW_THREADS / plan->G;
            plan->grid = ((long long)a->M + groups - 1) / groups;
            plan->low_occupancy = (long long)a->M * plan->G / 32 < 148LL * 8;
#if CSRSPMM_TUNE_ROW_PERSISTENT > 0
            // many short rows: a CTA that lives for four 16-entry rows costs more to start than to
            // run (cfg2: 20.5 -> 18.6 us; 65536 rows of 13: 53 -> 45 us; long rows prefer the
            // finer dynamic balance of one CTA per few rows)
            if (a->nnz <= (long long)CSRSPMM_TUNE_ROW_PERSISTENT_MAX_MEAN * (long long)a->M && plan->grid > 148LL * CSRSPMM_TUNE_ROW_PERSISTENT)
                plan->grid = 148LL * CSRSPMM_TUNE_ROW_PERSISTENT;
#endif
        }
    }
    if (plan->grid > 0x7fffffffLL) {
        set_last_error("grid of %lld CTAs exceeds the launch limit", plan->grid);
        return CSRSPMM_B200_ERR_UNSUPPORTED;
    }
    return CSRSPMM_B200_OK;
}

size_t worst_case_workspace(const csrspmm_b200_args* a, bool any_row_block)
{
    if (check_args(a, false) != CSRSPMM_B200_OK) return 0;
    // sized for the smallest tile any split kernel uses (most CTAs, most carry rows).  A row block of
    // a large matrix may fall under the small-problem threshold although the whole matrix does not,
    // so a caller that multiplies row blocks out of one scratch buffer asks for the small tile
    // whatever the size (any_row_block).
    int tile = (CSRSPMM_TUNE_MERGE_THREADS / 32) * CSRSPMM_TUNE_TMA_TG;  // TMA kernel
    for (int k = 0; k < kNumShapes; ++k) {
        const int t = merge_tile_for(k, any_row_block ? 0 : (long long)a->M + a->nnz, nullptr);
        if (t < tile) tile = t;
    }
    Plan p;
    fill_split_geometry(a, &p, tile);
    return p.workspace_bytes;
}

}  // namespace csrspmm_b200
