// csrspmm_b200_spmm_tiled: the SpMM in column panels whose slab of B stays in L2 (opt-in).
//
// No counterpart in the reference.  For matrices with long rows and a B much larger than L2 the
// whole-row and merge-path kernels read almost every gathered row of B from HBM; this entry point
// runs one pass of spmm_panel_kernel per panel of `panel_rows` columns of A (= rows of B), so each
// slab is fetched once and then served from L2.  What it costs is one read and one write of the
// running sums of every row that has an entry in the panel, plus a short dependent chain (cursor,
// first chunk, sums) per row and pass.  Measured on B200 that cost eats the saving: on 65 536 rows
// of 328-1000 ascending non-zeros over a B of 1-2 GiB the tiled product runs at 0.9-1.1 x the
// whole-row kernel (whose rows, all of one length, already sweep B together), and on skewed rows
// it is well behind the merge-path kernel.  It is therefore a call of its own, never chosen by
// AUTO, kept for matrices outside those tried.  The result is bit-identical to the whole-row
// kernel's.
#include <cuda_runtime.h>

#include <climits>
#include <cstring>

#include "../kernels/panel_kernel.cuh"
#include "csrspmm_b200.h"
#include "plan.h"

using namespace csrspmm_b200;

namespace {

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

// slab of B that one panel keeps in L2 (126 MB, shared with the lines of the streaming operands):
// 64 MiB measured best among 16-112 MiB on B200 -- smaller slabs mean more passes, each with its
// read and write of the running sums, larger ones start missing
constexpr size_t kSlabBytes = (size_t)64 << 20;

int32_t auto_panel_rows(const csrspmm_b200_args* a)
{
    if (a->Nd <= 0 || a->Kd <= 0) return 0;
    const size_t row_bytes = (size_t)a->ldb * 4;
    size_t rows = kSlabBytes / (row_bytes ? row_bytes : 4);
    rows = rows / 1024 * 1024;
    if (rows < 1024) rows = 1024;
    if (rows >= (size_t)a->Kd) return 0;  // B is no larger than one slab: nothing to tile
    return (int32_t)rows;
}

template <int S, int VW, int FMT>
void launch_panel(const SpmmParams& p, const PanelPass& pp, const Plan& plan, cudaStream_t st)
{
    constexpr int G = kShapes[S].G, NV = kShapes[S].NV;
    constexpr int U = VW == 1 ? 8 : row_unroll(NV);
    constexpr int MINB = row_min_blocks(NV);
    spmm_panel_kernel<G, NV, VW, U, FMT, MINB><<<(unsigned)plan.grid, kRowThreads, 0, st>>>(p, pp);
}

template <int VW, int FMT>
void dispatch_panel(const SpmmParams& p, const PanelPass& pp, const Plan& plan, cudaStream_t st)
{
    switch (plan.shape) {
        case 0: launch_panel<0, VW, FMT>(p, pp, plan, st); break;
        case 1: launch_panel<1, VW, FMT>(p, pp, plan, st); break;
        case 2: launch_panel<2, VW, FMT>(p, pp, plan, st); break;
        case 3: launch_panel<3, VW, FMT>(p, pp, plan, st); break;
        default: launch_panel<4, VW, FMT>(p, pp, plan, st); break;
    }
}

}  // namespace

extern "C" {

int32_t csrspmm_b200_tiled_panel_rows(const csrspmm_b200_args* args)
{
    if (check_args(args, false) != CSRSPMM_B200_OK) return 0;
    return auto_panel_rows(args);
}

size_t csrspmm_b200_tiled_workspace_bytes(const csrspmm_b200_args* args)
{
    if (check_args(args, false) != CSRSPMM_B200_OK) return 0;
    size_t total = align256(((size_t)args->M + 1) * 4);  // cursors
    if (args->beta != 0.0f) total += align256((size_t)args->M * (((size_t)args->Nd + 3) / 4 * 4) * 4);  // running sums
    return total;
}

int csrspmm_b200_spmm_tiled(const csrspmm_b200_args* args, int32_t panel_rows, csrspmm_b200_stream_t stream)
{
    int status = check_args(args, true);
    if (status != CSRSPMM_B200_OK) return status;
    if (args->M == 0 || args->Nd == 0) return CSRSPMM_B200_OK;
    if (panel_rows < 0) {
        set_last_error("spmm_tiled: panel_rows must be positive, or 0 for the library's choice");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (panel_rows == 0) panel_rows = auto_panel_rows(args);
    const long long passes = (panel_rows <= 0 || panel_rows >= args->Kd) ? 1 : ((long long)args->Kd + panel_rows - 1) / panel_rows;

    // geometry of the whole-row kernel for these sizes (lane-group shape, vector width, grid)
    csrspmm_b200_args a = *args;
    a.kernel = CSRSPMM_B200_KERNEL_ROW;
    Plan plan;
    status = make_plan(&a, &plan);
    if (status != CSRSPMM_B200_OK) return status;

    const size_t need = passes > 1 ? csrspmm_b200_tiled_workspace_bytes(args) : 0;
    char* ws = static_cast<char*>(args->workspace);
    bool owned = false;
    if (need > 0) {
        if (ws == nullptr) {
            cudaError_t e = cudaMallocAsync(reinterpret_cast<void**>(&ws), need, st);
            if (e != cudaSuccess) {
                set_last_error("spmm_tiled: cudaMallocAsync(%zu) failed: %s", need, cudaGetErrorString(e));
                return CSRSPMM_B200_ERR_CUDA;
            }
            owned = true;
        } else if (args->workspace_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 255u) != 0) {
            set_last_error("spmm_tiled: workspace of %zu bytes at %p: need %zu bytes, 256-byte aligned",
                           args->workspace_bytes, args->workspace, need);
            return CSRSPMM_B200_ERR_WORKSPACE;
        }
    }

    SpmmParams p;
    std::memset(&p, 0, sizeof(p));
    p.M = a.M;
    p.Kd = a.Kd;
    p.Nd = a.Nd;
    p.nnz = (int)a.nnz;
    p.ncolv = plan.ncolv;
    p.num_items = plan.num_items;
    p.row_ptr = a.row_ptr;
    p.rp_base = a.row_ptr_base;
    p.col_idx = a.col_idx;
    p.values = a.values;
    p.value_scale = a.value_scale;
    p.B = a.B;
    p.ldb = a.ldb;
    p.ldb_bytes = (unsigned)(a.ldb * 4);
    p.C = a.C;
    p.ldc = a.ldc;
    p.alpha = a.alpha;
    p.beta = a.beta;
    p.status_word = a.status_word;

    PanelPass pp;
    std::memset(&pp, 0, sizeof(pp));
    pp.cursor = reinterpret_cast<int*>(ws);
    if (a.beta != 0.0f && passes > 1) {
        pp.partial = reinterpret_cast<float*>(ws + align256(((size_t)a.M + 1) * 4));
        pp.ldp = ((long long)a.Nd + 3) / 4 * 4;
    } else {
        pp.partial = a.C;
        pp.ldp = a.ldc;
    }

    const bool e2m1 = a.value_format == CSRSPMM_B200_VALUES_E2M1;
    cudaError_t err = cudaSuccess;
    for (long long t = 0; t < passes && err == cudaSuccess; ++t) {
        pp.first = t == 0;
        pp.last = t == passes - 1;
        pp.col_limit = pp.last ? INT_MAX : (int)((t + 1) * panel_rows);
        if (plan.VW == 4) {
            if (e2m1) dispatch_panel<4, kValuesE2M1>(p, pp, plan, st);
            else dispatch_panel<4, kValuesF32>(p, pp, plan, st);
        } else {
            if (e2m1) dispatch_panel<1, kValuesE2M1>(p, pp, plan, st);
            else dispatch_panel<1, kValuesF32>(p, pp, plan, st);
        }
        err = cudaGetLastError();
    }
    if (owned) {
        cudaError_t ferr = cudaFreeAsync(ws, st);
        if (err == cudaSuccess) err = ferr;
    }
    if (err != cudaSuccess) {
        set_last_error("spmm_tiled: kernel launch failed: %s", cudaGetErrorString(err));
        return CSRSPMM_B200_ERR_CUDA;
    }
    return CSRSPMM_B200_OK;
}

}  // extern "C"
