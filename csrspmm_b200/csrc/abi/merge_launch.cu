// Starts the merge-path kernels (declared in launch.h).  One place for every entry point that runs
// them: csrspmm_b200_spmm, csrspmm_b200_spmm_noalloc, the row blocks and column panels of
// csrspmm_b200_spmm_host.  Stands where the reference's launchers fix their geometry
// (src/host/spmm_launcher.cu:63-70).
//
#include <cuda_runtime.h>

#include "../kernels/merge_kernel.cuh"
#include "launch.h"

namespace csrspmm_b200 {

namespace {

template <int S, int VW, int FMT>
void launch_merge(const SpmmParams& p, const Plan& plan, cudaStream_t st)
{
    constexpr int G = kShapes[S].G, NV = kShapes[S].NV, TG = kShapes[S].TG;
    constexpr int TGS = CSRSPMM_TUNE_MERGE_TG_SMALL < TG ? CSRSPMM_TUNE_MERGE_TG_SMALL : TG;
    constexpr int U = VW == 1 ? 8 : merge_unroll(NV);
    const unsigned grid = (unsigned)plan.grid;
    if (plan.small_tile) {  // few items: smaller tiles, more CTAs
        if (VW == 4 && plan.full) spmm_merge_kernel<G, NV, VW, TGS, U, FMT, (VW == 4)><<<grid, kMergeThreads, 0, st>>>(p);
        else spmm_merge_kernel<G, NV, VW, TGS, U, FMT, false><<<grid, kMergeThreads, 0, st>>>(p);
    } else {
        if (VW == 4 && plan.full) spmm_merge_kernel<G, NV, VW, TG, U, FMT, (VW == 4)><<<grid, kMergeThreads, 0, st>>>(p);
        else spmm_merge_kernel<G, NV, VW, TG, U, FMT, false><<<grid, kMergeThreads, 0, st>>>(p);
    }
}

// very narrow dense operands: lane groups of 1, 2 or 4 lanes (kNarrowShapes)
template <int K, int VW, int FMT>
void launch_merge_narrow(const SpmmParams& p, const Plan& plan, cudaStream_t st)
{
    constexpr int G = kNarrowShapes[K].G, NV = kNarrowShapes[K].NV, TG = kNarrowShapes[K].TG;
    constexpr int U = VW == 1 ? 8 : merge_unroll(NV);
    const unsigned grid = (unsigned)plan.grid;
    if (VW == 4 && plan.full) spmm_merge_kernel<G, NV, VW, TG, U, FMT, (VW == 4)><<<grid, kMergeThreads, 0, st>>>(p);
    else spmm_merge_kernel<G, NV, VW, TG, U, FMT, false><<<grid, kMergeThreads, 0, st>>>(p);
}

template <int VW, int FMT>
void dispatch_merge(const SpmmParams& p, const Plan& plan, cudaStream_t st)
{
    switch (plan.narrow) {
        case 1: launch_merge_narrow<0, VW, FMT>(p, plan, st); return;
        case 2: launch_merge_narrow<1, VW, FMT>(p, plan, st); return;
        case 3: launch_merge_narrow<2, VW, FMT>(p, plan, st); return;
        default: break;
    }
    switch (plan.shape) {
        case 0: launch_merge<0, VW, FMT>(p, plan, st); break;
        case 1: launch_merge<1, VW, FMT>(p, plan, st); break;
        case 2: launch_merge<2, VW, FMT>(p, plan, st); break;
        case 3: launch_merge<3, VW, FMT>(p, plan, st); break;
        default: launch_merge<4, VW, FMT>(p, plan, st); break;
    }
}

}  // namespace

cudaError_t launch_merge_kernel(const SpmmParams& p, const Plan& plan, bool e2m1, cudaStream_t st)
{
    if (plan.VW == 4) {
        if (e2m1) dispatch_merge<4, kValuesE2M1>(p, plan, st);
        else dispatch_merge<4, kValuesF32>(p, plan, st);
    } else {
        if (e2m1) dispatch_merge<1, kValuesE2M1>(p, plan, st);
        else dispatch_merge<1, kValuesF32>(p, plan, st);
    }
    return cudaGetLastError();
}

cudaError_t launch_fixup_kernel(const SpmmParams& p, const Plan& plan, cudaStream_t st)
{
    const int warps = 256 / 32;
    const unsigned grid = (unsigned)((plan.num_tiles + warps - 1) / warps);
    if (plan.VW == 4) spmm_fixup_kernel<4><<<grid, 256, 0, st>>>(p, (int)plan.num_tiles);
    else spmm_fixup_kernel<1><<<grid, 256, 0, st>>>(p, (int)plan.num_tiles);
    return cudaGetLastError();
}

}  // namespace csrspmm_b200
