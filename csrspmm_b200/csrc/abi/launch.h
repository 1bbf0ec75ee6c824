// Launch helpers shared by the entry points (cabi.cu, noalloc.cu, schedule.cu): one place fills the
// kernel parameter block from the argument block and one place starts the merge-path kernel and
// its fix-up, so that the entry points cannot drift apart.  Stands where the reference's launchers
// compute their fixed geometry (src/host/spmm_launcher.cu:17-25, 63-70).
#pragma once

#include <cuda_runtime.h>

#include "../kernels/common.cuh"
#include "csrspmm_b200.h"
#include "plan.h"

namespace csrspmm_b200 {

// Everything of SpmmParams except the scratch pointers (carry_row, carry_val, carry_ld).
void fill_params(const csrspmm_b200_args* a, const Plan& plan, SpmmParams* p);

// Points the carries of a split kernel at `workspace` (plan.workspace_bytes bytes, 256-byte aligned).
void set_carry_scratch(const Plan& plan, void* workspace, SpmmParams* p);

// The merge-path kernel for plan.shape / VW / small_tile / full, then nothing else; returns the
// launch error.  The fix-up is a separate call because a scheduled product runs other kernels
// in between.
cudaError_t launch_merge_kernel(const SpmmParams& p, const Plan& plan, bool e2m1, cudaStream_t st);
cudaError_t launch_fixup_kernel(const SpmmParams& p, const Plan& plan, cudaStream_t st);
// The whole-row kernel for a plan whose kernel is ROW.
cudaError_t launch_row_kernel(const SpmmParams& p, const Plan& plan, bool e2m1, cudaStream_t st);

// A product under a schedule (args.schedule != NULL): schedule.cu.
int enqueue_scheduled(const csrspmm_b200_args* a, cudaStream_t st);
// Scratch of that product; 0 when the schedule is empty or does not apply.
size_t scheduled_workspace_bytes(const csrspmm_b200_args* a);
// True when args.schedule is set and holds long rows, i.e. enqueue_scheduled will be used.
bool schedule_applies(const csrspmm_b200_args* a);

}  // namespace csrspmm_b200
