// The six asynchronous launch functions of the reference (include/csrspmm/spmm_launcher.cuh:8-43
// there).  Each enqueues C = alpha*A*B + beta*C on the legacy default stream and returns without
// waiting.  All pointers inside A, B, C are device pointers.
//
// Unlike the reference's launchers (src/host/spmm_launcher.cu:11-171), which use one fixed grid
// per function and report nothing, these hand the problem to the sm_100a kernel library, which
// picks the kernel from the row-length statistics and the dense width; a failed launch prints
// its reason on stderr and is remembered until csrspmm::spmm (or csrspmm::last_launch_status)
// asks for it.
#pragma once

#include <csrspmm/config.h>
#include <csrspmm/matrix.h>

namespace csrspmm {

void launch_naive(const CSRMatrix& A, const DenseMatrix& B, DenseMatrix& C, float alpha, float beta);

void launch_naive_smem(const CSRMatrix& A, const DenseMatrix& B, DenseMatrix& C, float alpha, float beta);

void launch_warp_per_row(const CSRMatrix& A, const DenseMatrix& B, DenseMatrix& C, float alpha, float beta);

void launch_warp_per_row_fp4(const CSRMatrix& A, const DenseMatrix& B, DenseMatrix& C, float alpha, float beta);

void launch_warp_per_row_smem(const CSRMatrix& A, const DenseMatrix& B, DenseMatrix& C, float alpha, float beta);

void launch_warp_per_row_smem_fp4(const CSRMatrix& A, const DenseMatrix& B, DenseMatrix& C, float alpha,
                                  float beta);

// Addition: status (a csrspmm_b200_status value, 0 = ok) of the most recent launch_* call on
// this thread; reading it clears it.
int last_launch_status();

}  // namespace csrspmm
