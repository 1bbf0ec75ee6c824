// Declarations of the six kernel symbols the reference publishes in namespace csrspmm::kernel
// (include/csrspmm/kernels.h:6-71 there), kept so that code including <csrspmm/csrspmm.h>
// still compiles.  Argument order: (M, N, K) = (rows of A, columns of A, columns of B).
//
// They are plain compatibility kernels inside the library (one thread per output element, or
// one warp per row); nothing in the library launches them.  The fast path is reached through
// csrspmm::launch_* / csrspmm::spmm, which call the sm_100a kernel library.
#pragma once
#include <csrspmm/matrix.h>

namespace csrspmm::kernel {

__global__ void csrspmm_naive(int M, int N, int K, float alpha, float beta,
                              const float* __restrict__ A_values, const int* __restrict__ A_col_idx,
                              const int* __restrict__ A_row_ptr, const float* __restrict__ B,
                              float* __restrict__ C);

__global__ void csrspmm_naive_smem(int M, int N, int K, float alpha, float beta,
                                   const float* __restrict__ A_values, const int* __restrict__ A_col_idx,
                                   const int* __restrict__ A_row_ptr, const float* __restrict__ B,
                                   float* __restrict__ C);

__global__ void csrspmm_warp_per_row(int M, int N, int K, float alpha, float beta,
                                     const float* __restrict__ A_values, const int* __restrict__ A_col_idx,
                                     const int* __restrict__ A_row_ptr, const float* __restrict__ B,
                                     float* __restrict__ C);

__global__ void csrspmm_warp_per_row_fp4(int M, int N, int K, float alpha, float beta,
                                         const float* __restrict__ A_values,
                                         const int* __restrict__ A_col_idx,
                                         const int* __restrict__ A_row_ptr, const float* __restrict__ B,
                                         float* __restrict__ C);

__global__ void csrspmm_warp_per_row_smem(int M, int N, int K, float alpha, float beta,
                                          const float* __restrict__ A_values,
                                          const int* __restrict__ A_col_idx,
                                          const int* __restrict__ A_row_ptr, const int A_max_row_nnz,
                                          const float* __restrict__ B, float* __restrict__ C);

__global__ void csrspmm_warp_per_row_smem_fp4(int M, int N, int K, float alpha, float beta,
                                              const float* __restrict__ A_values,
                                              const int* __restrict__ A_col_idx,
                                              const int* __restrict__ A_row_ptr, const int A_max_row_nnz,
                                              const float* __restrict__ B, float* __restrict__ C);

}  // namespace csrspmm::kernel
