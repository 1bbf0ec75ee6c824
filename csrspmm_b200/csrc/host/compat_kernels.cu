// Definitions of the six kernel symbols declared in include/csrspmm/kernels.h.
//
// The reference exposes its __global__ functions in a public header
// (include/csrspmm/kernels.h:6-71) although only its own launchers start them.  These are simple,
// correct stand-ins with the same signatures so that the header links: one thread per output
// element for the two "naive" names, one warp per row for the four "warp_per_row" names.  The
// library's own launchers never use them.
#include <csrspmm/kernels.h>

namespace csrspmm::kernel {

namespace {

__device__ __forceinline__ void finish(float* c, float alpha, float beta, float sum)
{
    *c = alpha * sum + (beta != 0.0f ? beta * *c : 0.0f);
}

__device__ void element_per_thread(int M, int K, float alpha, float beta, const float* vals,
                                   const int* cols, const int* row_ptr, const float* B, float* C)
{
    const int col = blockIdx.x * blockDim.x + threadIdx.x;
    const int row = blockIdx.y * blockDim.y + threadIdx.y;
    if (row >= M || col >= K) return;
    float sum = 0.0f;
    for (int j = row_ptr[row]; j < row_ptr[row + 1]; ++j)
        sum = fmaf(vals[j], B[(size_t)cols[j] * K + col], sum);
    finish(C + (size_t)row * K + col, alpha, beta, sum);
}

__device__ void row_per_warp(int M, int K, float alpha, float beta, const float* vals, const int* cols,
                             const int* row_ptr, const float* B, float* C)
{
    const int row = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (row >= M) return;
    for (int col = threadIdx.x % 32; col < K; col += 32) {
        float sum = 0.0f;
        for (int j = row_ptr[row]; j < row_ptr[row + 1]; ++j)
            sum = fmaf(vals[j], B[(size_t)cols[j] * K + col], sum);
        finish(C + (size_t)row * K + col, alpha, beta, sum);
    }
}

}  // namespace

__global__ void csrspmm_naive(int M, int, int K, float alpha, float beta, const float* __restrict__ A_values,
                              const int* __restrict__ A_col_idx, const int* __restrict__ A_row_ptr,
                              const float* __restrict__ B, float* __restrict__ C)
{
    element_per_thread(M, K, alpha, beta, A_values, A_col_idx, A_row_ptr, B, C);
}

__global__ void csrspmm_naive_smem(int M, int, int K, float alpha, float beta,
                                   const float* __restrict__ A_values, const int* __restrict__ A_col_idx,
                                   const int* __restrict__ A_row_ptr, const float* __restrict__ B,
                                   float* __restrict__ C)
{
    element_per_thread(M, K, alpha, beta, A_values, A_col_idx, A_row_ptr, B, C);
}

__global__ void csrspmm_warp_per_row(int M, int, int K, float alpha, float beta,
                                     const float* __restrict__ A_values, const int* __restrict__ A_col_idx,
                                     const int* __restrict__ A_row_ptr, const float* __restrict__ B,
                                     float* __restrict__ C)
{
    row_per_warp(M, K, alpha, beta, A_values, A_col_idx, A_row_ptr, B, C);
}

__global__ void csrspmm_warp_per_row_fp4(int M, int, int K, float alpha, float beta,
                                         const float* __restrict__ A_values,
                                         const int* __restrict__ A_col_idx,
                                         const int* __restrict__ A_row_ptr, const float* __restrict__ B,
                                         float* __restrict__ C)
{
    row_per_warp(M, K, alpha, beta, A_values, A_col_idx, A_row_ptr, B, C);
}

__global__ void csrspmm_warp_per_row_smem(int M, int, int K, float alpha, float beta,
                                          const float* __restrict__ A_values,
                                          const int* __restrict__ A_col_idx,
                                          const int* __restrict__ A_row_ptr, const int,
                                          const float* __restrict__ B, float* __restrict__ C)
{
    row_per_warp(M, K, alpha, beta, A_values, A_col_idx, A_row_ptr, B, C);
}

__global__ void csrspmm_warp_per_row_smem_fp4(int M, int, int K, float alpha, float beta,
                                              const float* __restrict__ A_values,
                                              const int* __restrict__ A_col_idx,
                                              const int* __restrict__ A_row_ptr, const int,
                                              const float* __restrict__ B, float* __restrict__ C)
{
    row_per_warp(M, K, alpha, beta, A_values, A_col_idx, A_row_ptr, B, C);
}

}  // namespace csrspmm::kernel
