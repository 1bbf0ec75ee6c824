// C-callable shim around the REFERENCE's own host functions (test infrastructure only).
//
// oracle/Makefile compiles this file together with the reference's unmodified
// src/host/csr_utils.cpp and src/host/dense_utils.cpp, taken from the reference checkout where
// it lies, into oracle/_ref/.  Nothing from the reference is copied into this repository; only
// the declarations in the reference's include/csrspmm/*.h are used, at build time.  The shim
// lets the Python tests run the reference's dense2csr / csr2dense / dense_gemm_cpu /
// dense_compare on the CPU to pin the oracle restatement and to produce the golden vectors.
#include <csrspmm/csr_utils.h>
#include <csrspmm/dense_utils.h>
#include <csrspmm/matrix.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>

extern "C" {

// dense (H x W, row-major) -> CSR through csrspmm::dense2csr.  Returns nnz; the three arrays
// are malloc'd by the reference and must be released with ref_free.
int ref_dense2csr(int H, int W, const float* dense, float tol, int** row_ptr, int** col_idx,
                  float** values, int* max_row_nnz)
{
    csrspmm::DenseMatrix d;
    d.height = H;
    d.width = W;
    d.data = const_cast<float*>(dense);
    csrspmm::CSRMatrix csr;
    csrspmm::dense2csr(d, csr, tol);
    *row_ptr = csr.row_ptr;
    *col_idx = csr.col_idx;
    *values = csr.values;
    *max_row_nnz = csr.max_row_nnz;
    return csr.nnz;
}

void ref_free(void* p) { std::free(p); }

// CSR -> dense through csrspmm::csr2dense; out must hold H*W floats.
void ref_csr2dense(int H, int W, int nnz, const int* row_ptr, const int* col_idx,
                   const float* values, float* out)
{
    csrspmm::CSRMatrix csr;
    csr.height = H;
    csr.width = W;
    csr.nnz = nnz;
    csr.row_ptr = const_cast<int*>(row_ptr);
    csr.col_idx = const_cast<int*>(col_idx);
    csr.values = const_cast<float*>(values);
    csrspmm::DenseMatrix d;
    csrspmm::csr2dense(csr, d);
    std::memcpy(out, d.data, sizeof(float) * size_t(H) * size_t(W));
    std::free(d.data);
}

// C (M x K) = alpha * A (M x N, dense) * B (N x K) + beta * C through csrspmm::dense_gemm_cpu.
void ref_dense_gemm_cpu(int M, int N, int K, float alpha, float beta, const float* A,
                        const float* B, float* C)
{
    csrspmm::DenseMatrix a, b, c;
    a.height = M; a.width = N; a.data = const_cast<float*>(A);
    b.height = N; b.width = K; b.data = const_cast<float*>(B);
    c.height = M; c.width = K; c.data = C;
    csrspmm::dense_gemm_cpu(M, N, K, alpha, beta, a, b, c);
}

int ref_dense_compare(int H, int W, const float* A, const float* B, float tol)
{
    csrspmm::DenseMatrix a, b;
    a.height = H; a.width = W; a.data = const_cast<float*>(A);
    b.height = H; b.width = W; b.data = const_cast<float*>(B);
    return csrspmm::dense_compare(a, b, tol) ? 1 : 0;
}

float ref_compression_ratio(int H, int W, int nnz)
{
    csrspmm::CSRMatrix csr;
    csr.height = H; csr.width = W; csr.nnz = nnz;
    return csrspmm::compression_ratio(csr);
}

}  // extern "C"
