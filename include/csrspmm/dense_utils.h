// Host-side dense-matrix helpers with the reference's signatures
// (include/csrspmm/dense_utils.h:7-32).  Same ownership rule as csr_utils.h.
#pragma once
#include <csrspmm/matrix.h>

namespace csrspmm {

void dense_alloc_host(DenseMatrix& A, int height, int width);
void dense_alloc_device(DenseMatrix& A, int height, int width);

void dense_free_host(DenseMatrix& A);
void dense_free_device(DenseMatrix& A);

void dense_host2device(const DenseMatrix& hA, DenseMatrix& dA);
void dense_device2host(const DenseMatrix& dA, DenseMatrix& hA);

// Uniform values in [low, high); an entry is zero with probability `sparsity`; integer_values
// truncates toward zero.  One rand_r stream seeded with 1234 runs through the whole matrix.
void dense_init_random(DenseMatrix& A, float low = -1.0f, float hight = 1.0f, float sparsity = 0.0f,
                       bool integer_values = false);

void print_dense(const DenseMatrix& A);

// true when shapes agree and every |a - b| <= tol; prints the first mismatch.
bool dense_compare(const DenseMatrix& A, const DenseMatrix& B, float tol = 1e-4f);

// C (M x K) = alpha * A (M x N) * B (N x K) + beta * C, plain triple loop on the host.
void dense_gemm_cpu(int M, int N, int K, float alpha, float beta, const DenseMatrix& A,
                    const DenseMatrix& B, DenseMatrix& C);

}  // namespace csrspmm
