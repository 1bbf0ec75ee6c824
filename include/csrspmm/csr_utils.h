// Host-side CSR helpers with the reference's signatures (include/csrspmm/csr_utils.h:6-18).
// Ownership rule kept from the reference: a function that produces a matrix allocates into an
// EMPTY destination (all pointers null) and ends the process with a message when it is not;
// host memory comes from malloc, device memory from cudaMalloc.
#pragma once
#include <csrspmm/matrix.h>

namespace csrspmm {

void csr_alloc_host(CSRMatrix& csr, int height, int width, int nnz);
void csr_free_host(CSRMatrix& csr);

void csr_alloc_device(CSRMatrix& csr, int height, int width, int nnz);
void csr_free_device(CSRMatrix& csr);

// Keeps entries with fabs(v) > tol, columns ascending; also fills max_row_nnz.
void dense2csr(const DenseMatrix& dense, CSRMatrix& csr, float tol = 0.0f);
void csr2dense(const CSRMatrix& csr, DenseMatrix& dense);
void print_csr(const CSRMatrix& csr);
float compression_ratio(const CSRMatrix& csr);

void csr_host2device(const CSRMatrix& hA, CSRMatrix& dA);
void csr_device2host(const CSRMatrix& dA, CSRMatrix& hA);

// Additions: the same conversions for matrices that already live on the device (the reference
// converts on the host only).  d_csr / d_dense must be empty; they are allocated with cudaMalloc
// and filled with exactly what dense2csr / csr2dense would give for the same data.
void dense2csr_device(const DenseMatrix& d_dense, CSRMatrix& d_csr, float tol = 0.0f);
void csr2dense_device(const CSRMatrix& d_csr, DenseMatrix& d_dense);

}  // namespace csrspmm
