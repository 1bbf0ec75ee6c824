// csrspmm::csr_* host utilities (declared in include/csrspmm/csr_utils.h).
//
// Same contract as the reference's src/host/csr_utils.cpp:13-239: allocate only into an empty
// destination, malloc/free on the host and cudaMalloc/cudaFree on the device, fatal message +
// exit(1) on misuse, csr_free_* zero the dimensions, the host<->device copies carry max_row_nnz.
// Written afresh with every size computed in size_t, so that matrices whose height*width or
// byte counts pass 2^31 are handled (the reference multiplies ints, src/host/csr_utils.cpp:88,193).
#include <csrspmm/csr_utils.h>
#include <csrspmm/error_check.h>
#include <csrspmm/matrix.h>

#include "csrspmm_b200.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace csrspmm {

namespace {

[[noreturn]] void die(const char* msg)
{
    std::fprintf(stderr, "%s\n", msg);
    std::exit(1);
}

bool any_pointer(const CSRMatrix& m) { return m.row_ptr || m.col_idx || m.values; }
bool all_pointers(const CSRMatrix& m) { return m.row_ptr && m.col_idx && m.values; }

void set_dims(CSRMatrix& m, int height, int width, int nnz)
{
    m.height = height;
    m.width = width;
    m.nnz = nnz;
}

size_t rowptr_bytes(int height) { return (size_t(height) + 1) * sizeof(int); }

}  // namespace

void csr_alloc_host(CSRMatrix& csr, int height, int width, int nnz)
{
    if (any_pointer(csr)) die("csr_alloc_host error: already allocated host memory.");
    set_dims(csr, height, width, nnz);
    // malloc(0) may return null; keep the three pointers non-null so the matrix counts as allocated
    csr.row_ptr = static_cast<int*>(std::malloc(rowptr_bytes(height)));
    csr.col_idx = static_cast<int*>(std::malloc(std::max<size_t>(size_t(nnz) * sizeof(int), 4)));
    csr.values = static_cast<float*>(std::malloc(std::max<size_t>(size_t(nnz) * sizeof(float), 4)));
    if (!all_pointers(csr)) die("csr_alloc_host: malloc failed");
}

void csr_free_host(CSRMatrix& csr)
{
    std::free(csr.row_ptr);
    std::free(csr.col_idx);
    std::free(csr.values);
    csr.row_ptr = nullptr;
    csr.col_idx = nullptr;
    csr.values = nullptr;
    set_dims(csr, 0, 0, 0);
    csr.max_row_nnz = 0;
}

void csr_alloc_device(CSRMatrix& csr, int height, int width, int nnz)
{
    if (any_pointer(csr)) die("csr_alloc_device error: already allocated device memory.");
    set_dims(csr, height, width, nnz);
    cudaCheck(cudaMalloc(reinterpret_cast<void**>(&csr.row_ptr), rowptr_bytes(height)));
    cudaCheck(cudaMalloc(reinterpret_cast<void**>(&csr.col_idx), std::max<size_t>(size_t(nnz) * sizeof(int), 4)));
    cudaCheck(cudaMalloc(reinterpret_cast<void**>(&csr.values), std::max<size_t>(size_t(nnz) * sizeof(float), 4)));
}

void csr_free_device(CSRMatrix& csr)
{
    if (csr.row_ptr) cudaCheck(cudaFree(csr.row_ptr));
    if (csr.col_idx) cudaCheck(cudaFree(csr.col_idx));
    if (csr.values) cudaCheck(cudaFree(csr.values));
    csr.row_ptr = nullptr;
    csr.col_idx = nullptr;
    csr.values = nullptr;
    set_dims(csr, 0, 0, 0);
    csr.max_row_nnz = 0;
}

void dense2csr(const DenseMatrix& dense, CSRMatrix& csr, float tol)
{
    if (!dense.data || dense.height <= 0 || dense.width <= 0) die("dense2csr: invalid dense matrix");
    if (any_pointer(csr)) die("dense2csr error: destination must be null.");

    const size_t H = size_t(dense.height), W = size_t(dense.width);
    size_t count = 0;
    for (size_t i = 0; i < H * W; ++i) count += std::fabs(dense.data[i]) > tol ? 1 : 0;
    if (count > size_t(0x7fffffff)) die("dense2csr: more than 2^31-1 non-zeros");

    csr_alloc_host(csr, dense.height, dense.width, int(count));

    int next = 0, longest = 0;
    csr.row_ptr[0] = 0;
    for (size_t r = 0; r < H; ++r) {
        const float* row = dense.data + r * W;
        const int begin = next;
        for (size_t c = 0; c < W; ++c) {
            if (std::fabs(row[c]) > tol) {
                csr.col_idx[next] = int(c);
                csr.values[next] = row[c];
                ++next;
            }
        }
        csr.row_ptr[r + 1] = next;
        longest = std::max(longest, next - begin);
    }
    csr.max_row_nnz = longest;
}

void csr2dense(const CSRMatrix& csr, DenseMatrix& dense)
{
    if (!all_pointers(csr) || csr.height <= 0 || csr.width <= 0) die("csr2dense: invalid csr");
    if (dense.data != nullptr) die("csr2dense error: destination must be null.");

    const size_t H = size_t(csr.height), W = size_t(csr.width);
    dense.data = static_cast<float*>(std::calloc(H * W, sizeof(float)));
    if (!dense.data) die("csr2dense: malloc failed");
    dense.height = csr.height;
    dense.width = csr.width;
    for (size_t r = 0; r < H; ++r)
        for (int p = csr.row_ptr[r]; p < csr.row_ptr[r + 1]; ++p)
            dense.data[r * W + size_t(csr.col_idx[p])] = csr.values[p];
}

void print_csr(const CSRMatrix& csr)
{
    std::printf("CSRMatrix (HOST): %d×%d, nnz=%d, max_row_nnz=%d\n", csr.height, csr.width, csr.nnz,
                csr.max_row_nnz);
    std::printf("row_ptr: [ ");
    for (int i = 0; i <= csr.height; ++i) std::printf("%d ", csr.row_ptr[i]);
    std::printf("]\ncol_idx: [ ");
    for (int i = 0; i < csr.nnz; ++i) std::printf("%d ", csr.col_idx[i]);
    std::printf("]\nvalues:  [ ");
    for (int i = 0; i < csr.nnz; ++i) std::printf("%g ", csr.values[i]);
    std::printf("]\n");
}

float compression_ratio(const CSRMatrix& csr)
{
    // dense element count over stored words (values + column indices + row offsets)
    const double dense_words = double(csr.height) * double(csr.width);
    const double csr_words = 2.0 * double(csr.nnz) + double(csr.height) + 1.0;
    return float(dense_words / csr_words);
}

void csr_host2device(const CSRMatrix& hA, CSRMatrix& dA)
{
    if (!all_pointers(hA)) die("csr_host2device: host CSRMatrix invalid");
    if (any_pointer(dA)) die("csr_host2device error: destination must be null.");
    csr_alloc_device(dA, hA.height, hA.width, hA.nnz);
    dA.max_row_nnz = hA.max_row_nnz;
    cudaCheck(cudaMemcpy(dA.row_ptr, hA.row_ptr, rowptr_bytes(hA.height), cudaMemcpyHostToDevice));
    cudaCheck(cudaMemcpy(dA.col_idx, hA.col_idx, size_t(hA.nnz) * sizeof(int), cudaMemcpyHostToDevice));
    cudaCheck(cudaMemcpy(dA.values, hA.values, size_t(hA.nnz) * sizeof(float), cudaMemcpyHostToDevice));
}

void csr_device2host(const CSRMatrix& dA, CSRMatrix& hA)
{
    if (!all_pointers(dA)) die("csr_device2host: device pointer invalid");
    if (any_pointer(hA)) die("csr_device2host error: destination must be null.");
    csr_alloc_host(hA, dA.height, dA.width, dA.nnz);
    hA.max_row_nnz = dA.max_row_nnz;
    cudaCheck(cudaMemcpy(hA.row_ptr, dA.row_ptr, rowptr_bytes(dA.height), cudaMemcpyDeviceToHost));
    cudaCheck(cudaMemcpy(hA.col_idx, dA.col_idx, size_t(dA.nnz) * sizeof(int), cudaMemcpyDeviceToHost));
    cudaCheck(cudaMemcpy(hA.values, dA.values, size_t(dA.nnz) * sizeof(float), cudaMemcpyDeviceToHost));
}

void dense2csr_device(const DenseMatrix& d_dense, CSRMatrix& d_csr, float tol)
{
    if (!d_dense.data || d_dense.height <= 0 || d_dense.width <= 0) die("dense2csr_device: invalid dense matrix");
    if (any_pointer(d_csr)) die("dense2csr_device error: destination must be null.");
    int* row_ptr = nullptr;
    cudaCheck(cudaMalloc(reinterpret_cast<void**>(&row_ptr), rowptr_bytes(d_dense.height)));
    int64_t nnz = 0;
    int32_t longest = 0;
    if (csrspmm_b200_dense2csr_count(d_dense.height, d_dense.width, d_dense.data, d_dense.width, tol, row_ptr, &nnz,
                                     &longest, nullptr) != CSRSPMM_B200_OK)
        die(csrspmm_b200_last_error());
    set_dims(d_csr, d_dense.height, d_dense.width, int(nnz));
    d_csr.row_ptr = row_ptr;
    d_csr.max_row_nnz = longest;
    cudaCheck(cudaMalloc(reinterpret_cast<void**>(&d_csr.col_idx), std::max<size_t>(size_t(nnz) * sizeof(int), 4)));
    cudaCheck(cudaMalloc(reinterpret_cast<void**>(&d_csr.values), std::max<size_t>(size_t(nnz) * sizeof(float), 4)));
    if (csrspmm_b200_dense2csr_fill(d_dense.height, d_dense.width, d_dense.data, d_dense.width, tol, d_csr.row_ptr,
                                    d_csr.col_idx, d_csr.values, nullptr) != CSRSPMM_B200_OK)
        die(csrspmm_b200_last_error());
    cudaCheck(cudaDeviceSynchronize());
}

void csr2dense_device(const CSRMatrix& d_csr, DenseMatrix& d_dense)
{
    if (!all_pointers(d_csr) || d_csr.height <= 0 || d_csr.width <= 0) die("csr2dense_device: invalid csr");
    if (d_dense.data != nullptr) die("csr2dense_device error: destination must be null.");
    d_dense.height = d_csr.height;
    d_dense.width = d_csr.width;
    cudaCheck(cudaMalloc(reinterpret_cast<void**>(&d_dense.data),
                         size_t(d_csr.height) * size_t(d_csr.width) * sizeof(float)));
    if (csrspmm_b200_csr2dense(d_csr.height, d_csr.width, d_csr.row_ptr, d_csr.col_idx, d_csr.values, d_dense.data,
                               d_csr.width, nullptr) != CSRSPMM_B200_OK)
        die(csrspmm_b200_last_error());
    cudaCheck(cudaDeviceSynchronize());
}

}  // namespace csrspmm
