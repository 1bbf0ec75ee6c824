// Plain-data views of the two operand kinds, laid out exactly as the reference lays them out
// (include/csrspmm/matrix.h:6-23 there), because its callers fill them field by field:
//   CSRMatrix   { int height, width, nnz; int* row_ptr; int* col_idx; float* values; int max_row_nnz; }
//   DenseMatrix { int height, width; float* data; }      row-major, leading dimension == width
// The same struct describes host or device memory; which one is a convention of the function
// that receives it.  Sizes stay `int` for layout compatibility; the library computes every
// byte count and element offset in 64 bits.
#pragma once
#include <cuda_runtime.h>

namespace csrspmm {

struct CSRMatrix {
    int height = 0;  // rows
    int width = 0;   // columns
    int nnz = 0;     // stored non-zeros

    int* row_ptr = nullptr;   // height + 1 offsets into col_idx / values
    int* col_idx = nullptr;   // nnz column indices
    float* values = nullptr;  // nnz values

    int max_row_nnz = 0;  // longest row; filled by dense2csr, carried by the copies
};

struct DenseMatrix {
    int height = 0;
    int width = 0;
    float* data = nullptr;  // height * width floats
};

}  // namespace csrspmm
