// cudaCheck / cublasCheck / cusparseCheck: print the failure with file and line, then end the
// process.  Same macro names and fatal behaviour as the reference's
// include/csrspmm/error_check.h:11-40, which its benchmarks use directly.  The macros name the
// check functions unqualified, as the reference's do: use them inside namespace csrspmm or
// after a using-declaration.
#pragma once
#include <cstdio>
#include <cstdlib>
#include <iostream>

#include <cublas_v2.h>
#include <cuda_runtime.h>
#include <cusparse.h>

namespace csrspmm {

inline void cudaErrorCheck(cudaError_t err, const char* file, int line)
{
    if (err == cudaSuccess) return;
    std::fprintf(stderr, "CUDA Error: %s at %s:%d\n", cudaGetErrorString(err), file, line);
    std::exit(EXIT_FAILURE);
}

inline void cublasErrorCheck(cublasStatus_t status, const char* file, int line)
{
    if (status == CUBLAS_STATUS_SUCCESS) return;
    std::fprintf(stderr, "cuBLAS Error: %d at %s:%d\n", int(status), file, line);
    std::exit(EXIT_FAILURE);
}

inline void cusparseErrorCheck(cusparseStatus_t status, const char* file, int line)
{
    if (status == CUSPARSE_STATUS_SUCCESS) return;
    std::fprintf(stderr, "cuSPARSE error %d at %s:%d\n", int(status), file, line);
    std::exit(EXIT_FAILURE);
}

#define cudaCheck(err) (cudaErrorCheck(err, __FILE__, __LINE__))
#define cublasCheck(err) (cublasErrorCheck(err, __FILE__, __LINE__))
#define cusparseCheck(err) (cusparseErrorCheck(err, __FILE__, __LINE__))

}  // namespace csrspmm
