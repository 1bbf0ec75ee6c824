// cuSPARSE comparator for the benchmark (NOT part of the SpMM library: built into its own shared
// object, loaded only by bench.py).  Times cusparseSpMM on the same device buffers the library
// is timed on, set up as the reference's comparator does (benchmarks/bench_cusparse.cu:126-155:
// 32-bit indices, base 0, fp32, row-major B and C with ld = Nd), with a choice of algorithm and
// an optional cusparseSpMM_preprocess.  Events bracket each repetition on the given stream; an
// optional L2 flush (memset of a caller buffer) runs between repetitions, outside the brackets.
#include <cuda_runtime.h>
#include <cusparse.h>

#include <algorithm>
#include <cstdio>
#include <vector>

extern "C" {

// alg: 0 = CUSPARSE_SPMM_ALG_DEFAULT, 1..3 = CUSPARSE_SPMM_CSR_ALG1..3.
// Returns 0 on success (median seconds in *seconds_out), else a negative cuSPARSE/CUDA code.
int csrspmm_cmp_cusparse_spmm(int M, int Kd, int Nd, long long nnz, const int* row_ptr, const int* col_idx,
                              const float* values, const float* B, float* C, float alpha, float beta, int alg,
                              int preprocess, int warmup, int reps, void* flush_buf, size_t flush_bytes,
                              void* stream_v, double* seconds_out, size_t* buffer_bytes_out)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    cusparseHandle_t h = nullptr;
    cusparseSpMatDescr_t A = nullptr;
    cusparseDnMatDescr_t Bd = nullptr, Cd = nullptr;
    void* buf = nullptr;
    int rc = 0;
    std::vector<cudaEvent_t> ev0(reps), ev1(reps);
    for (int i = 0; i < reps; ++i) {
        cudaEventCreate(&ev0[i]);
        cudaEventCreate(&ev1[i]);
    }
    const cusparseSpMMAlg_t algs[4] = {CUSPARSE_SPMM_ALG_DEFAULT, CUSPARSE_SPMM_CSR_ALG1, CUSPARSE_SPMM_CSR_ALG2,
                                       CUSPARSE_SPMM_CSR_ALG3};
    const cusparseSpMMAlg_t a = algs[alg < 0 || alg > 3 ? 0 : alg];
#define CS(x)                                   \
    do {                                        \
        cusparseStatus_t s__ = (x);             \
        if (s__ != CUSPARSE_STATUS_SUCCESS) {   \
            rc = -1000 - int(s__);              \
            goto done;                          \
        }                                       \
    } while (0)
#define CU(x)                                   \
    do {                                        \
        cudaError_t e__ = (x);                  \
        if (e__ != cudaSuccess) {               \
            rc = -int(e__);                     \
            goto done;                          \
        }                                       \
    } while (0)
    {
        size_t bytes = 0;
        CS(cusparseCreate(&h));
        CS(cusparseSetStream(h, stream));
        CS(cusparseCreateCsr(&A, M, Kd, nnz, (void*)row_ptr, (void*)col_idx, (void*)values, CUSPARSE_INDEX_32I,
                             CUSPARSE_INDEX_32I, CUSPARSE_INDEX_BASE_ZERO, CUDA_R_32F));
        CS(cusparseCreateDnMat(&Bd, Kd, Nd, Nd, (void*)B, CUDA_R_32F, CUSPARSE_ORDER_ROW));
        CS(cusparseCreateDnMat(&Cd, M, Nd, Nd, (void*)C, CUDA_R_32F, CUSPARSE_ORDER_ROW));
        CS(cusparseSpMM_bufferSize(h, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, A,
                                   Bd, &beta, Cd, CUDA_R_32F, a, &bytes));
        if (buffer_bytes_out) *buffer_bytes_out = bytes;
        if (bytes > 0) CU(cudaMalloc(&buf, bytes));
        if (preprocess)
            CS(cusparseSpMM_preprocess(h, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha,
                                       A, Bd, &beta, Cd, CUDA_R_32F, a, buf));
        for (int i = 0; i < warmup + reps; ++i) {
            if (flush_buf) CU(cudaMemsetAsync(flush_buf, 0, flush_bytes, stream));
            if (i >= warmup) CU(cudaEventRecord(ev0[i - warmup], stream));
            CS(cusparseSpMM(h, CUSPARSE_OPERATION_NON_TRANSPOSE, CUSPARSE_OPERATION_NON_TRANSPOSE, &alpha, A, Bd,
                            &beta, Cd, CUDA_R_32F, a, buf));
            if (i >= warmup) CU(cudaEventRecord(ev1[i - warmup], stream));
        }
        CU(cudaStreamSynchronize(stream));
        std::vector<float> ms(reps);
        for (int i = 0; i < reps; ++i) CU(cudaEventElapsedTime(&ms[i], ev0[i], ev1[i]));
        std::sort(ms.begin(), ms.end());
        *seconds_out = double(ms[reps / 2]) * 1e-3;
    }
done:
    if (buf) cudaFree(buf);
    if (Cd) cusparseDestroyDnMat(Cd);
    if (Bd) cusparseDestroyDnMat(Bd);
    if (A) cusparseDestroySpMat(A);
    if (h) cusparseDestroy(h);
    for (int i = 0; i < reps; ++i) {
        cudaEventDestroy(ev0[i]);
        cudaEventDestroy(ev1[i]);
    }
    return rc;
#undef CS
#undef CU
}

}  // extern "C"
