// C-callable shim around the REFERENCE's own GPU launchers (test infrastructure only).
//
// oracle/Makefile (target refgpu) compiles this file together with the reference's unmodified
// src/device/*.cu and src/host/spmm_launcher.cu for sm_100a, with the reference's own CUDA flags
// (-O3 --use_fast_math, relocatable device code), into oracle/_ref/libcsrspmm_ref_gpu.so.  Nothing
// of the reference is copied into this repository.  The GPU tests use it to compare this
// library's results with what the reference's kernels compute on the same device buffers, and to
// time those kernels next to ours.  csrspmm_naive_smem is never launched: its barrier sits in
// divergent code (src/device/csrspmm_naive_smem.cu:19,37,40).
#include <cuda_runtime.h>

#include <csrspmm/matrix.h>
#include <csrspmm/spmm_launcher.cuh>

extern "C" {

// algo: 0 Naive, 2 WarpPerRow, 3 WarpPerRowFp4, 4 WarpPerRowSmem, 5 WarpPerRowSmemFp4 (the values
// of csrspmm::Algorithm; 1 = NaiveSmem is refused).  Device pointers, legacy default stream,
// asynchronous.  Returns the cudaError_t of the launch (0 = ok), -1 for a refused algorithm,
// -2 when the shapes would overflow the reference's 32-bit element offsets.
int ref_gpu_spmm(int algo, int M, int Kd, int Nd, int nnz, int* row_ptr, int* col_idx, float* values, int max_row_nnz,
                 float* B, float* C, float alpha, float beta)
{
    // the kernels index B[col * K + c] and C[row * K + c] in int (src/device/csrspmm_naive.cu:34,38)
    if ((long long)Kd * Nd > 0x7fffffffLL || (long long)M * Nd > 0x7fffffffLL) return -2;
    csrspmm::CSRMatrix A;
    A.height = M;
    A.width = Kd;
    A.nnz = nnz;
    A.row_ptr = row_ptr;
    A.col_idx = col_idx;
    A.values = values;
    A.max_row_nnz = max_row_nnz;
    csrspmm::DenseMatrix Bm, Cm;
    Bm.height = Kd;
    Bm.width = Nd;
    Bm.data = B;
    Cm.height = M;
    Cm.width = Nd;
    Cm.data = C;
    switch (algo) {
        case 0:
            if ((M + 31) / 32 > 65535) return -2;  // grid.y limit of its (32, 32) blocks
            csrspmm::launch_naive(A, Bm, Cm, alpha, beta);
            break;
        case 2: csrspmm::launch_warp_per_row(A, Bm, Cm, alpha, beta); break;
        case 3:
            if (Nd % 4 != 0) return -2;  // float4 accesses would be misaligned
            csrspmm::launch_warp_per_row_fp4(A, Bm, Cm, alpha, beta);
            break;
        case 4:
            if ((long long)max_row_nnz * 32 > 48 * 1024) return -2;  // 4 warps x max_row_nnz x 8 bytes of shared memory
            csrspmm::launch_warp_per_row_smem(A, Bm, Cm, alpha, beta);
            break;
        case 5:
            if (Nd % 4 != 0 || (long long)max_row_nnz * 32 > 48 * 1024) return -2;
            csrspmm::launch_warp_per_row_smem_fp4(A, Bm, Cm, alpha, beta);
            break;
        default: return -1;
    }
    return (int)cudaGetLastError();
}

}  // extern "C"
