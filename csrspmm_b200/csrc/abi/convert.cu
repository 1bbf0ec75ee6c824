// extern "C" entry points for device-side dense <-> CSR conversion (declared in
// include/csrspmm_b200.h).  Counterparts of the reference's host-only dense2csr / csr2dense
// (src/host/csr_utils.cpp:70-145); results are identical, the matrices stay on the device.
#include <cuda_runtime.h>

#include <cstring>

#include "../kernels/codec_kernels.cuh"
#include "../kernels/convert_kernels.cuh"
#include "csrspmm_b200.h"
#include "plan.h"

using namespace csrspmm_b200;

#define CUDA_TRY(expr)                                                                        \
    do {                                                                                      \
        cudaError_t e__ = (expr);                                                             \
        if (e__ != cudaSuccess) {                                                             \
            set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, \
                           __LINE__);                                                         \
            return CSRSPMM_B200_ERR_CUDA;                                                     \
        }                                                                                     \
    } while (0)

extern "C" {

int csrspmm_b200_dense2csr_count(int32_t H, int32_t W, const float* dense, int64_t ld, float tol, int32_t* row_ptr,
                                 int64_t* nnz_out, int32_t* max_row_nnz_out, csrspmm_b200_stream_t stream)
{
    if (H < 0 || W < 0 || ld < W || row_ptr == nullptr || nnz_out == nullptr || (H > 0 && W > 0 && dense == nullptr)) {
        set_last_error("dense2csr_count: bad argument");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const long long n = H;  // row_ptr[1..H] is scanned
    const int nblocks = (int)((n + kScanBlock - 1) / kScanBlock);
    int* scratch = nullptr;  // [0] = max row, [1..] = block sums
    CUDA_TRY(cudaMallocAsync(reinterpret_cast<void**>(&scratch), sizeof(int) * (size_t)(nblocks + 2), st));
    CUDA_TRY(cudaMemsetAsync(scratch, 0, sizeof(int), st));
    CUDA_TRY(cudaMemsetAsync(row_ptr, 0, sizeof(int), st));
    int last = 0, mx = 0;
    if (H > 0) {
        const unsigned grid = (unsigned)((n + 7) / 8);
        dense_count_kernel<<<grid, 256, 0, st>>>(H, W, dense, ld, tol, row_ptr, scratch);
        scan_blocks_kernel<<<nblocks, kScanBlock, 0, st>>>(row_ptr + 1, n, scratch + 1);
        scan_block_sums_kernel<<<1, kScanBlock, 0, st>>>(scratch + 1, nblocks);
        add_block_offsets_kernel<<<nblocks, kScanBlock, 0, st>>>(row_ptr + 1, n, scratch + 1);
        CUDA_TRY(cudaGetLastError());
        CUDA_TRY(cudaMemcpyAsync(&last, row_ptr + H, sizeof(int), cudaMemcpyDeviceToHost, st));
        CUDA_TRY(cudaMemcpyAsync(&mx, scratch, sizeof(int), cudaMemcpyDeviceToHost, st));
    }
    CUDA_TRY(cudaFreeAsync(scratch, st));
    CUDA_TRY(cudaStreamSynchronize(st));
    *nnz_out = last;
    if (max_row_nnz_out) *max_row_nnz_out = mx;
    if (last < 0) {  // more than 2^31 - 1 kept entries: the int32 offsets wrapped
        set_last_error("dense2csr_count: more than 2^31-1 non-zeros");
        return CSRSPMM_B200_ERR_UNSUPPORTED;
    }
    return CSRSPMM_B200_OK;
}

int csrspmm_b200_dense2csr_fill(int32_t H, int32_t W, const float* dense, int64_t ld, float tol, const int32_t* row_ptr,
                                int32_t* col_idx, float* values, csrspmm_b200_stream_t stream)
{
    if (H < 0 || W < 0 || ld < W || row_ptr == nullptr) {
        set_last_error("dense2csr_fill: bad argument");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (H == 0 || W == 0) return CSRSPMM_B200_OK;
    if (dense == nullptr || col_idx == nullptr || values == nullptr) {
        set_last_error("dense2csr_fill: null pointer");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    dense_fill_kernel<<<(unsigned)(((long long)H + 7) / 8), 256, 0, st>>>(H, W, dense, ld, tol, row_ptr, col_idx, values);
    CUDA_TRY(cudaGetLastError());
    return CSRSPMM_B200_OK;
}

int csrspmm_b200_csr2dense(int32_t H, int32_t W, const int32_t* row_ptr, const int32_t* col_idx, const float* values,
                           float* dense, int64_t ld, csrspmm_b200_stream_t stream)
{
    if (H < 0 || W < 0 || ld < W || (H > 0 && (row_ptr == nullptr || (W > 0 && dense == nullptr)))) {
        set_last_error("csr2dense: bad argument");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (H == 0 || W == 0) return CSRSPMM_B200_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    CUDA_TRY(cudaMemset2DAsync(dense, (size_t)ld * 4, 0, (size_t)W * 4, (size_t)H, st));
    csr_scatter_kernel<<<(unsigned)(((long long)H + 7) / 8), 256, 0, st>>>(H, W, row_ptr, col_idx, values, dense, ld);
    CUDA_TRY(cudaGetLastError());
    return CSRSPMM_B200_OK;
}

// ---- e2m1 codec on the device ------------------------------------------------------------------

int csrspmm_b200_e2m1_scale_device(int64_t n, const float* values, float* scale_out, csrspmm_b200_stream_t stream)
{
    if (n < 0 || scale_out == nullptr || (n > 0 && values == nullptr)) {
        set_last_error("e2m1_scale_device: bad argument");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    *scale_out = 1.0f;
    if (n == 0) return CSRSPMM_B200_OK;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    unsigned* d_bits = nullptr;
    CUDA_TRY(cudaMallocAsync(reinterpret_cast<void**>(&d_bits), sizeof(unsigned), st));
    CUDA_TRY(cudaMemsetAsync(d_bits, 0, sizeof(unsigned), st));
    const long long want = (n + 255) / 256;
    const unsigned grid = (unsigned)(want < 148 * 16 ? want : 148 * 16);
    e2m1_absmax_kernel<<<grid, 256, 0, st>>>(n, values, d_bits);
    CUDA_TRY(cudaGetLastError());
    unsigned bits = 0;
    CUDA_TRY(cudaMemcpyAsync(&bits, d_bits, sizeof(unsigned), cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaFreeAsync(d_bits, st));
    CUDA_TRY(cudaStreamSynchronize(st));
    float mx;
    static_assert(sizeof(mx) == sizeof(bits), "float is 32 bits");
    memcpy(&mx, &bits, sizeof(mx));
    *scale_out = mx > 0.0f ? mx / 6.0f : 1.0f;
    return CSRSPMM_B200_OK;
}

int csrspmm_b200_e2m1_encode_device(int64_t n, const float* values, float scale, uint8_t* packed,
                                    csrspmm_b200_stream_t stream)
{
    if (n < 0 || (n > 0 && (values == nullptr || packed == nullptr)) || !(scale > 0.0f)) {
        set_last_error("e2m1_encode_device: bad argument");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (n == 0) return CSRSPMM_B200_OK;
    const long long want = ((n + 1) / 2 + 255) / 256;
    const unsigned grid = (unsigned)(want < 148 * 16 ? want : 148 * 16);
    e2m1_encode_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(n, values, scale, packed);
    CUDA_TRY(cudaGetLastError());
    return CSRSPMM_B200_OK;
}

int csrspmm_b200_e2m1_decode_device(int64_t n, const uint8_t* packed, float scale, float* values,
                                    csrspmm_b200_stream_t stream)
{
    if (n < 0 || (n > 0 && (values == nullptr || packed == nullptr))) {
        set_last_error("e2m1_decode_device: bad argument");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (n == 0) return CSRSPMM_B200_OK;
    const long long want = (n + 255) / 256;
    const unsigned grid = (unsigned)(want < 148 * 16 ? want : 148 * 16);
    e2m1_decode_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(n, packed, scale, values);
    CUDA_TRY(cudaGetLastError());
    return CSRSPMM_B200_OK;
}

}  // extern "C"
