// Small device-side helpers around the SpMM kernels: CSR validation and row statistics.
// Neither has a counterpart in the reference, whose host layer checks nothing
// (src/host/spmm_launcher.cu:11-171) and leaves max_row_nnz to the caller
// (src/host/csr_utils.cpp:105-110).
#pragma once

#include "common.cuh"

namespace csrspmm_b200 {

// problems: OR of the CSRSPMM_B200_CSR_* bits.
__global__ void validate_csr_kernel(int M, int Kd, long long nnz, const int* __restrict__ row_ptr,
                                    const int* __restrict__ col_idx, unsigned* problems)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    unsigned bad = 0;
    if (tid == 0) {
        if (row_ptr[0] != 0) bad |= 1u;
        if ((long long)row_ptr[M] != nnz) bad |= 2u;
    }
    for (long long r = tid; r < M; r += stride) {
        const int rs = row_ptr[r], re = row_ptr[r + 1];
        if (re < rs) {
            bad |= 4u;
            continue;
        }
        if (rs < 0 || (long long)re > nnz) continue;  // already reported through the end checks
        int prev = -1;
        for (int j = rs; j < re; ++j) {
            const int c = col_idx[j];
            if (c < 0 || c >= Kd) bad |= 8u;
            if (c <= prev) bad |= 16u;
            prev = c;
        }
    }
    if (bad) atomicOr(problems, bad);
}

// stats[0] = longest row, [1] = empty rows, [2] = rows longer than `long_threshold`,
// [3] = nnz in those rows.
__global__ void row_stats_kernel(int M, const int* __restrict__ row_ptr, long long long_threshold,
                                 unsigned long long* stats)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    unsigned long long mx = 0, empty = 0, nlong = 0, nnz_long = 0;
    for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < M; r += stride) {
        const long long len = (long long)row_ptr[r + 1] - row_ptr[r];
        if (len <= 0) ++empty;
        if (len > (long long)mx) mx = (unsigned long long)len;
        if (len > long_threshold) {
            ++nlong;
            nnz_long += (unsigned long long)len;
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        empty += __shfl_xor_sync(0xffffffffu, empty, o);
        nlong += __shfl_xor_sync(0xffffffffu, nlong, o);
        nnz_long += __shfl_xor_sync(0xffffffffu, nnz_long, o);
    }
    if ((threadIdx.x & 31) == 0) {
        atomicMax(stats + 0, mx);
        if (empty) atomicAdd(stats + 1, empty);
        if (nlong) atomicAdd(stats + 2, nlong);
        if (nnz_long) atomicAdd(stats + 3, nnz_long);
    }
}

}  // namespace csrspmm_b200
