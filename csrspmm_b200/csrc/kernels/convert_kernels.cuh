// Device-side dense <-> CSR conversion.
//
// The reference converts on one host core (src/host/csr_utils.cpp:70-145: count, allocate, fill
// row by row with fabs(v) > tol, ascending columns, max_row_nnz; and zero-fill + scatter for the
// way back), which is O(M * Kd) and sized with 32-bit products.  These kernels produce the same
// arrays, bit for bit, from a device-resident matrix: one warp per row, 32 columns per step,
// ballot + popcount for the position of each kept entry, so the order inside a row is ascending.
#pragma once

#include <cuda_runtime.h>

namespace csrspmm_b200 {

// counts[r] = number of entries of row r with |v| > tol (written to row_ptr[r + 1]; row_ptr[0] = 0)
__global__ void dense_count_kernel(int H, int W, const float* __restrict__ dense, long long ld, float tol,
                                   int* __restrict__ row_ptr, int* __restrict__ max_row)
{
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= H) return;
    const float* src = dense + row * ld;
    int count = 0;
    for (int c0 = 0; c0 < W; c0 += 32) {
        const int c = c0 + lane;
        const bool keep = c < W && fabsf(src[c]) > tol;
        count += __popc(__ballot_sync(0xffffffffu, keep));
    }
    if (lane == 0) {
        row_ptr[row + 1] = count;
        if (row == 0) row_ptr[0] = 0;
        atomicMax(max_row, count);
    }
}

// ---- inclusive scan of data[0..n) in three launches (block scan, scan of block sums, add) --------
constexpr int kScanBlock = 1024;

__device__ __forceinline__ int block_inclusive_scan(int v, int* warp_sums)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    if (lane == 31) warp_sums[warp] = v;
    __syncthreads();
    if (warp == 0) {
        int w = lane < (blockDim.x >> 5) ? warp_sums[lane] : 0;
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += t;
        }
        warp_sums[lane] = w;
    }
    __syncthreads();
    if (warp > 0) v += warp_sums[warp - 1];
    return v;
}

__global__ void scan_blocks_kernel(int* data, long long n, int* block_sums)
{
    __shared__ int warp_sums[32];
    const long long i = (long long)blockIdx.x * kScanBlock + threadIdx.x;
    int v = i < n ? data[i] : 0;
    v = block_inclusive_scan(v, warp_sums);
    if (i < n) data[i] = v;
    if (threadIdx.x == kScanBlock - 1) block_sums[blockIdx.x] = v;
}

// one block: exclusive offsets of the block sums, in place, carrying a running total
__global__ void scan_block_sums_kernel(int* block_sums, int nblocks)
{
    __shared__ int warp_sums[32];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < nblocks; base += kScanBlock) {
        const int i = base + threadIdx.x;
        const int own = i < nblocks ? block_sums[i] : 0;
        const int incl = block_inclusive_scan(own, warp_sums);
        const int c = carry;
        if (i < nblocks) block_sums[i] = c + incl - own;
        __syncthreads();
        if (threadIdx.x == kScanBlock - 1) carry = c + incl;
        __syncthreads();
    }
}

__global__ void add_block_offsets_kernel(int* data, long long n, const int* block_offsets)
{
    const long long i = (long long)blockIdx.x * kScanBlock + threadIdx.x;
    if (i < n) data[i] += block_offsets[blockIdx.x];
}

__global__ void dense_fill_kernel(int H, int W, const float* __restrict__ dense, long long ld, float tol,
                                  const int* __restrict__ row_ptr, int* __restrict__ col_idx,
                                  float* __restrict__ values)
{
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= H) return;
    const float* src = dense + row * ld;
    int pos = row_ptr[row];
    for (int c0 = 0; c0 < W; c0 += 32) {
        const int c = c0 + lane;
        const float v = c < W ? src[c] : 0.0f;
        const bool keep = c < W && fabsf(v) > tol;
        const unsigned mask = __ballot_sync(0xffffffffu, keep);
        if (keep) {
            const int at = pos + __popc(mask & ((1u << lane) - 1u));
            col_idx[at] = c;
            values[at] = v;
        }
        pos += __popc(mask);
    }
}

__global__ void csr_scatter_kernel(int H, int W, const int* __restrict__ row_ptr, const int* __restrict__ col_idx,
                                   const float* __restrict__ values, float* __restrict__ dense, long long ld)
{
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= H) return;
    float* dst = dense + row * ld;
    // a repeated column index keeps the last stored value, like the sequential host loop
    const int rs = row_ptr[row], re = row_ptr[row + 1];
    for (int j0 = rs; j0 < re; j0 += 32) {
        const int j = j0 + lane;
        const int c = j < re ? col_idx[j] : -1;
        const float v = j < re ? values[j] : 0.0f;
        // later lanes win over earlier ones with the same column
        bool last = c >= 0 && c < W;
        for (int o = 1; o < 32; ++o) {
            const int other = __shfl_down_sync(0xffffffffu, c, o);
            if (lane + o < 32 && other == c) last = false;
        }
        if (last) dst[c] = v;
        __syncwarp();
    }
}

}  // namespace csrspmm_b200
