// e2m1 value codec on the device: the same format, scale rule and rounding as the host codec
// (csrspmm_b200_e2m1_scale / _encode / _decode), for values that already live on the GPU.
// No counterpart in the reference, whose "Fp4" kernels take fp32 values
// (src/device/csrspmm_warp_per_row_fp4.cu:9-19).
#pragma once

#include "common.cuh"

namespace csrspmm_b200 {

// max |v| over the array, NaNs ignored, as the bits of a non-negative float in *out_bits
// (non-negative floats order like their unsigned bit patterns, so atomicMax on the bits works)
__global__ void __launch_bounds__(256) e2m1_absmax_kernel(long long n, const float* __restrict__ values,
                                                          unsigned* out_bits)
{
    float mx = 0.0f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float a = fabsf(__ldg(values + i));
        if (a > mx) mx = a;  // false for NaN
    }
    unsigned bits = __float_as_uint(mx);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, off));
    if ((threadIdx.x & 31) == 0 && bits != 0) atomicMax(out_bits, bits);
}

// nearest code point, ties to the even code, saturating at 6, sign kept, NaN -> +0
__device__ __forceinline__ unsigned e2m1_encode_one(float v, float scale)
{
    if (v != v) return 0u;
    const float q = __fdiv_rn(v, scale);
    const unsigned s = (__float_as_uint(q) >> 31) ? 8u : 0u;
    const float a = fabsf(q);
    // midpoints between the magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6; a tie goes down when the lower code is even
    unsigned code = 7u;
    if (a < 0.25f || a == 0.25f) code = 0u;
    else if (a < 0.75f) code = 1u;
    else if (a < 1.25f || a == 1.25f) code = 2u;
    else if (a < 1.75f) code = 3u;
    else if (a < 2.5f || a == 2.5f) code = 4u;
    else if (a < 3.5f) code = 5u;
    else if (a < 5.0f || a == 5.0f) code = 6u;
    return s | code;
}

// one thread per output byte (elements 2k and 2k+1)
__global__ void __launch_bounds__(256) e2m1_encode_kernel(long long n, const float* __restrict__ values, float scale,
                                                          unsigned char* __restrict__ packed)
{
    const long long nbytes = (n + 1) / 2;
    for (long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x; k < nbytes; k += (long long)gridDim.x * blockDim.x) {
        const unsigned lo = e2m1_encode_one(__ldg(values + 2 * k), scale);
        const unsigned hi = (2 * k + 1 < n) ? e2m1_encode_one(__ldg(values + 2 * k + 1), scale) : 0u;
        packed[k] = (unsigned char)(lo | (hi << 4));
    }
}

__global__ void __launch_bounds__(256) e2m1_decode_kernel(long long n, const unsigned char* __restrict__ packed,
                                                          float scale, float* __restrict__ values)
{
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const unsigned byte = __ldg(packed + (i >> 1));
        values[i] = decode_e2m1((i & 1) ? (byte >> 4) : (byte & 15u), scale);
    }
}

}  // namespace csrspmm_b200
