// Shared device-side helpers of the sm_100a CSR SpMM kernels.
//
// Arithmetic contract (what the CPU oracle restates from the reference kernels,
// src/device/csrspmm_naive.cu:27-38): every output element is an fp32 accumulator that takes
// val[j] * B[col[j], c] by fused multiply-add, and the epilogue is
// alpha*sum + (beta != 0 ? beta*C_old : 0) with the products and the sum rounded separately;
// C is never read when beta == 0.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "tuning.h"

namespace csrspmm_b200 {

// Bits OR-ed into the optional device status word.
constexpr int kStatusBadTile = 1;      // merge-path coordinates inconsistent (malformed row_ptr)
constexpr int kStatusColClamped = 2;   // a column index outside [0, Kd) was clamped
constexpr int kStatusWaitTimeout = 4;  // a bounded wait on an mbarrier gave up

// Attempts of a bounded wait before it gives up (each attempt is itself a short hardware wait).
constexpr unsigned kWaitSpinLimit = 1u << 22;

constexpr int kValuesF32 = 0;
constexpr int kValuesE2M1 = 1;

struct SpmmParams {
    int M;
    int Kd;
    int Nd;
    int nnz;
    int ncolv;            // columns in units of the vector width: ceil(Nd / VW)
    long long num_items;  // M + nnz (merge-path length)
    const int* row_ptr;
    int rp_base;          // subtracted from every row_ptr entry (row block of a larger matrix)
    const int* col_idx;
    const void* values;
    float value_scale;
    const float* B;
    long long ldb;
    unsigned ldb_bytes;  // ldb * 4 (< 2^32, checked on the host): one wide multiply per B-row address
    float* C;
    long long ldc;
    float alpha;
    float beta;
    int* carry_row;      // one per tile: row the tile leaves unfinished, or -1
    float* carry_val;    // one row of carry_ld floats per tile
    long long carry_ld;  // multiple of 4
    int* status_word;    // may be null
    unsigned wait_limit; // bulk-copy kernel: attempts a wait on a row copy makes before it gives up
    int skip_len;        // merge kernel with SKIP: rows of this many entries or more are left to the
                         // scheduled pieces (neither summed nor written); 0 = every row is mine
};

__device__ __forceinline__ void report_status(const SpmmParams& p, int bit)
{
    if (p.status_word != nullptr) atomicOr(p.status_word, bit);
}

// ---- value formats ------------------------------------------------------------------------------

// e2m1 code (s eem) -> fp32: magnitude in {0, .5, 1, 1.5, 2, 3, 4, 6} built directly as IEEE
// bits, then one rounded multiply by the tensor scale, then the sign.
__device__ __forceinline__ float decode_e2m1(unsigned code, float scale)
{
    const unsigned m = code & 1u;
    const unsigned e = (code >> 1) & 3u;
    const unsigned bits = e ? (((126u + e) << 23) | (m << 22)) : (m ? 0x3F000000u : 0u);
    const float v = __fmul_rn(__uint_as_float(bits), scale);
    return (code & 8u) ? -v : v;
}

template <int FMT>
__device__ __forceinline__ float load_value(const void* values, int j, float scale)
{
    if constexpr (FMT == kValuesF32) {
        return __ldcs(reinterpret_cast<const float*>(values) + j);
    } else {
        const unsigned byte = __ldg(reinterpret_cast<const unsigned char*>(values) + (j >> 1));
        return decode_e2m1((j & 1) ? (byte >> 4) : (byte & 15u), scale);
    }
}

// ---- L2 residency policy for the gathered operand -------------------------------------------------
// B is the only operand that is re-read (once per non-zero that names the row); A streams through
// once and C is written once.  When B is larger than L2 its lines compete with that streaming
// traffic; B loads can carry an evict_last policy and C stores can be streaming stores
// (compile-time options in tuning.h, off by default: they did not pay on B200).
__device__ __forceinline__ unsigned long long make_b_policy()
{
    unsigned long long pol = 0;
#if CSRSPMM_TUNE_B_EVICT_LAST_PCT >= 100
    asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
#elif CSRSPMM_TUNE_B_EVICT_LAST_PCT > 0
    asm("createpolicy.fractional.L2::evict_last.L2::evict_first.b64 %0, %1;"
        : "=l"(pol)
        : "f"(CSRSPMM_TUNE_B_EVICT_LAST_PCT / 100.0f));
#endif
    return pol;
}

// ---- asynchronous global -> shared copies (per-thread completion groups) ----------------------------
__device__ __forceinline__ unsigned smem_addr(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }

template <int VW>
__device__ __forceinline__ void async_copy_vec(unsigned dst, const void* src)
{
    if constexpr (VW == 4) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
template <int VW>
__device__ __forceinline__ void async_copy_vec_hint(unsigned dst, const void* src, unsigned long long policy)
{
    if constexpr (VW == 4)
        asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "l"(policy) : "memory");
    else
        asm volatile("cp.async.ca.shared.global.L2::cache_hint [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "l"(policy) : "memory");
}
__device__ __forceinline__ void async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ---- column vectors (VW = 4: float4, 16-byte aligned; VW = 1: one float) --------------------------

template <int VW>
struct Vec;

template <>
struct Vec<4> {
    float4 v;
    __device__ __forceinline__ void zero() { v = make_float4(0.f, 0.f, 0.f, 0.f); }
    __device__ __forceinline__ void load_nc(const float* p) { v = __ldg(reinterpret_cast<const float4*>(p)); }
    __device__ __forceinline__ void load_b(const float* p, unsigned long long pol)
    {
#if CSRSPMM_TUNE_B_EVICT_LAST_PCT > 0
        asm("ld.global.nc.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
            : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
            : "l"(p), "l"(pol));
#else
        (void)pol;
        load_nc(p);
#endif
    }
    // read-only load carrying an L2 eviction policy made by createpolicy
    __device__ __forceinline__ void load_hint(const float* p, unsigned long long pol)
    {
        asm("ld.global.nc.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
            : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
            : "l"(p), "l"(pol));
    }
    __device__ __forceinline__ void load(const float* p) { v = *reinterpret_cast<const float4*>(p); }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = v; }
    __device__ __forceinline__ void store_streaming(float* p) const { __stcs(reinterpret_cast<float4*>(p), v); }
    __device__ __forceinline__ Vec shuffle(int src_lane) const  // this value as held by src_lane of the warp
    {
        Vec r;
        r.v.x = __shfl_sync(0xffffffffu, v.x, src_lane);
        r.v.y = __shfl_sync(0xffffffffu, v.y, src_lane);
        r.v.z = __shfl_sync(0xffffffffu, v.z, src_lane);
        r.v.w = __shfl_sync(0xffffffffu, v.w, src_lane);
        return r;
    }
    __device__ __forceinline__ void fma(float a, const Vec& b)
    {
        v.x = __fmaf_rn(a, b.v.x, v.x);
        v.y = __fmaf_rn(a, b.v.y, v.y);
        v.z = __fmaf_rn(a, b.v.z, v.z);
        v.w = __fmaf_rn(a, b.v.w, v.w);
    }
    __device__ __forceinline__ void add(const Vec& b)
    {
        v.x = __fadd_rn(v.x, b.v.x);
        v.y = __fadd_rn(v.y, b.v.y);
        v.z = __fadd_rn(v.z, b.v.z);
        v.w = __fadd_rn(v.w, b.v.w);
    }
    // alpha*this + beta*old, nothing fused
    __device__ __forceinline__ Vec epilogue(float alpha, float beta, const Vec& old) const
    {
        Vec r;
        r.v.x = __fadd_rn(__fmul_rn(alpha, v.x), __fmul_rn(beta, old.v.x));
        r.v.y = __fadd_rn(__fmul_rn(alpha, v.y), __fmul_rn(beta, old.v.y));
        r.v.z = __fadd_rn(__fmul_rn(alpha, v.z), __fmul_rn(beta, old.v.z));
        r.v.w = __fadd_rn(__fmul_rn(alpha, v.w), __fmul_rn(beta, old.v.w));
        return r;
    }
    __device__ __forceinline__ Vec epilogue0(float alpha) const
    {
        Vec r;
        r.v.x = __fadd_rn(__fmul_rn(alpha, v.x), 0.0f);
        r.v.y = __fadd_rn(__fmul_rn(alpha, v.y), 0.0f);
        r.v.z = __fadd_rn(__fmul_rn(alpha, v.z), 0.0f);
        r.v.w = __fadd_rn(__fmul_rn(alpha, v.w), 0.0f);
        return r;
    }
    // old + alpha*this (fix-up of a finished row)
    __device__ __forceinline__ Vec add_scaled_to(float alpha, const Vec& old) const
    {
        Vec r;
        r.v.x = __fadd_rn(old.v.x, __fmul_rn(alpha, v.x));
        r.v.y = __fadd_rn(old.v.y, __fmul_rn(alpha, v.y));
        r.v.z = __fadd_rn(old.v.z, __fmul_rn(alpha, v.z));
        r.v.w = __fadd_rn(old.v.w, __fmul_rn(alpha, v.w));
        return r;
    }
};

template <>
struct Vec<1> {
    float v;
    __device__ __forceinline__ void zero() { v = 0.f; }
    __device__ __forceinline__ void load_nc(const float* p) { v = __ldg(p); }
    __device__ __forceinline__ void load_b(const float* p, unsigned long long pol)
    {
#if CSRSPMM_TUNE_B_EVICT_LAST_PCT > 0
        asm("ld.global.nc.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(p), "l"(pol));
#else
        (void)pol;
        load_nc(p);
#endif
    }
    __device__ __forceinline__ void load_hint(const float* p, unsigned long long pol)
    {
        asm("ld.global.nc.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(p), "l"(pol));
    }
    __device__ __forceinline__ void load(const float* p) { v = *p; }
    __device__ __forceinline__ void store(float* p) const { *p = v; }
    __device__ __forceinline__ void store_streaming(float* p) const { __stcs(p, v); }
    __device__ __forceinline__ Vec shuffle(int src_lane) const
    {
        Vec r;
        r.v = __shfl_sync(0xffffffffu, v, src_lane);
        return r;
    }
    __device__ __forceinline__ void fma(float a, const Vec& b) { v = __fmaf_rn(a, b.v, v); }
    __device__ __forceinline__ void add(const Vec& b) { v = __fadd_rn(v, b.v); }
    __device__ __forceinline__ Vec epilogue(float alpha, float beta, const Vec& old) const
    {
        Vec r;
        r.v = __fadd_rn(__fmul_rn(alpha, v), __fmul_rn(beta, old.v));
        return r;
    }
    __device__ __forceinline__ Vec epilogue0(float alpha) const
    {
        Vec r;
        r.v = __fadd_rn(__fmul_rn(alpha, v), 0.0f);
        return r;
    }
    __device__ __forceinline__ Vec add_scaled_to(float alpha, const Vec& old) const
    {
        Vec r;
        r.v = __fadd_rn(old.v, __fmul_rn(alpha, v));
        return r;
    }
};

// Write one finished row segment: C[row, cv] = alpha*acc + beta*C_old for this lane's NV vectors.
template <int G, int NV, int VW>
__device__ __forceinline__ void store_row(const SpmmParams& p, int row, int cb, int lane,
                                          const Vec<VW> (&acc)[NV])
{
    float* crow = p.C + (long long)row * p.ldc;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int cv = cb + lane + v * G;
        if (cv < p.ncolv) {
            float* cp = crow + (long long)cv * VW;
#if CSRSPMM_TUNE_C_STREAMING
            if (p.beta != 0.0f) {
                Vec<VW> old;
                old.load(cp);
                acc[v].epilogue(p.alpha, p.beta, old).store_streaming(cp);
            } else {
                acc[v].epilogue0(p.alpha).store_streaming(cp);
            }
#else
            if (p.beta != 0.0f) {
                Vec<VW> old;
                old.load(cp);
                acc[v].epilogue(p.alpha, p.beta, old).store(cp);
            } else {
                acc[v].epilogue0(p.alpha).store(cp);
            }
#endif
        }
    }
}

}  // namespace csrspmm_b200
