/*
 * CPU oracle for the CSR x dense SpMM hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, on the CPU, the arithmetic of the reference's GPU kernels so
 * that the CUDA library can be checked against it.  It is never linked into, loaded
 * by, or called from the product library: only the test-suite, the smoke check and
 * the benchmark's CPU-baseline legs may use it.
 *
 * Parity status: PINNED for the fp32 path.  The reference ships no host CSR SpMM, so
 * the restatement below is checked bit-for-bit against the reference's own host code
 * (dense2csr + dense_gemm_cpu, src/host/csr_utils.cpp:70-111 and
 * src/host/dense_utils.cpp:109-126) compiled unmodified into oracle/_ref, and against
 * golden vectors generated from that build (tests/golden).  The e2m1 codec at the end
 * of this file has NO counterpart in the reference ("Fp4" there means float4 loads):
 * parity unpinned for that part; it is defined here and checked only for
 * self-consistency.
 *
 * Build: see oracle/Makefile (gcc, -ffp-contract=off so that nothing is fused unless
 * fmaf() is written out).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_MAX_STACK_COLS 1024

/* ------------------------------------------------------------------------------------------
 * One row of C.  Follows src/device/csrspmm_naive.cu:27-38:
 *   row range from row_ptr; per output column one fp32 accumulator that takes the row's
 *   non-zeros in stored order (sum += val * B[col*K + c]); epilogue
 *   alpha*sum + (beta != 0 ? beta*C : 0), C not read when beta == 0.
 * mode 0: accumulation is a fused multiply-add (what nvcc emits for the reference kernels and
 *         what the sm_100a kernels issue explicitly).
 * mode 1: multiply and add rounded separately (what src/host/dense_utils.cpp:118-120 does when
 *         compiled without contraction).
 * The epilogue is never fused: t = alpha*sum, u = beta*old, out = t + u.
 * ------------------------------------------------------------------------------------------ */
static void row_f32(int Nd, int ncols, int32_t rs, int32_t re, const int32_t* col_idx,
                    const float* vals, const float* B, int64_t ldb, float* crow, float alpha,
                    float beta, int mode, float* acc)
{
    (void)Nd;
    for (int c = 0; c < ncols; ++c) acc[c] = 0.0f;
    if (mode == 0) {
        for (int32_t j = rs; j < re; ++j) {
            const float a = vals[j];
            const float* brow = B + (int64_t)col_idx[j] * ldb;
            for (int c = 0; c < ncols; ++c) acc[c] = fmaf(a, brow[c], acc[c]);
        }
    } else {
        for (int32_t j = rs; j < re; ++j) {
            const float a = vals[j];
            const float* brow = B + (int64_t)col_idx[j] * ldb;
            for (int c = 0; c < ncols; ++c) {
                const float p = a * brow[c];
                acc[c] = acc[c] + p;
            }
        }
    }
    if (beta != 0.0f) {
        for (int c = 0; c < ncols; ++c) {
            const float t = alpha * acc[c];
            const float u = beta * crow[c];
            crow[c] = t + u;
        }
    } else {
        for (int c = 0; c < ncols; ++c) {
            const float t = alpha * acc[c];
            crow[c] = t + 0.0f;
        }
    }
}

/* C[0:M, 0:ncols] = alpha*A*B + beta*C.  ncols <= Nd lets a caller express the reference's
 * float4 kernels, which only write the first 4*floor(Nd/4) columns
 * (src/device/csrspmm_warp_per_row_fp4.cu:29-32). threads <= 1 runs serially. */
void oracle_spmm_f32(int M, int Nd, int ncols, const int32_t* row_ptr, const int32_t* col_idx,
                     const float* vals, const float* B, int64_t ldb, float* C, int64_t ldc,
                     float alpha, float beta, int mode, int threads)
{
    if (ncols > Nd) ncols = Nd;
#ifdef _OPENMP
    if (threads < 1) threads = 1;
#pragma omp parallel num_threads(threads)
    {
        float stack_acc[ORACLE_MAX_STACK_COLS];
        float* acc = ncols <= ORACLE_MAX_STACK_COLS ? stack_acc
                                                    : (float*)malloc(sizeof(float) * (size_t)ncols);
#pragma omp for schedule(dynamic, 256)
        for (int r = 0; r < M; ++r)
            row_f32(Nd, ncols, row_ptr[r], row_ptr[r + 1], col_idx, vals, B, ldb,
                    C + (int64_t)r * ldc, alpha, beta, mode, acc);
        if (acc != stack_acc) free(acc);
    }
#else
    (void)threads;
    float* acc = (float*)malloc(sizeof(float) * (size_t)(ncols > 0 ? ncols : 1));
    for (int r = 0; r < M; ++r)
        row_f32(Nd, ncols, row_ptr[r], row_ptr[r + 1], col_idx, vals, B, ldb,
                C + (int64_t)r * ldc, alpha, beta, mode, acc);
    free(acc);
#endif
}

/* The same sum carried in double: out64 = alpha*sum + beta*old (all in double) and
 * mag = |alpha|*sum|a*b| + |beta*old|, the scale against which a re-associated fp32 sum is
 * judged.  C_old may be NULL when beta == 0. */
void oracle_spmm_f64(int M, int Nd, const int32_t* row_ptr, const int32_t* col_idx,
                     const float* vals, const float* B, int64_t ldb, const float* C_old,
                     int64_t ldc, float alpha, float beta, double* out64, double* mag,
                     int threads)
{
#ifdef _OPENMP
    if (threads < 1) threads = 1;
#pragma omp parallel for schedule(dynamic, 256) num_threads(threads)
#endif
    for (int r = 0; r < M; ++r) {
        double* o = out64 + (int64_t)r * Nd;
        double* g = mag ? mag + (int64_t)r * Nd : NULL;
        for (int c = 0; c < Nd; ++c) {
            o[c] = 0.0;
            if (g) g[c] = 0.0;
        }
        for (int32_t j = row_ptr[r]; j < row_ptr[r + 1]; ++j) {
            const double a = (double)vals[j];
            const float* brow = B + (int64_t)col_idx[j] * ldb;
            for (int c = 0; c < Nd; ++c) {
                const double p = a * (double)brow[c];
                o[c] += p;
                if (g) g[c] += fabs(p);
            }
        }
        for (int c = 0; c < Nd; ++c) {
            const double old = (beta != 0.0f) ? (double)beta * (double)C_old[(int64_t)r * ldc + c] : 0.0;
            o[c] = (double)alpha * o[c] + old;
            if (g) g[c] = fabs((double)alpha) * g[c] + fabs(old);
        }
    }
}

/* Selected rows only (rows[i] indexes A and C): lets a full-size run be checked on a sample.
 * out is nrows x Nd, dense; C_old, if beta != 0, is the full C. */
void oracle_spmm_rows_f32(int nrows, const int32_t* rows, int Nd, const int32_t* row_ptr,
                          const int32_t* col_idx, const float* vals, const float* B, int64_t ldb,
                          const float* C_old, int64_t ldc, float alpha, float beta, int mode,
                          float* out)
{
    float* acc = (float*)malloc(sizeof(float) * (size_t)(Nd > 0 ? Nd : 1));
    for (int i = 0; i < nrows; ++i) {
        const int r = rows[i];
        float* o = out + (int64_t)i * Nd;
        if (beta != 0.0f)
            memcpy(o, C_old + (int64_t)r * ldc, sizeof(float) * (size_t)Nd);
        row_f32(Nd, Nd, row_ptr[r], row_ptr[r + 1], col_idx, vals, B, ldb, o, alpha, beta, mode, acc);
    }
    free(acc);
}

/* ------------------------------------------------------------------------------------------
 * dense -> CSR, following src/host/csr_utils.cpp:85-110: keep v when fabs(v) > tol, columns in
 * ascending order, max_row_nnz = longest row.  Two passes: count, then fill caller buffers.
 * ------------------------------------------------------------------------------------------ */
int64_t oracle_dense2csr_count(int H, int W, const float* dense, float tol)
{
    int64_t nnz = 0;
    for (int64_t i = 0; i < (int64_t)H * W; ++i)
        if (fabsf(dense[i]) > tol) ++nnz;
    return nnz;
}

int oracle_dense2csr_fill(int H, int W, const float* dense, float tol, int32_t* row_ptr,
                          int32_t* col_idx, float* vals)
{
    int32_t idx = 0;
    int mx = 0;
    row_ptr[0] = 0;
    for (int i = 0; i < H; ++i) {
        for (int j = 0; j < W; ++j) {
            const float v = dense[(int64_t)i * W + j];
            if (fabsf(v) > tol) {
                col_idx[idx] = j;
                vals[idx] = v;
                ++idx;
            }
        }
        row_ptr[i + 1] = idx;
        if (row_ptr[i + 1] - row_ptr[i] > mx) mx = row_ptr[i + 1] - row_ptr[i];
    }
    return mx;
}

/* CSR -> dense, following src/host/csr_utils.cpp:114-145 (zero fill, last write wins). */
void oracle_csr2dense(int H, int W, const int32_t* row_ptr, const int32_t* col_idx,
                      const float* vals, float* dense)
{
    memset(dense, 0, sizeof(float) * (size_t)H * (size_t)W);
    for (int i = 0; i < H; ++i)
        for (int32_t p = row_ptr[i]; p < row_ptr[i + 1]; ++p)
            dense[(int64_t)i * W + col_idx[p]] = vals[p];
}

/* ------------------------------------------------------------------------------------------
 * e2m1 (4-bit: 1 sign, 2 exponent, 1 mantissa) value codec.  No counterpart in the reference:
 * parity unpinned.  Format defined by this library:
 *   code = s<<3 | e<<1 | m ; magnitude = e ? (1 + m/2) * 2^(e-1) : m/2
 *        -> {0, 0.5, 1, 1.5, 2, 3, 4, 6}
 *   element j lives in byte j>>1, low nibble when j is even, high nibble when j is odd
 *   one fp32 scale per tensor; decoded value = magnitude * scale, one fp32 rounding
 *   encode: q = v/scale, nearest magnitude, ties to the even code, saturate at 6,
 *           sign bit kept (also for zero), NaN -> +0
 * ------------------------------------------------------------------------------------------ */
static const float k_e2m1_mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

uint8_t oracle_e2m1_encode_one(float v, float scale)
{
    if (v != v) return 0;
    const float q = v / scale;
    const uint8_t s = signbit(q) ? 8u : 0u;
    const float a = fabsf(q);
    uint8_t code = 7;
    for (int k = 0; k < 7; ++k) {
        const float mid = 0.5f * (k_e2m1_mag[k] + k_e2m1_mag[k + 1]);
        if (a < mid || (a == mid && (k & 1) == 0)) {
            code = (uint8_t)k;
            break;
        }
    }
    return (uint8_t)(s | code);
}

float oracle_e2m1_decode_one(uint8_t code, float scale)
{
    const float m = k_e2m1_mag[code & 7u];
    const float v = m * scale;
    return (code & 8u) ? -v : v;
}

float oracle_e2m1_scale(int64_t n, const float* v)
{
    float mx = 0.0f;
    for (int64_t i = 0; i < n; ++i) {
        const float a = fabsf(v[i]);
        if (a > mx) mx = a;
    }
    return mx > 0.0f ? mx / 6.0f : 1.0f;
}

/* packed must hold (n+1)/2 bytes; an odd tail leaves the last high nibble zero. */
void oracle_e2m1_encode(int64_t n, const float* v, float scale, uint8_t* packed)
{
    memset(packed, 0, (size_t)((n + 1) / 2));
    for (int64_t i = 0; i < n; ++i) {
        const uint8_t c = oracle_e2m1_encode_one(v[i], scale);
        packed[i >> 1] |= (uint8_t)((i & 1) ? (c << 4) : c);
    }
}

void oracle_e2m1_decode(int64_t n, const uint8_t* packed, float scale, float* out)
{
    for (int64_t i = 0; i < n; ++i) {
        const uint8_t byte = packed[i >> 1];
        const uint8_t c = (i & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 15u);
        out[i] = oracle_e2m1_decode_one(c, scale);
    }
}

int oracle_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
