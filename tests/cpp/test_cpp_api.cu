// Exercises the csrspmm:: C++ API the way the reference's own test program does
// (tests/test_csrspmm.cu:56-108 there): dense A -> dense2csr -> host2device -> spmm ->
// device2host -> compare with dense_gemm_cpu -- but for every Algorithm in one run, for
// integer and real-valued data, and with a non-zero exit code on any failure.
#include <cstdio>
#include <cstdlib>
#include <cmath>
#include <cstring>
#include <string>

#include <csrspmm/csrspmm.h>
#include <csrspmm/csr_utils.h>
#include <csrspmm/dense_utils.h>
#include <csrspmm/error_check.h>
#include <csrspmm/spmm_launcher.cuh>

using namespace csrspmm;

static int failures = 0;

#define EXPECT(cond)                                                        \
    do {                                                                    \
        if (!(cond)) {                                                      \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);   \
            ++failures;                                                     \
        }                                                                   \
    } while (0)

static bool all_finite(const DenseMatrix& m)
{
    for (size_t k = 0; k < size_t(m.height) * size_t(m.width); ++k)
        if (!std::isfinite(m.data[k])) return false;
    return true;
}

static void run_case(int M, int N, int K, float sparsity, float alpha, float beta, bool integer_values)
{
    const char* names[] = {"Naive", "NaiveSmem", "WarpPerRow", "WarpPerRowFp4", "WarpPerRowSmem", "WarpPerRowSmemFp4"};
    DenseMatrix hA, hB, hC;
    dense_alloc_host(hA, M, N);
    dense_alloc_host(hB, N, K);
    dense_alloc_host(hC, M, K);
    dense_init_random(hA, -10.0f, 10.0f, sparsity, integer_values);
    dense_init_random(hB, -10.0f, 10.0f, 0.0f, integer_values);
    dense_init_random(hC, -10.0f, 10.0f, 0.0f, integer_values);

    CSRMatrix hA_csr;
    dense2csr(hA, hA_csr, 0.0f);
    EXPECT(hA_csr.row_ptr[0] == 0 && hA_csr.row_ptr[M] == hA_csr.nnz);

    DenseMatrix back;
    csr2dense(hA_csr, back);
    EXPECT(dense_compare(hA, back, 0.0f));  // round trip
    dense_free_host(back);

    DenseMatrix hRef;
    dense_alloc_host(hRef, M, K);
    std::memcpy(hRef.data, hC.data, sizeof(float) * size_t(M) * size_t(K));
    dense_gemm_cpu(M, N, K, alpha, beta, hA, hB, hRef);

    CSRMatrix dA;
    csr_host2device(hA_csr, dA);
    EXPECT(dA.max_row_nnz == hA_csr.max_row_nnz && dA.nnz == hA_csr.nnz);
    CSRMatrix hA_again;
    csr_device2host(dA, hA_again);
    EXPECT(std::memcmp(hA_again.col_idx, hA_csr.col_idx, sizeof(int) * size_t(hA_csr.nnz)) == 0);
    csr_free_host(hA_again);
    EXPECT(hA_again.row_ptr == nullptr && hA_again.height == 0);

    // device-side conversions give the same arrays as the host ones
    {
        DenseMatrix dA_dense, dBack, hBack;
        dense_host2device(hA, dA_dense);
        CSRMatrix dA2, hA2;
        dense2csr_device(dA_dense, dA2, 0.0f);
        csr_device2host(dA2, hA2);
        EXPECT(hA2.nnz == hA_csr.nnz && hA2.max_row_nnz == hA_csr.max_row_nnz);
        EXPECT(std::memcmp(hA2.row_ptr, hA_csr.row_ptr, sizeof(int) * size_t(M + 1)) == 0);
        EXPECT(std::memcmp(hA2.col_idx, hA_csr.col_idx, sizeof(int) * size_t(hA_csr.nnz)) == 0);
        EXPECT(std::memcmp(hA2.values, hA_csr.values, sizeof(float) * size_t(hA_csr.nnz)) == 0);
        csr2dense_device(dA2, dBack);
        dense_device2host(dBack, hBack);
        EXPECT(dense_compare(hA, hBack, 0.0f));
        dense_free_host(hBack);
        dense_free_device(dBack);
        dense_free_device(dA_dense);
        csr_free_device(dA2);
        csr_free_host(hA2);
    }

    DenseMatrix dB;
    dense_host2device(hB, dB);
    for (const char* name : names) {
        DenseMatrix dC, hOut;
        dense_host2device(hC, dC);
        spmm(dA, dB, dC, alpha, beta, parse_algorithm(name));
        dense_device2host(dC, hOut);
        // integer data: every sum is exact in fp32; real data: accumulation-order tolerance
        // scaled by the magnitude of the sums (|a|,|b| <= 10, up to N terms)
        const float tol = integer_values ? 1e-2f : 1e-5f * 100.0f * float(N) + 1e-6f;
        // dense_compare keeps the reference's test (fabs(a-b) > tol, false for NaN), so finiteness is checked here
        const bool ok = dense_compare(hOut, hRef, tol) && all_finite(hOut);
        std::printf("%-18s %dx%dx%d s=%.2f a=%.2f b=%.2f int=%d nnz=%d max_row=%d : %s\n", name, M, N, K,
                    sparsity, alpha, beta, int(integer_values), hA_csr.nnz, hA_csr.max_row_nnz,
                    ok ? "ok" : "MISMATCH");
        EXPECT(ok);
        dense_free_host(hOut);
        dense_free_device(dC);
    }
    // asynchronous launcher + explicit sync
    {
        DenseMatrix dC, hOut;
        dense_host2device(hC, dC);
        launch_warp_per_row_fp4(dA, dB, dC, alpha, beta);
        EXPECT(last_launch_status() == 0);
        cudaCheck(cudaDeviceSynchronize());
        dense_device2host(dC, hOut);
        EXPECT(dense_compare(hOut, hRef, integer_values ? 1e-2f : 1e-5f * 100.0f * float(N) + 1e-6f));
        EXPECT(all_finite(hOut));
        dense_free_host(hOut);
        dense_free_device(dC);
    }
    dense_free_device(dB);
    csr_free_device(dA);
    csr_free_host(hA_csr);
    dense_free_host(hA);
    dense_free_host(hB);
    dense_free_host(hC);
    dense_free_host(hRef);
}

int main()
{
    EXPECT(parse_algorithm("WarpPerRowSmemFp4") == Algorithm::WarpPerRowSmemFp4);
    EXPECT(parse_algorithm("warp_per_row") == Algorithm::Naive);  // unknown -> Naive (+ warning)
    EXPECT(int(Algorithm::Naive) == 0 && int(Algorithm::NaiveSmem) == 1 && int(Algorithm::WarpPerRow) == 2 &&
           int(Algorithm::WarpPerRowFp4) == 3 && int(Algorithm::WarpPerRowSmem) == 4 &&
           int(Algorithm::WarpPerRowSmemFp4) == 5);
    EXPECT(WARP_SIZE == 32);

    run_case(256, 256, 64, 0.7f, 1.0f, 0.5f, true);     // the reference test's defaults, smaller
    run_case(300, 513, 128, 0.9f, 1.0f, 0.5f, true);    // M not a multiple of 4, odd width of A
    run_case(64, 2048, 256, 0.05f, 2.0f, -1.0f, true);  // rows longer than 1536: beyond the reference's smem kernels
    run_case(129, 77, 36, 0.5f, 1.5f, 0.0f, false);     // real values, beta = 0
    run_case(50, 40, 7, 0.8f, 1.0f, 1.0f, false);       // dense width not a multiple of 4

    std::printf(failures ? "FAILED (%d)\n" : "ALL OK\n", failures);
    return failures ? 1 : 0;
}
