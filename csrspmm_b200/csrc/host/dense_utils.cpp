// csrspmm::dense_* host utilities (declared in include/csrspmm/dense_utils.h).
//
// Same contract as the reference's src/host/dense_utils.cpp:12-162, written afresh with size_t
// sizing (the reference multiplies ints, src/host/dense_utils.cpp:20,38,52).  One deliberate
// difference: the reference re-creates its rand_r seed for every element
// (src/host/dense_utils.cpp:54-56), so all elements come out equal; dense_init_random here keeps
// ONE stream seeded with 1234 for the whole matrix, which is what the signature promises.
#include <csrspmm/dense_utils.h>
#include <csrspmm/error_check.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace csrspmm {

namespace {
[[noreturn]] void die(const char* msg)
{
    std::fprintf(stderr, "%s\n", msg);
    std::exit(1);
}
size_t elems(const DenseMatrix& A) { return size_t(A.height) * size_t(A.width); }
}  // namespace

void dense_alloc_host(DenseMatrix& A, int height, int width)
{
    if (A.data != nullptr) die("dense_alloc_host error: already allocated host memory.");
    A.height = height;
    A.width = width;
    A.data = static_cast<float*>(std::malloc(elems(A) * sizeof(float) + 4));
    if (A.data == nullptr) die("dense_alloc_host: malloc failed");
}

void dense_free_host(DenseMatrix& A)
{
    std::free(A.data);
    A.data = nullptr;
}

void dense_alloc_device(DenseMatrix& A, int height, int width)
{
    if (A.data != nullptr) die("dense_alloc_host error: already allocated device memory.");
    A.height = height;
    A.width = width;
    cudaCheck(cudaMalloc(reinterpret_cast<void**>(&A.data), elems(A) * sizeof(float) + 4));
}

void dense_free_device(DenseMatrix& A)
{
    cudaCheck(cudaFree(A.data));
    A.data = nullptr;
}

void dense_init_random(DenseMatrix& A, float low, float high, float sparsity, bool integer_values)
{
    unsigned int seed = 1234;
    const size_t total = elems(A);
    for (size_t i = 0; i < total; ++i) {
        const float keep_draw = float(rand_r(&seed)) / float(RAND_MAX);
        if (keep_draw < sparsity) {
            A.data[i] = 0.0f;
            continue;
        }
        const float v = float(rand_r(&seed)) / float(RAND_MAX) * (high - low) + low;
        A.data[i] = integer_values ? float(int(v)) : v;
    }
}

void print_dense(const DenseMatrix& A)
{
    std::printf("DenseMatrix (%dx%d):\n", A.height, A.width);
    for (int r = 0; r < A.height; ++r) {
        std::printf("  [ ");
        for (int c = 0; c < A.width; ++c)
            std::printf(c + 1 < A.width ? "%g, " : "%g", A.data[size_t(r) * size_t(A.width) + size_t(c)]);
        std::printf(" ]\n");
    }
    std::printf("\n");
}

bool dense_compare(const DenseMatrix& A, const DenseMatrix& B, float tol)
{
    if (A.height != B.height || A.width != B.width) {
        std::printf("Dense compare failed: shape mismatch\n");
        return false;
    }
    const size_t total = elems(A);
    for (size_t i = 0; i < total; ++i) {
        if (std::fabs(A.data[i] - B.data[i]) > tol) {
            std::printf("Mismatch at index %zu: %g vs %g\n", i, A.data[i], B.data[i]);
            return false;
        }
    }
    return true;
}

void dense_gemm_cpu(int M, int N, int K, float alpha, float beta, const DenseMatrix& A,
                    const DenseMatrix& B, DenseMatrix& C)
{
    // one fp32 accumulator per output, k ascending; C is always read (also for beta == 0), as in
    // the reference's src/host/dense_utils.cpp:114-123
    for (size_t i = 0; i < size_t(M); ++i) {
        for (size_t j = 0; j < size_t(K); ++j) {
            float sum = 0.0f;
            for (size_t k = 0; k < size_t(N); ++k)
                sum += A.data[i * size_t(N) + k] * B.data[k * size_t(K) + j];
            float& out = C.data[i * size_t(K) + j];
            out = alpha * sum + beta * out;
        }
    }
}

void dense_host2device(const DenseMatrix& hA, DenseMatrix& dA)
{
    if (!hA.data) die("dense_host2device: host data is null");
    if (dA.data != nullptr) die("dense_host2device error: Only accept null destination.");
    dense_alloc_device(dA, hA.height, hA.width);
    cudaCheck(cudaMemcpy(dA.data, hA.data, elems(hA) * sizeof(float), cudaMemcpyHostToDevice));
}

void dense_device2host(const DenseMatrix& dA, DenseMatrix& hA)
{
    if (!dA.data) die("dense_device2host: device data is null");
    if (hA.data != nullptr) die("dense_device2host error: only accept null destination.");
    dense_alloc_host(hA, dA.height, dA.width);
    cudaCheck(cudaMemcpy(hA.data, dA.data, elems(dA) * sizeof(float), cudaMemcpyDeviceToHost));
}

}  // namespace csrspmm
