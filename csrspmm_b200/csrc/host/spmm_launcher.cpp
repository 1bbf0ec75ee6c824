// csrspmm::launch_* (declared in include/csrspmm/spmm_launcher.cuh) and csrspmm::spmm /
// parse_algorithm (include/csrspmm/csrspmm.h).
//
// The reference gives each launcher its own fixed grid and kernel
// (src/host/spmm_launcher.cu:11-171) and its spmm() switches over them (src/csrspmm.cpp:42-71).
// Here every launcher fills the C-ABI argument block from the two POD views and lets the kernel
// library plan the launch; the entry value records which reference kernel was asked for.
#include <csrspmm/csrspmm.h>
#include <csrspmm/error_check.h>
#include <csrspmm/spmm_launcher.cuh>

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <mutex>

#include "csrspmm_b200.h"

namespace csrspmm {

namespace {

thread_local int g_last_launch_status = CSRSPMM_B200_OK;

// The longest row of a device-resident matrix, measured once (one small kernel and a host read on
// the legacy default stream) and remembered per (device, row_ptr address, rows, nnz).  It steers
// the kernel choice only: a matrix whose rows are known to be even takes the whole-row kernel,
// anything else the merge-path kernel.  CSRMatrix::max_row_nnz is the caller's claim -- the
// reference's wrappers leave it unset on three of five ops
// (torch_csrspmm/torch_csrspmm_warp_per_row.cpp:34-40) and a stale value would send a skewed matrix
// to the whole-row kernel -- so it is used only when measuring fails.  A stale cache entry (another
// matrix of the same size placed at the same address) costs speed, never correctness.
struct RowStatsEntry {
    int device;
    const int* row_ptr;
    int rows;
    int nnz;
    int longest;
};
constexpr int kRowStatsEntries = 64;
std::mutex g_row_stats_mutex;
RowStatsEntry g_row_stats[kRowStatsEntries] = {};
int g_row_stats_next = 0;

int longest_row_of(const CSRMatrix& A)
{
    if (A.height <= 0 || A.nnz <= 0 || A.row_ptr == nullptr) return 0;
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess) return A.max_row_nnz;
    {
        std::lock_guard<std::mutex> lock(g_row_stats_mutex);
        for (const RowStatsEntry& e : g_row_stats)
            if (e.row_ptr == A.row_ptr && e.device == device && e.rows == A.height && e.nnz == A.nnz) return e.longest;
    }
    int64_t stats[4] = {0, 0, 0, 0};
    if (csrspmm_b200_row_stats_device(A.height, A.row_ptr, stats, nullptr) != CSRSPMM_B200_OK) return A.max_row_nnz;
    const int longest = stats[0] > 0x7fffffff ? 0x7fffffff : (int)stats[0];
    std::lock_guard<std::mutex> lock(g_row_stats_mutex);
    g_row_stats[g_row_stats_next] = RowStatsEntry{device, A.row_ptr, A.height, A.nnz, longest};
    g_row_stats_next = (g_row_stats_next + 1) % kRowStatsEntries;
    return longest;
}

void launch(const CSRMatrix& A, const DenseMatrix& B, DenseMatrix& C, float alpha, float beta,
            csrspmm_b200_entry entry)
{
    csrspmm_b200_args a = {};
    a.struct_size = sizeof(a);
    a.M = A.height;
    a.Kd = A.width;
    a.Nd = B.width;
    a.nnz = A.nnz;
    a.row_ptr = A.row_ptr;
    a.col_idx = A.col_idx;
    a.values = A.values;
    a.value_format = CSRSPMM_B200_VALUES_F32;
    a.value_scale = 1.0f;
    a.B = B.data;
    a.ldb = B.width;
    a.C = C.data;
    a.ldc = B.width;  // C is M x Nd with the reference's packed layout, whatever C.width says
    a.alpha = alpha;
    a.beta = beta;
    a.entry = entry;
    a.kernel = CSRSPMM_B200_KERNEL_AUTO;
    a.max_row_nnz = longest_row_of(A);
    const int status = csrspmm_b200_spmm(&a, nullptr);  // legacy default stream, like the reference
    g_last_launch_status = status;
    if (status != CSRSPMM_B200_OK)
        std::fprintf(stderr, "[csrspmm] launch failed: %s: %s\n", csrspmm_b200_status_string(status),
                     csrspmm_b200_last_error());
}

}  // namespace

int last_launch_status()
{
    const int s = g_last_launch_status;
    g_last_launch_status = CSRSPMM_B200_OK;
    return s;
}

void launch_naive(const CSRMatrix& A, const DenseMatrix& B, DenseMatrix& C, float alpha, float beta)
{
    launch(A, B, C, alpha, beta, CSRSPMM_B200_ENTRY_NAIVE);
}

void launch_naive_smem(const CSRMatrix& A, const DenseMatrix& B, DenseMatrix& C, float alpha, float beta)
{
    launch(A, B, C, alpha, beta, CSRSPMM_B200_ENTRY_NAIVE_SMEM);
}

void launch_warp_per_row(const CSRMatrix& A, const DenseMatrix& B, DenseMatrix& C, float alpha, float beta)
{
    launch(A, B, C, alpha, beta, CSRSPMM_B200_ENTRY_WARP_PER_ROW);
}

void launch_warp_per_row_fp4(const CSRMatrix& A, const DenseMatrix& B, DenseMatrix& C, float alpha,
                             float beta)
{
    launch(A, B, C, alpha, beta, CSRSPMM_B200_ENTRY_WARP_PER_ROW_FP4);
}

void launch_warp_per_row_smem(const CSRMatrix& A, const DenseMatrix& B, DenseMatrix& C, float alpha,
                              float beta)
{
    launch(A, B, C, alpha, beta, CSRSPMM_B200_ENTRY_WARP_PER_ROW_SMEM);
}

void launch_warp_per_row_smem_fp4(const CSRMatrix& A, const DenseMatrix& B, DenseMatrix& C, float alpha,
                                  float beta)
{
    launch(A, B, C, alpha, beta, CSRSPMM_B200_ENTRY_WARP_PER_ROW_SMEM_FP4);
}

Algorithm parse_algorithm(const std::string& name)
{
    static const struct {
        const char* name;
        Algorithm algo;
    } table[] = {{"Naive", Algorithm::Naive},
                 {"NaiveSmem", Algorithm::NaiveSmem},
                 {"WarpPerRow", Algorithm::WarpPerRow},
                 {"WarpPerRowFp4", Algorithm::WarpPerRowFp4},
                 {"WarpPerRowSmem", Algorithm::WarpPerRowSmem},
                 {"WarpPerRowSmemFp4", Algorithm::WarpPerRowSmemFp4}};
    for (const auto& e : table)
        if (name == e.name) return e.algo;
    std::cerr << "[csrspmm] Unknown algorithm: " << name << ", using Naive\n";
    return Algorithm::Naive;
}

void spmm(const CSRMatrix& A, const DenseMatrix& B, DenseMatrix& C, float alpha, float beta, Algorithm algo)
{
    switch (algo) {
        case Algorithm::Naive: launch_naive(A, B, C, alpha, beta); break;
        case Algorithm::NaiveSmem: launch_naive_smem(A, B, C, alpha, beta); break;
        case Algorithm::WarpPerRow: launch_warp_per_row(A, B, C, alpha, beta); break;
        case Algorithm::WarpPerRowFp4: launch_warp_per_row_fp4(A, B, C, alpha, beta); break;
        case Algorithm::WarpPerRowSmem: launch_warp_per_row_smem(A, B, C, alpha, beta); break;
        case Algorithm::WarpPerRowSmemFp4: launch_warp_per_row_smem_fp4(A, B, C, alpha, beta); break;
        default: std::printf("[csrspmm::spmm] Invalid Algorithm.\n"); return;
    }
    // synchronous and fatal, as src/csrspmm.cpp:73-74 of the reference
    if (last_launch_status() != CSRSPMM_B200_OK) std::exit(EXIT_FAILURE);
    cudaCheck(cudaGetLastError());
    cudaCheck(cudaDeviceSynchronize());
}

}  // namespace csrspmm
