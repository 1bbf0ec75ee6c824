// High-level entry point: C = alpha * A * B + beta * C with A in CSR (M x Kd), B dense row-major
// (Kd x Nd), C dense row-major (M x Nd).  Same surface as the reference's
// include/csrspmm/csrspmm.h:10-34: the Algorithm enumerators and their order, parse_algorithm's
// exact case-sensitive names with fall-back to Naive plus a warning on stderr, and a spmm() that
// returns only after the device finished, ending the process on a CUDA error.
//
// Every Algorithm value computes the same C.  The value records which of the reference's
// kernels the caller asked for and is used as a hint when the sm_100a kernel is chosen.
#pragma once
#include <string>

#include <csrspmm/config.h>
#include <csrspmm/csr_utils.h>
#include <csrspmm/kernels.h>
#include <csrspmm/matrix.h>

namespace csrspmm {

enum class Algorithm {
    Naive,
    NaiveSmem,
    WarpPerRow,
    WarpPerRowFp4,
    WarpPerRowSmem,
    WarpPerRowSmemFp4
};

Algorithm parse_algorithm(const std::string& name);

void spmm(const CSRMatrix& A, const DenseMatrix& B, DenseMatrix& C, float alpha, float beta,
          Algorithm algo = Algorithm::Naive);

}  // namespace csrspmm
