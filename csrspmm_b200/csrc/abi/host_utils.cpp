// Host-only entry points of the C ABI: CSR validation, the multi-GPU row partition and the
// e2m1 value codec.  None of them has a counterpart in the reference (its host layer,
// src/host/csr_utils.cpp and src/host/spmm_launcher.cu, validates and partitions nothing, and
// its "Fp4" kernels take fp32 values, src/device/csrspmm_warp_per_row_fp4.cu:9-19).
#include <cmath>
#include <cstring>

#include "csrspmm_b200.h"
#include "plan.h"

using namespace csrspmm_b200;

extern "C" {

int csrspmm_b200_validate_csr_host(int32_t M, int32_t Kd, int64_t nnz, const int32_t* row_ptr,
                                   const int32_t* col_idx, uint32_t* problems)
{
    if (M < 0 || Kd < 0 || nnz < 0 || row_ptr == nullptr || (nnz > 0 && col_idx == nullptr)) {
        set_last_error("validate_csr_host: bad argument");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    uint32_t bad = 0;
    if (row_ptr[0] != 0) bad |= CSRSPMM_B200_CSR_BAD_ROWPTR0;
    if ((int64_t)row_ptr[M] != nnz) bad |= CSRSPMM_B200_CSR_BAD_ROWPTR_END;
    for (int32_t r = 0; r < M; ++r) {
        const int32_t rs = row_ptr[r], re = row_ptr[r + 1];
        if (re < rs) {
            bad |= CSRSPMM_B200_CSR_NOT_MONOTONE;
            continue;
        }
        if (rs < 0 || (int64_t)re > nnz) continue;  // covered by the end checks / monotonicity
        int32_t prev = -1;
        for (int32_t j = rs; j < re; ++j) {
            const int32_t c = col_idx[j];
            if (c < 0 || c >= Kd) bad |= CSRSPMM_B200_CSR_COL_RANGE;
            if (c <= prev) bad |= CSRSPMM_B200_CSR_COL_UNSORTED;
            prev = c;
        }
    }
    if (problems != nullptr) *problems = bad;
    if (bad & 15u) {
        set_last_error("CSR validation failed, problem bits 0x%x", bad);
        return CSRSPMM_B200_ERR_INVALID_CSR;
    }
    return CSRSPMM_B200_OK;
}

int csrspmm_b200_partition_rows(int32_t M, const int32_t* row_ptr, int32_t parts, double row_weight,
                                int32_t* bounds)
{
    if (M < 0 || parts < 1 || row_ptr == nullptr || bounds == nullptr || row_weight < 0.0) {
        set_last_error("partition_rows: bad argument");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    // cost(r) = prefix cost of rows [0, r) = (row_ptr[r] - row_ptr[0]) + row_weight * r, which is
    // non-decreasing, so each boundary is a binary search for g/parts of the total.
    const double base = (double)row_ptr[0];
    auto cost = [&](int32_t r) { return ((double)row_ptr[r] - base) + row_weight * (double)r; };
    const double total = cost(M);
    bounds[0] = 0;
    for (int32_t g = 1; g < parts; ++g) {
        const double target = total * (double)g / (double)parts;
        int32_t lo = bounds[g - 1], hi = M;
        while (lo < hi) {  // first r with cost(r) >= target
            const int32_t mid = lo + (hi - lo) / 2;
            if (cost(mid) < target) lo = mid + 1;
            else hi = mid;
        }
        // the row before may be the closer cut
        if (lo > bounds[g - 1] && target - cost(lo - 1) < cost(lo) - target) --lo;
        bounds[g] = lo;
    }
    bounds[parts] = M;
    return CSRSPMM_B200_OK;
}

// ---- e2m1 ------------------------------------------------------------------------------------
static const float kMag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

static inline uint8_t encode_one(float v, float scale)
{
    if (v != v) return 0;
    const float q = v / scale;
    const uint8_t s = std::signbit(q) ? 8u : 0u;
    const float a = std::fabs(q);
    uint8_t code = 7;
    for (int k = 0; k < 7; ++k) {
        const float mid = 0.5f * (kMag[k] + kMag[k + 1]);
        if (a < mid || (a == mid && (k & 1) == 0)) {
            code = (uint8_t)k;
            break;
        }
    }
    return (uint8_t)(s | code);
}

float csrspmm_b200_e2m1_scale(int64_t n, const float* values)
{
    float mx = 0.0f;
    for (int64_t i = 0; i < n; ++i) {
        const float a = std::fabs(values[i]);
        if (a > mx) mx = a;
    }
    return mx > 0.0f ? mx / 6.0f : 1.0f;
}

int csrspmm_b200_e2m1_encode(int64_t n, const float* values, float scale, uint8_t* packed)
{
    if (n < 0 || (n > 0 && (values == nullptr || packed == nullptr)) || !(scale > 0.0f)) {
        set_last_error("e2m1_encode: bad argument");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    std::memset(packed, 0, (size_t)((n + 1) / 2));
    for (int64_t i = 0; i < n; ++i) {
        const uint8_t c = encode_one(values[i], scale);
        packed[i >> 1] |= (uint8_t)((i & 1) ? (c << 4) : c);
    }
    return CSRSPMM_B200_OK;
}

int csrspmm_b200_e2m1_decode(int64_t n, const uint8_t* packed, float scale, float* values)
{
    if (n < 0 || (n > 0 && (values == nullptr || packed == nullptr))) {
        set_last_error("e2m1_decode: bad argument");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    for (int64_t i = 0; i < n; ++i) {
        const uint8_t byte = packed[i >> 1];
        const uint8_t c = (i & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 15u);
        const float v = kMag[c & 7u] * scale;
        values[i] = (c & 8u) ? -v : v;
    }
    return CSRSPMM_B200_OK;
}

}  // extern "C"
