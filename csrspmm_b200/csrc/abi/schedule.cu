// Per-matrix schedules (csrspmm_b200_schedule_*) and the product that runs under one.
//
// The reference's spmm() has a place for a per-matrix decision and leaves it a stub: both branches
// of its row-length test pick Naive (src/csrspmm.cpp:34-40), and nothing is kept between calls.
// Here the analysis is real and persists: a schedule lists the long rows of one sparsity pattern
// and the pieces they are cut into, ordered by slab of B (kernels/sliced_kernel.cuh says why), and
// a product with args.schedule set runs
//     scheduled pieces  ->  per-row sum of their slots  ->  merge-path kernel over the other rows
//                                                           (+ its fix-up)
// on the caller's stream.  Built on the device: a pass over row_ptr lists the long rows, one warp
// per long row walks its columns once (ascending check, slab boundaries, piece counts), and a third
// pass writes the slab-major piece list.  Two small host reads size the arrays in between.
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../kernels/merge_kernel.cuh"
#include "../kernels/sliced_kernel.cuh"
#include "csrspmm_b200.h"
#include "launch.h"
#include "plan.h"

using namespace csrspmm_b200;

struct csrspmm_b200_schedule {
    uint32_t magic;
    int device;
    int32_t M, Kd, Nd;
    int64_t nnz;
    int32_t threshold, slab_rows, num_slabs, piece_nnz;
    int32_t num_long;
    int64_t long_nnz;
    int64_t num_pieces;
    int32_t columns_sorted;
    int4* pieces;     // device, num_pieces
    int4* long_rows;  // device, num_long: {row, first slot, slot count, 0}
    size_t device_bytes;
    double build_ms;
};

namespace {

constexpr uint32_t kScheduleMagic = 0x53434844u;  // "SCHD"
constexpr int kSlicedCtasPerSm = 3;  // more than fit is harmless: a late CTA finds the list used up
constexpr size_t kTicketBytes = 256;  // the ticket counter of the pieces kernel, in the call's scratch

#define CUDA_TRY(expr)                                                                      \
    do {                                                                                    \
        cudaError_t e__ = (expr);                                                           \
        if (e__ != cudaSuccess) {                                                           \
            set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, \
                           __LINE__);                                                       \
            return CSRSPMM_B200_ERR_CUDA;                                                   \
        }                                                                                   \
    } while (0)

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

int env_int(const char* name)
{
    const char* e = std::getenv(name);
    return (e != nullptr && *e != 0) ? std::atoi(e) : 0;
}

// Slab of B that should stay in L2 while its pieces run.  The 126 MB of L2 are two partitions, one per die, and
// a line that SMs of both dies read is held in both (tests/cpp/l2_partition_probe.cu measures it), so a slab
// of 64 MiB that every SM gathers from fills the L2 about once over, next to the streams of A and the slots;
// the pieces kernel then reads B from HBM about twice (once per die).  Smaller slabs are read once but cut
// the rows into more pieces, each with a slot of its own; measured on config 5 (rows of B of 2 KB), persistent
// pieces kernel, threshold 1024: 48 / 64 / 96 MiB gave 36.2 / 36.0 / 36.0 ms, against 40.5 ms without a schedule.
constexpr size_t kSlabBytes = (size_t)64 << 20;
// A row is scheduled when it has this many entries per slab on average: each piece costs a slot
// written and read back (one row of Nd floats each way), so a few entries per piece buy nothing.
// Config 5, 128 slabs of 64 MiB, persistent pieces kernel: 2 / 3 / 4 / 6 / 8 / 12 / 16 entries per
// slab gave 38.1 / 37.1 / 36.9 / 36.8 / 36.8 / 37.2 / 37.4 ms.
constexpr int kMinEntriesPerSlab = 8;
constexpr int kDefaultPiece = 64;
constexpr int kMaxPiece = 512;
// Below this many bytes per row of B the library schedules nothing unless a threshold is given.  With
// narrow rows the long rows' half of a product and the short rows' half add up either way, the
// pieces turn an HBM-bound half into an L2-bound one that is only a third shorter, and the slots and
// the stepping over scheduled rows in the merge-path kernel cost more than that.  Config 3 (256-byte
// rows): 0.60 ms without a schedule, 1.0 ms with one, although its pieces read 0.43 GB from HBM
// instead of 2.1 GB.
constexpr size_t kMinRowBytesForAuto = 1024;
// ... and nothing when the scheduled rows together name each row of B fewer than this many times: what the
// pieces save is the re-use of a slab's rows while it sits in L2, and a row block of a matrix cut across N
// GPUs has 1/N of the re-use (config 5: 8.1 / 4.0 / 2.0 / 1.0 entries per row of B on 1 / 2 / 4 / 8 GPUs;
// 40.5 -> 36.7 ms, 20.3 -> 18.7 ms and 10.2 -> 9.75 ms at 1, 2 and 4 GPUs).  At one use per row of B every
// row is fetched from HBM once either way and the slots come on top (8 GPUs: 5.09 ms without, 5.18 ms with).
constexpr double kMinReuseForAuto = 1.5;

bool valid(const csrspmm_b200_schedule* s) { return s != nullptr && s->magic == kScheduleMagic; }

bool env_forces_other_kernel()
{
    const char* e = std::getenv("CSRSPMM_FORCE_KERNEL");
    return e != nullptr && (!std::strcmp(e, "row") || !std::strcmp(e, "tma"));
}

// ---- kernel dispatch --------------------------------------------------------------------------------

template <class K>
cudaError_t allow_dynamic_smem(K kern, size_t bytes, bool (&configured)[64], size_t (&granted)[64])
{
    // the opt-in to more than 48 KB of dynamic shared memory is per device and instantiation;
    // repeated with a larger size when a later call needs more
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !configured[dev] || granted[dev] < bytes) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) {
            configured[dev] = true;
            granted[dev] = bytes;
        }
    }
    return cudaSuccess;
}

template <int S, int VW, int FMT, bool FULL>
cudaError_t launch_sliced_one(const SpmmParams& p, const SlicedParams& q, unsigned grid, cudaStream_t st)
{
    constexpr int G = kPieceShapes[S].G, NV = kPieceShapes[S].NV;
    constexpr int D = VW == 1 ? 16 : kPieceShapes[S].D;
    auto kern = spmm_sliced_kernel<G, NV, VW, D, FMT, FULL, CSRSPMM_TUNE_SLICED_MINB>;
    const size_t smem = sliced_smem_bytes(G, NV, VW, D, q.pieces_per_group, q.piece_cap);
    static bool configured[64] = {};
    static size_t granted[64] = {};
    cudaError_t e = allow_dynamic_smem(kern, smem, configured, granted);
    if (e != cudaSuccess) return e;
    kern<<<grid, kSlicedThreads, smem, st>>>(p, q);
    return cudaGetLastError();
}

template <int S, int VW, int FMT>
cudaError_t launch_sliced(const SpmmParams& p, const SlicedParams& q, const Plan& plan, unsigned grid, cudaStream_t st)
{
    if (VW == 4 && kPieceShapes[S].G * kPieceShapes[S].NV == plan.ncolv) return launch_sliced_one<S, VW, FMT, (VW == 4)>(p, q, grid, st);
    return launch_sliced_one<S, VW, FMT, false>(p, q, grid, st);
}

template <int VW, int FMT>
cudaError_t dispatch_sliced(const SpmmParams& p, const SlicedParams& q, const Plan& plan, unsigned grid, cudaStream_t st)
{
    switch (plan.shape) {
        case 0: return launch_sliced<0, VW, FMT>(p, q, plan, grid, st);
        case 1: return launch_sliced<1, VW, FMT>(p, q, plan, grid, st);
        case 2: return launch_sliced<2, VW, FMT>(p, q, plan, grid, st);
        case 3: return launch_sliced<3, VW, FMT>(p, q, plan, grid, st);
        default: return launch_sliced<4, VW, FMT>(p, q, plan, grid, st);
    }
}

// the merge-path kernel that leaves the scheduled rows alone (regular tile only)
template <int S, int VW, int FMT>
void launch_merge_skip(const SpmmParams& p, const Plan& plan, cudaStream_t st)
{
    constexpr int G = kShapes[S].G, NV = kShapes[S].NV, TG = kShapes[S].TG;
    constexpr int U = VW == 1 ? 8 : merge_unroll(NV);
    const unsigned grid = (unsigned)plan.grid;
    if (VW == 4 && plan.full) spmm_merge_kernel<G, NV, VW, TG, U, FMT, (VW == 4), true><<<grid, kMergeThreads, 0, st>>>(p);
    else spmm_merge_kernel<G, NV, VW, TG, U, FMT, false, true><<<grid, kMergeThreads, 0, st>>>(p);
}

template <int VW, int FMT>
void dispatch_merge_skip(const SpmmParams& p, const Plan& plan, cudaStream_t st)
{
    switch (plan.shape) {
        case 0: launch_merge_skip<0, VW, FMT>(p, plan, st); break;
        case 1: launch_merge_skip<1, VW, FMT>(p, plan, st); break;
        case 2: launch_merge_skip<2, VW, FMT>(p, plan, st); break;
        case 3: launch_merge_skip<3, VW, FMT>(p, plan, st); break;
        default: launch_merge_skip<4, VW, FMT>(p, plan, st); break;
    }
}

// Plan of the merge-path part of a scheduled product: MERGE, regular tile.
int scheduled_plan(const csrspmm_b200_args* a, Plan* plan)
{
    csrspmm_b200_args m = *a;
    m.kernel = CSRSPMM_B200_KERNEL_MERGE;
    m.schedule = nullptr;
    int status = make_plan(&m, plan, /*allow_narrow=*/false);  // the SKIP build exists for the regular shapes only
    if (status != CSRSPMM_B200_OK) return status;
    if (plan->small_tile) {  // few items but a large B: keep the one instantiated tile
        plan->small_tile = false;
        const int tile = (CSRSPMM_TUNE_MERGE_THREADS / kShapes[plan->shape].G) * kShapes[plan->shape].TG;
        plan->tile = tile;
        plan->num_tiles = (plan->num_items + tile - 1) / tile;
        plan->grid = plan->num_tiles;
        plan->workspace_bytes = 0;  // recomputed below
    }
    plan->carry_row_bytes = align256((size_t)plan->num_tiles * sizeof(int32_t));
    plan->workspace_bytes = plan->carry_row_bytes + align256((size_t)plan->num_tiles * (size_t)plan->carry_ld * sizeof(float));
    return CSRSPMM_B200_OK;
}

}  // namespace

namespace csrspmm_b200 {

bool schedule_applies(const csrspmm_b200_args* a)
{
    if (a == nullptr || !valid(a->schedule) || a->schedule->num_long <= 0 || a->schedule->num_pieces <= 0 ||
        env_forces_other_kernel())
        return false;
    if (a->kernel == CSRSPMM_B200_KERNEL_AUTO) {
        // rows known to be even: the whole-row kernel is what AUTO would run, and it is the better choice
        csrspmm_b200_args plain = *a;
        plain.schedule = nullptr;
        Plan plan;
        if (make_plan(&plain, &plan) == CSRSPMM_B200_OK && plan.kernel == CSRSPMM_B200_KERNEL_ROW) return false;
    }
    return true;
}

size_t scheduled_workspace_bytes(const csrspmm_b200_args* a)
{
    if (!schedule_applies(a) || check_args(a, false) != CSRSPMM_B200_OK) return 0;
    Plan plan;
    if (scheduled_plan(a, &plan) != CSRSPMM_B200_OK) return 0;
    const size_t slot_ld = ((size_t)a->Nd + 3) / 4 * 4;
    return plan.workspace_bytes + kTicketBytes + align256((size_t)a->schedule->num_pieces * slot_ld * sizeof(float));
}

int enqueue_scheduled(const csrspmm_b200_args* a, cudaStream_t st)
{
    const csrspmm_b200_schedule* s = a->schedule;
    if (a->kernel != CSRSPMM_B200_KERNEL_AUTO && a->kernel != CSRSPMM_B200_KERNEL_MERGE) {
        set_last_error("a schedule runs with kernel AUTO or MERGE, not %d", a->kernel);
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (a->row_ptr_base != 0) {
        set_last_error("a schedule describes a whole matrix: row_ptr_base must be 0");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (a->M != s->M || a->Kd != s->Kd || a->nnz != s->nnz) {
        set_last_error("schedule was built for M=%d Kd=%d nnz=%lld, the call has M=%d Kd=%d nnz=%lld", s->M, s->Kd,
                       (long long)s->nnz, a->M, a->Kd, (long long)a->nnz);
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    int device = -1;
    CUDA_TRY(cudaGetDevice(&device));
    if (device != s->device) {
        set_last_error("schedule lives on device %d, the current device is %d", s->device, device);
        return CSRSPMM_B200_ERR_BAD_ARG;
    }

    Plan plan;
    int status = scheduled_plan(a, &plan);
    if (status != CSRSPMM_B200_OK) return status;
    const size_t slot_ld = ((size_t)a->Nd + 3) / 4 * 4;
    const size_t need = plan.workspace_bytes + kTicketBytes + align256((size_t)s->num_pieces * slot_ld * sizeof(float));

    void* ws = nullptr;
    bool ws_owned = false;
    if (a->workspace != nullptr) {
        if (a->workspace_bytes < need || (reinterpret_cast<uintptr_t>(a->workspace) & 255u) != 0) {
            set_last_error("workspace of %zu bytes at %p: a scheduled product needs %zu bytes, 256-byte aligned",
                           a->workspace_bytes, a->workspace, need);
            return CSRSPMM_B200_ERR_WORKSPACE;
        }
        ws = a->workspace;
    } else {
        CUDA_TRY(cudaMallocAsync(&ws, need, st));
        ws_owned = true;
    }

    SpmmParams p;
    fill_params(a, plan, &p);
    set_carry_scratch(plan, ws, &p);
    p.skip_len = s->threshold;

    SlicedParams q;
    std::memset(&q, 0, sizeof(q));
    q.pieces = s->pieces;
    q.num_pieces = (int)s->num_pieces;
    q.pieces_per_group = CSRSPMM_TUNE_SLICED_PIECES_PER_GROUP;
    q.piece_cap = s->piece_nnz;
    q.tickets = reinterpret_cast<unsigned*>(static_cast<char*>(ws) + plan.workspace_bytes);
    q.slots = reinterpret_cast<float*>(static_cast<char*>(ws) + plan.workspace_bytes + kTicketBytes);
    q.slot_ld = (long long)slot_ld;
    q.long_rows = s->long_rows;
    q.num_long_rows = s->num_long;
    q.evict_last = CSRSPMM_TUNE_SLICED_EVICT_LAST;

    const bool e2m1 = a->value_format == CSRSPMM_B200_VALUES_E2M1;
    // a persistent grid: every warp draws runs of pieces until the list is used up
    const long long per_cta = (long long)(kSlicedThreads / kPieceShapes[plan.shape].G) * q.pieces_per_group;
    const long long ctas_of_work = (s->num_pieces + per_cta - 1) / per_cta + 1;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const unsigned grid_pieces = (unsigned)std::min<long long>(ctas_of_work, (long long)sms * kSlicedCtasPerSm);
    cudaError_t err = cudaMemsetAsync(q.tickets, 0, kTicketBytes, st);
    if (err == cudaSuccess) {
        if (plan.VW == 4) {
            err = e2m1 ? dispatch_sliced<4, kValuesE2M1>(p, q, plan, grid_pieces, st) : dispatch_sliced<4, kValuesF32>(p, q, plan, grid_pieces, st);
        } else {
            err = e2m1 ? dispatch_sliced<1, kValuesE2M1>(p, q, plan, grid_pieces, st) : dispatch_sliced<1, kValuesF32>(p, q, plan, grid_pieces, st);
        }
    }
    if (err == cudaSuccess) {
        const long long threads = (long long)s->num_long * plan.ncolv;
        const unsigned grid = (unsigned)((threads + 255) / 256);
        if (plan.VW == 4) spmm_slot_reduce_kernel<4><<<grid, 256, 0, st>>>(p, q);
        else spmm_slot_reduce_kernel<1><<<grid, 256, 0, st>>>(p, q);
        err = cudaGetLastError();
    }
    if (err == cudaSuccess) {
        if (plan.VW == 4) {
            if (e2m1) dispatch_merge_skip<4, kValuesE2M1>(p, plan, st);
            else dispatch_merge_skip<4, kValuesF32>(p, plan, st);
        } else {
            if (e2m1) dispatch_merge_skip<1, kValuesE2M1>(p, plan, st);
            else dispatch_merge_skip<1, kValuesF32>(p, plan, st);
        }
        if (err == cudaSuccess) err = cudaGetLastError();
        if (err == cudaSuccess) err = launch_fixup_kernel(p, plan, st);
    }
    if (ws_owned) {
        cudaError_t ferr = cudaFreeAsync(ws, st);
        if (err == cudaSuccess) err = ferr;
    }
    if (err != cudaSuccess) {
        set_last_error("scheduled product: kernel launch failed: %s", cudaGetErrorString(err));
        return CSRSPMM_B200_ERR_CUDA;
    }
    return CSRSPMM_B200_OK;
}

}  // namespace csrspmm_b200

extern "C" {

int csrspmm_b200_schedule_create(const csrspmm_b200_args* a, const csrspmm_b200_schedule_options* options,
                                 csrspmm_b200_schedule** out, csrspmm_b200_stream_t stream)
{
    if (out == nullptr) {
        set_last_error("schedule_create: out is null");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    *out = nullptr;
    int status = check_args(a, false);
    if (status != CSRSPMM_B200_OK) return status;
    if (a->M > 0 && (a->row_ptr == nullptr || (a->nnz > 0 && a->col_idx == nullptr))) {
        set_last_error("schedule_create: null row_ptr or col_idx");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (a->row_ptr_base != 0) {
        set_last_error("schedule_create: row_ptr_base must be 0 (a schedule describes a whole matrix)");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    if (options != nullptr && options->struct_size != sizeof(csrspmm_b200_schedule_options)) {
        set_last_error("schedule_create: options.struct_size is %u, expected %zu", options->struct_size,
                       sizeof(csrspmm_b200_schedule_options));
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    const auto t0 = std::chrono::steady_clock::now();
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

    int threshold = options ? options->long_row_threshold : 0;
    int slab_rows = options ? options->slab_rows : 0;
    int piece = options ? options->piece_nnz : 0;
    if (threshold <= 0) threshold = env_int("CSRSPMM_SCHED_THRESHOLD");
    if (piece <= 0) piece = env_int("CSRSPMM_SCHED_PIECE");
    if (piece <= 0) piece = kDefaultPiece;
    if (piece > kMaxPiece) piece = kMaxPiece;  // a lane group stages a whole piece in shared memory
    const size_t row_bytes = (size_t)(a->ldb > 0 ? a->ldb : 1) * 4;
    if (slab_rows <= 0) {
        size_t slab = kSlabBytes;
        if (const int mib = env_int("CSRSPMM_SCHED_SLAB_MIB")) slab = (size_t)mib << 20;
        size_t rows = slab / row_bytes;
        if (rows < 256) rows = 256;
        slab_rows = rows > (size_t)0x7fffffff ? 0x7fffffff : (int)rows;
    }
    const int Kd = a->Kd > 0 ? a->Kd : 1;
    long long num_slabs_ll = ((long long)Kd + slab_rows - 1) / slab_rows;
    if (num_slabs_ll > 4096) {  // keep the per-row table bounded: widen the slabs instead
        slab_rows = (int)(((long long)Kd + 4095) / 4096);
        num_slabs_ll = ((long long)Kd + slab_rows - 1) / slab_rows;
    }
    const int num_slabs = (int)num_slabs_ll;
    // a B that fits one slab is served from L2 whatever the order: nothing to schedule
    const bool pointless = num_slabs <= 1;
    bool pointless_auto = false;
    const bool auto_threshold = threshold <= 0;
    if (threshold <= 0) {
        const long long t = (long long)kMinEntriesPerSlab * num_slabs;
        threshold = t > 0x3fffffff ? 0x3fffffff : (int)t;
        if (threshold < 32) threshold = 32;
        pointless_auto = (size_t)a->Nd * 4 < kMinRowBytesForAuto;
    }

    csrspmm_b200_schedule* s = new (std::nothrow) csrspmm_b200_schedule();
    if (s == nullptr) {
        set_last_error("schedule_create: out of host memory");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    std::memset(s, 0, sizeof(*s));
    s->magic = kScheduleMagic;
    s->M = a->M;
    s->Kd = a->Kd;
    s->Nd = a->Nd;
    s->nnz = a->nnz;
    s->threshold = threshold;
    s->slab_rows = slab_rows;
    s->num_slabs = num_slabs;
    s->piece_nnz = piece;
    s->columns_sorted = 1;

    unsigned* d_counters = nullptr;
    int* d_rows = nullptr;
    int* d_bounds = nullptr;
    unsigned* d_slab = nullptr;
    auto fail = [&](int code) {
        cudaStreamSynchronize(st);
        cudaFree(d_counters);
        cudaFree(d_rows);
        cudaFree(d_bounds);
        cudaFree(d_slab);
        cudaFree(s->pieces);
        cudaFree(s->long_rows);
        delete s;
        return code;
    };
#define SCHED_TRY(expr)                                                                       \
    do {                                                                                      \
        cudaError_t e__ = (expr);                                                             \
        if (e__ != cudaSuccess) {                                                             \
            set_last_error("schedule_create: %s failed: %s", #expr, cudaGetErrorString(e__)); \
            return fail(CSRSPMM_B200_ERR_CUDA);                                               \
        }                                                                                     \
    } while (0)

    SCHED_TRY(cudaGetDevice(&s->device));
    if (!pointless && !pointless_auto && a->M > 0 && a->nnz > 0) {
        SCHED_TRY(cudaMalloc(reinterpret_cast<void**>(&d_counters), kSchedCounters * sizeof(unsigned)));
        SCHED_TRY(cudaMemsetAsync(d_counters, 0, kSchedCounters * sizeof(unsigned), st));
        // a row of `threshold` entries or more: at most nnz / threshold of them
        const long long cap_ll = a->nnz / threshold + 1;
        const int capacity = (int)(cap_ll < (long long)a->M ? cap_ll : (long long)a->M);
        SCHED_TRY(cudaMalloc(reinterpret_cast<void**>(&d_rows), (size_t)capacity * sizeof(int)));
        long long blocks = ((long long)a->M + 255) / 256;
        if (blocks > 148 * 16) blocks = 148 * 16;
        sched_list_long_rows_kernel<<<(unsigned)blocks, 256, 0, st>>>(a->M, a->row_ptr, threshold, d_rows, capacity, d_counters);
        SCHED_TRY(cudaGetLastError());
        unsigned h_counters[kSchedCounters] = {};
        SCHED_TRY(cudaMemcpyAsync(h_counters, d_counters, sizeof(h_counters), cudaMemcpyDeviceToHost, st));
        SCHED_TRY(cudaStreamSynchronize(st));
        long long num_long = h_counters[0];
        if (num_long > capacity) num_long = capacity;  // only a malformed row_ptr gets here
        unsigned long long long_nnz = 0;
        std::memcpy(&long_nnz, &h_counters[2], sizeof(long_nnz));
        if (auto_threshold && (double)long_nnz < kMinReuseForAuto * (double)Kd) num_long = 0;  // too little re-use of B

        if (num_long > 0) {
            const size_t bounds_bytes = (size_t)num_long * (size_t)(num_slabs + 1) * sizeof(int);
            SCHED_TRY(cudaMalloc(reinterpret_cast<void**>(&d_bounds), bounds_bytes));
            SCHED_TRY(cudaMemsetAsync(d_bounds, 0, bounds_bytes, st));
            SCHED_TRY(cudaMalloc(reinterpret_cast<void**>(&d_slab), (size_t)num_slabs * 2 * sizeof(unsigned)));
            SCHED_TRY(cudaMemsetAsync(d_slab, 0, (size_t)num_slabs * 2 * sizeof(unsigned), st));
            SCHED_TRY(cudaMalloc(reinterpret_cast<void**>(&s->long_rows), (size_t)num_long * sizeof(int4)));
            const int warps = 8;
            sched_cut_rows_kernel<<<(unsigned)((num_long + warps - 1) / warps), warps * 32, 0, st>>>(
                (int)num_long, d_rows, a->row_ptr, a->col_idx, (int)a->nnz, slab_rows, num_slabs, piece, d_bounds, d_slab,
                s->long_rows, d_counters);
            SCHED_TRY(cudaGetLastError());
            std::vector<unsigned> slab_count((size_t)num_slabs);
            SCHED_TRY(cudaMemcpyAsync(h_counters, d_counters, sizeof(h_counters), cudaMemcpyDeviceToHost, st));
            SCHED_TRY(cudaMemcpyAsync(slab_count.data(), d_slab, (size_t)num_slabs * sizeof(unsigned), cudaMemcpyDeviceToHost, st));
            SCHED_TRY(cudaStreamSynchronize(st));
            const bool sorted = h_counters[4] == 0;
            long long total = 0;
            std::vector<unsigned> slab_first((size_t)num_slabs);
            for (int k = 0; k < num_slabs; ++k) {
                slab_first[(size_t)k] = (unsigned)total;
                total += slab_count[(size_t)k];
            }
            if (!sorted) {
                s->columns_sorted = 0;  // an empty schedule: the plain kernels run
            } else if (total > 0 && total <= 0x7fffffffLL && total == (long long)h_counters[5]) {
                SCHED_TRY(cudaMalloc(reinterpret_cast<void**>(&s->pieces), (size_t)total * sizeof(int4)));
                unsigned* d_fill = d_slab + num_slabs;
                SCHED_TRY(cudaMemcpyAsync(d_fill, slab_first.data(), (size_t)num_slabs * sizeof(unsigned), cudaMemcpyHostToDevice, st));
                sched_emit_pieces_kernel<<<(unsigned)((num_long + 127) / 128), 128, 0, st>>>(
                    (int)num_long, num_slabs, piece, d_bounds, d_fill, s->long_rows, s->pieces, (int)total);
                SCHED_TRY(cudaGetLastError());
                SCHED_TRY(cudaStreamSynchronize(st));
                s->num_long = (int32_t)num_long;
                s->long_nnz = (int64_t)long_nnz;
                s->num_pieces = total;
                s->device_bytes = (size_t)total * sizeof(int4) + (size_t)num_long * sizeof(int4);
            }
        }
        cudaFree(d_counters);
        cudaFree(d_rows);
        cudaFree(d_bounds);
        cudaFree(d_slab);
        d_counters = nullptr;
        d_rows = nullptr;
        d_bounds = nullptr;
        d_slab = nullptr;
        if (s->num_long == 0) {  // nothing scheduled: keep no device memory
            cudaFree(s->pieces);
            cudaFree(s->long_rows);
            s->pieces = nullptr;
            s->long_rows = nullptr;
        }
    }
#undef SCHED_TRY
    s->build_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    *out = s;
    return CSRSPMM_B200_OK;
}

int csrspmm_b200_schedule_destroy(csrspmm_b200_schedule* s)
{
    if (s == nullptr) return CSRSPMM_B200_OK;
    if (!valid(s)) {
        set_last_error("schedule_destroy: not a schedule");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    int current = -1;
    const bool switched = cudaGetDevice(&current) == cudaSuccess && current != s->device && cudaSetDevice(s->device) == cudaSuccess;
    cudaFree(s->pieces);
    cudaFree(s->long_rows);
    if (switched) cudaSetDevice(current);
    s->magic = 0;
    delete s;
    return CSRSPMM_B200_OK;
}

int csrspmm_b200_schedule_info_get(const csrspmm_b200_schedule* s, csrspmm_b200_schedule_info* info)
{
    if (!valid(s) || info == nullptr || info->struct_size != sizeof(csrspmm_b200_schedule_info)) {
        set_last_error("schedule_info_get: bad schedule or info.struct_size");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    info->M = s->M;
    info->Kd = s->Kd;
    info->Nd = s->Nd;
    info->nnz = s->nnz;
    info->long_row_threshold = s->threshold;
    info->slab_rows = s->slab_rows;
    info->num_slabs = s->num_slabs;
    info->piece_nnz = s->piece_nnz;
    info->long_rows = s->num_long;
    info->long_nnz = s->long_nnz;
    info->pieces = s->num_pieces;
    info->columns_sorted = s->columns_sorted;
    info->device_bytes = s->device_bytes;
    info->build_ms = s->build_ms;
    return CSRSPMM_B200_OK;
}

}  // extern "C"
