// extern "C" entry points of the kernel library (declared in include/csrspmm_b200.h).
//
// This file owns every kernel launch.  It stands where the reference's launchers do
// (src/host/spmm_launcher.cu:11-171), but chooses the geometry from the problem instead of
// fixing it, reports failures as status codes instead of ignoring them, and takes the stream
// from the caller instead of always using the legacy default stream.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "../kernels/aux_kernels.cuh"
#include "../kernels/merge_kernel.cuh"
#include "../kernels/row_kernel.cuh"
#include "../kernels/tma_kernel.cuh"
#include "csrspmm_b200.h"
#include "launch.h"
#include "plan.h"

using namespace csrspmm_b200;

namespace csrspmm_b200 {

void fill_params(const csrspmm_b200_args* a, const Plan& plan, SpmmParams* out)
{
    SpmmParams p;
    std::memset(&p, 0, sizeof(p));
    p.M = a->M;
    p.Kd = a->Kd;
    p.Nd = a->Nd;
    p.nnz = (int)a->nnz;
    p.ncolv = plan.ncolv;
    p.num_items = plan.num_items;
    p.row_ptr = a->row_ptr;
    p.rp_base = a->row_ptr_base;
    p.col_idx = a->col_idx;
    p.values = a->values;
    p.value_scale = a->value_scale;
    p.B = a->B;
    p.ldb = a->ldb;
    p.ldb_bytes = (unsigned)(a->ldb * 4);
    p.C = a->C;
    p.ldc = a->ldc;
    p.alpha = a->alpha;
    p.beta = a->beta;
    p.status_word = a->status_word;
    // CSRSPMM_TEST_WAIT_LIMIT=<n> (tests only): a wait on a row copy gives up after n attempts, so the
    // give-up path can be exercised without anything being stuck (the drain wait keeps the full limit)
    p.wait_limit = kWaitSpinLimit;
    if (const char* e = std::getenv("CSRSPMM_TEST_WAIT_LIMIT"))
        if (*e != 0) p.wait_limit = (unsigned)std::strtoul(e, nullptr, 10);
    *out = p;
}

void set_carry_scratch(const Plan& plan, void* workspace, SpmmParams* p)
{
    p->carry_row = static_cast<int*>(workspace);
    p->carry_val = reinterpret_cast<float*>(static_cast<char*>(workspace) + plan.carry_row_bytes);
    p->carry_ld = plan.carry_ld;
}

}  // namespace csrspmm_b200

namespace {

#define CUDA_TRY(expr)                                                                      \
    do {                                                                                    \
        cudaError_t e__ = (expr);                                                           \
        if (e__ != cudaSuccess) {                                                           \
            set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, \
                           __LINE__);                                                       \
            return CSRSPMM_B200_ERR_CUDA;                                                   \
        }                                                                                   \
    } while (0)

template <int S, int VW, int FMT>
void launch_row(const SpmmParams& p, const Plan& plan, cudaStream_t st)
{
    constexpr int G = kShapes[S].G, NV = kShapes[S].NV;
    constexpr int U = VW == 1 ? 8 : row_unroll(NV);
    constexpr int ULOW = VW == 1 ? 8 : row_unroll_low(NV);
    constexpr int MINB = row_min_blocks(NV);
    const unsigned grid = (unsigned)plan.grid;
    if (VW == 4 && plan.full) {
        if (plan.low_occupancy && ULOW != U)
            spmm_row_kernel<G, NV, VW, ULOW, FMT, (VW == 4), 2><<<grid, kRowThreads, 0, st>>>(p);
        else
            spmm_row_kernel<G, NV, VW, U, FMT, (VW == 4), MINB><<<grid, kRowThreads, 0, st>>>(p);
    } else {
        if (plan.low_occupancy && ULOW != U)
            spmm_row_kernel<G, NV, VW, ULOW, FMT, false, 2><<<grid, kRowThreads, 0, st>>>(p);
        else
            spmm_row_kernel<G, NV, VW, U, FMT, false, MINB><<<grid, kRowThreads, 0, st>>>(p);
    }
}

template <int NV, int FMT>
cudaError_t launch_tma(const SpmmParams& p, const Plan& plan, cudaStream_t st)
{
    auto kern = spmm_tma_kernel<NV, CSRSPMM_TUNE_TMA_TG, CSRSPMM_TUNE_TMA_SLOTS, FMT>;
    // The opt-in to more than 48 KB of dynamic shared memory is made once per device and
    // instantiation, for the largest ring the kernel can ask for (rows of 2 KB), so that later
    // calls -- inside a stream capture too -- are a plain launch.  Racing first calls repeat the
    // same setting.
    constexpr int kMaxRing = (CSRSPMM_TUNE_MERGE_THREADS / 32) * (CSRSPMM_TUNE_TMA_SLOTS * 2048 > 512 * NV ? CSRSPMM_TUNE_TMA_SLOTS * 2048 : 512 * NV);
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !configured[dev] || (int)plan.dynamic_smem > kMaxRing) {
        const int want = (int)plan.dynamic_smem > kMaxRing ? (int)plan.dynamic_smem : kMaxRing;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, want);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    kern<<<(unsigned)plan.grid, kMergeThreads, plan.dynamic_smem, st>>>(p, (unsigned)plan.tma_slot_bytes,
                                                                        (unsigned)(plan.dynamic_smem / (CSRSPMM_TUNE_MERGE_THREADS / 32)));
    return cudaSuccess;
}

template <int VW, int FMT>
void dispatch_row(const SpmmParams& p, const Plan& plan, cudaStream_t st)
{
    switch (plan.shape) {
        case 0: launch_row<0, VW, FMT>(p, plan, st); break;
        case 1: launch_row<1, VW, FMT>(p, plan, st); break;
        case 2: launch_row<2, VW, FMT>(p, plan, st); break;
        case 3: launch_row<3, VW, FMT>(p, plan, st); break;
        default: launch_row<4, VW, FMT>(p, plan, st); break;
    }
}

template <int FMT>
cudaError_t dispatch_tma(const SpmmParams& p, const Plan& plan, cudaStream_t st)
{
    switch (plan.NV) {
        case 1: return launch_tma<1, FMT>(p, plan, st);
        case 2: return launch_tma<2, FMT>(p, plan, st);
        default: return launch_tma<4, FMT>(p, plan, st);
    }
}

// CSRSPMM_VALIDATE=1 in the environment: check the CSR structure on the device before every
// product (costs a kernel and a stream synchronisation; off by default).
bool validation_requested()
{
    static const bool on = [] {
        const char* e = std::getenv("CSRSPMM_VALIDATE");
        return e != nullptr && *e != 0 && *e != '0';
    }();
    return on;
}

int enqueue(const csrspmm_b200_args* a, cudaStream_t st)
{
    int status = check_args(a, true);
    if (status != CSRSPMM_B200_OK) return status;
    if (a->M == 0 || a->Nd == 0) return CSRSPMM_B200_OK;
    if (validation_requested() && a->row_ptr_base == 0) {
        uint32_t problems = 0;
        status = csrspmm_b200_validate_csr_device(a->M, a->Kd, a->nnz, a->row_ptr, a->col_idx, &problems,
                                                  reinterpret_cast<csrspmm_b200_stream_t>(st));
        if (status != CSRSPMM_B200_OK) return status;
    }

    if (schedule_applies(a)) return enqueue_scheduled(a, st);

    Plan plan;
    status = make_plan(a, &plan);
    if (status != CSRSPMM_B200_OK) return status;

    SpmmParams p;
    fill_params(a, plan, &p);

    const bool split = plan.kernel != CSRSPMM_B200_KERNEL_ROW;
    void* ws = nullptr;
    bool ws_owned = false;
    if (split) {
        if (a->workspace != nullptr) {
            if (a->workspace_bytes < plan.workspace_bytes ||
                (reinterpret_cast<uintptr_t>(a->workspace) & 255u) != 0) {
                set_last_error("workspace of %zu bytes at %p: need %zu bytes, 256-byte aligned",
                               a->workspace_bytes, a->workspace, plan.workspace_bytes);
                return CSRSPMM_B200_ERR_WORKSPACE;
            }
            ws = a->workspace;
        } else {
            CUDA_TRY(cudaMallocAsync(&ws, plan.workspace_bytes, st));
            ws_owned = true;
        }
        set_carry_scratch(plan, ws, &p);
    }

    const bool e2m1 = a->value_format == CSRSPMM_B200_VALUES_E2M1;
    cudaError_t attr_err = cudaSuccess;
    if (plan.kernel == CSRSPMM_B200_KERNEL_ROW) {
        attr_err = launch_row_kernel(p, plan, e2m1, st);
    } else if (plan.kernel == CSRSPMM_B200_KERNEL_MERGE) {
        attr_err = launch_merge_kernel(p, plan, e2m1, st);
    } else {
        attr_err = e2m1 ? dispatch_tma<kValuesE2M1>(p, plan, st) : dispatch_tma<kValuesF32>(p, plan, st);
    }
    cudaError_t err = attr_err != cudaSuccess ? attr_err : cudaGetLastError();

    if (err == cudaSuccess && split) err = launch_fixup_kernel(p, plan, st);
    if (ws_owned) {
        cudaError_t ferr = cudaFreeAsync(ws, st);
        if (err == cudaSuccess) err = ferr;
    }
    if (err != cudaSuccess) {
        set_last_error("kernel launch failed: %s", cudaGetErrorString(err));
        return CSRSPMM_B200_ERR_CUDA;
    }
    return CSRSPMM_B200_OK;
}

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

// True when `ptr` is device memory of the current context (an operand the caller kept on the GPU).
bool on_device(const void* ptr)
{
    if (ptr == nullptr) return false;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
        cudaGetLastError();  // plain host memory on older drivers: not an error for us
        return false;
    }
    return attr.type == cudaMemoryTypeDevice;
}

// ---- host round trip in column panels -------------------------------------------------------
//
// C[:, panel] depends on B[:, panel] only, so a wide product whose operands start in host memory
// can be cut into column panels: while panel q is being multiplied, panel q+1 of B is still
// arriving and panel q-1 of C is already leaving, which keeps both directions of the host link
// busy at once.  Each output element is still one sequential sum, so the result equals the
// unsplit product bit for bit.  On the device a panel is stored contiguously (ld = its width).
constexpr int kMaxPanels = CSRSPMM_B200_MAX_PANELS;

// Column panels of a host round trip over Nd columns: `requested` > 0 asks for that many equal panels,
// else CSRSPMM_HOST_PANELS in the environment (1 = off), else the rule -- a B of 256 MiB and more
// with Nd >= 256 goes in panels of 128 columns (512-byte segments in the strided host copies; wider when
// that would make more than eight) between a first and a last panel of 64: the first panel's upload and the last panel's download overlap
// nothing, so they are the short ones, while 256-byte segments copy too slowly to use throughout
// (config 5 from host memory, one GPU, same box: 217.5 ms this way, 221.1 ms with four panels of 128,
// 240 ms with eight of 64).
// Widths are multiples of 32 columns except possibly the last.  Returns the count and fills
// first[]/width[] (kMaxPanels entries each) when they are given.
int column_panel_layout(int32_t Kd, int32_t Nd, int requested, int32_t* first, int32_t* width)
{
    int want = requested;
    if (want <= 0)
        if (const char* e = std::getenv("CSRSPMM_HOST_PANELS")) want = std::atoi(e);
    if (want <= 0) {
        const size_t b_bytes = (size_t)Kd * (size_t)Nd * 4;
        if (b_bytes >= ((size_t)256 << 20) && Nd >= 256) {
            int mid = 128;  // at most eight panels between the first and the last
            if ((Nd - 128 + mid - 1) / mid > 8) mid = ((Nd - 128 + 7) / 8 + 31) / 32 * 32;
            int count = 0, c0 = 0;
            auto put = [&](int w) {
                if (first) first[count] = c0;
                if (width) width[count] = w;
                c0 += w;
                ++count;
            };
            put(64);
            while (Nd - c0 > mid + 64) put(mid);
            const int rest = Nd - c0;  // 65 .. mid + 64 columns: all but the last 64 in one panel
            if (rest > 64) put((rest - 64 + 31) / 32 * 32 < rest ? (rest - 64 + 31) / 32 * 32 : rest);
            if (Nd - c0 > 0) put(Nd - c0);
            return count;
        }
        want = 1;
    }
    if (want > kMaxPanels) want = kMaxPanels;
    if (want > Nd / 32) want = Nd / 32;  // never narrower than 32 columns
    if (want < 1) want = 1;
    const int pw = want > 1 ? ((Nd + want - 1) / want + 31) / 32 * 32 : (Nd > 0 ? Nd : 1);
    int count = 0;
    for (int c0 = 0; c0 < Nd || count == 0; c0 += pw) {
        if (first) first[count] = c0;
        if (width) width[count] = (Nd - c0 < pw) ? (Nd - c0 > 0 ? Nd - c0 : 0) : pw;
        ++count;
    }
    return count;
}

struct HostBuffers {
    int32_t* rp;
    int32_t* ci;
    char* va;
    float* B;
    float* C;
    void* ws;
    size_t ws_bytes;
    int32_t* status;
};

int spmm_host_panels(const csrspmm_b200_args* a, const HostBuffers& d, int panels, cudaStream_t st, int* word)
{
    int32_t first[kMaxPanels], width[kMaxPanels];
    panels = column_panel_layout(a->Kd, a->Nd, panels, first, width);

    cudaStream_t compute = nullptr, out = nullptr;
    cudaEvent_t up[kMaxPanels] = {}, done[kMaxPanels] = {};
    int n_up = 0, n_done = 0;
    auto cleanup = [&]() {
        for (int k = 0; k < n_up; ++k) cudaEventDestroy(up[k]);
        for (int k = 0; k < n_done; ++k) cudaEventDestroy(done[k]);
        if (compute) cudaStreamDestroy(compute);
        if (out) cudaStreamDestroy(out);
    };
#define CUDA_TRY_PANEL(expr)                                                                \
    do {                                                                                    \
        cudaError_t e__ = (expr);                                                           \
        if (e__ != cudaSuccess) {                                                           \
            set_last_error("%s failed: %s", #expr, cudaGetErrorString(e__));                \
            cudaDeviceSynchronize();                                                        \
            cleanup();                                                                      \
            return CSRSPMM_B200_ERR_CUDA;                                                   \
        }                                                                                   \
    } while (0)

    CUDA_TRY_PANEL(cudaStreamCreateWithFlags(&compute, cudaStreamNonBlocking));
    CUDA_TRY_PANEL(cudaStreamCreateWithFlags(&out, cudaStreamNonBlocking));
    for (; n_up < panels; ++n_up) CUDA_TRY_PANEL(cudaEventCreateWithFlags(&up[n_up], cudaEventDisableTiming));
    for (; n_done < panels; ++n_done) CUDA_TRY_PANEL(cudaEventCreateWithFlags(&done[n_done], cudaEventDisableTiming));

    for (int q = 0; q < panels; ++q) {
        const int c0 = first[q], w = width[q];
        float* dB = d.B + (size_t)a->Kd * (size_t)c0;
        float* dC = d.C + (size_t)a->M * (size_t)c0;
        if (a->beta != 0.0f)
            CUDA_TRY_PANEL(cudaMemcpy2DAsync(dC, (size_t)w * 4, a->C + c0, (size_t)a->ldc * 4, (size_t)w * 4,
                                             (size_t)a->M, cudaMemcpyHostToDevice, st));
        if (a->Kd > 0)
            CUDA_TRY_PANEL(cudaMemcpy2DAsync(dB, (size_t)w * 4, a->B + c0, (size_t)a->ldb * 4, (size_t)w * 4,
                                             (size_t)a->Kd, cudaMemcpyHostToDevice, st));
        CUDA_TRY_PANEL(cudaEventRecord(up[q], st));
        CUDA_TRY_PANEL(cudaStreamWaitEvent(compute, up[q], 0));

        csrspmm_b200_args pa = *a;
        pa.Nd = w;
        pa.row_ptr = d.rp;
        pa.col_idx = d.ci;
        pa.values = d.va;
        pa.B = dB;
        pa.ldb = w;
        pa.C = dC;
        pa.ldc = w;
        pa.workspace = d.ws;
        pa.workspace_bytes = d.ws_bytes;
        pa.status_word = d.status;
        const int status = enqueue(&pa, compute);
        if (status != CSRSPMM_B200_OK) {
            cudaDeviceSynchronize();
            cleanup();
            return status;
        }
        CUDA_TRY_PANEL(cudaEventRecord(done[q], compute));
        CUDA_TRY_PANEL(cudaStreamWaitEvent(out, done[q], 0));
        CUDA_TRY_PANEL(cudaMemcpy2DAsync(a->C + c0, (size_t)a->ldc * 4, dC, (size_t)w * 4, (size_t)w * 4, (size_t)a->M,
                                         cudaMemcpyDeviceToHost, out));
    }
    CUDA_TRY_PANEL(cudaMemcpyAsync(word, d.status, 4, cudaMemcpyDeviceToHost, compute));
    CUDA_TRY_PANEL(cudaStreamSynchronize(compute));
    CUDA_TRY_PANEL(cudaStreamSynchronize(out));
    CUDA_TRY_PANEL(cudaStreamSynchronize(st));
    cleanup();
    return CSRSPMM_B200_OK;
#undef CUDA_TRY_PANEL
}

}  // namespace

namespace csrspmm_b200 {

cudaError_t launch_row_kernel(const SpmmParams& p, const Plan& plan, bool e2m1, cudaStream_t st)
{
    if (plan.VW == 4) {
        if (e2m1) dispatch_row<4, kValuesE2M1>(p, plan, st);
        else dispatch_row<4, kValuesF32>(p, plan, st);
    } else {
        if (e2m1) dispatch_row<1, kValuesE2M1>(p, plan, st);
        else dispatch_row<1, kValuesF32>(p, plan, st);
    }
    return cudaGetLastError();
}

}  // namespace csrspmm_b200

extern "C" {

int csrspmm_b200_abi_version(void) { return CSRSPMM_B200_ABI_VERSION; }

const char* csrspmm_b200_status_string(int status)
{
    switch (status) {
        case CSRSPMM_B200_OK: return "ok";
        case CSRSPMM_B200_ERR_BAD_ARG: return "bad argument";
        case CSRSPMM_B200_ERR_INVALID_CSR: return "invalid CSR matrix";
        case CSRSPMM_B200_ERR_UNSUPPORTED: return "unsupported shape or layout for the requested kernel";
        case CSRSPMM_B200_ERR_CUDA: return "CUDA error";
        case CSRSPMM_B200_ERR_DEVICE_WAIT: return "device-side wait gave up";
        case CSRSPMM_B200_ERR_WORKSPACE: return "workspace too small or misaligned";
        case CSRSPMM_B200_ERR_NO_DEVICE: return "no usable device";
        default: return "unknown status";
    }
}

const char* csrspmm_b200_last_error(void) { return get_last_error(); }

int csrspmm_b200_spmm(const csrspmm_b200_args* args, csrspmm_b200_stream_t stream)
{
    return enqueue(args, reinterpret_cast<cudaStream_t>(stream));
}

int csrspmm_b200_spmm_sync(const csrspmm_b200_args* args, csrspmm_b200_stream_t stream)
{
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int status = enqueue(args, st);
    if (status != CSRSPMM_B200_OK) return status;
    CUDA_TRY(cudaStreamSynchronize(st));
    if (args->status_word != nullptr) {
        int word = 0;
        CUDA_TRY(cudaMemcpy(&word, args->status_word, sizeof(int), cudaMemcpyDeviceToHost));
        if (word & kStatusWaitTimeout) {
            set_last_error("device status word 0x%x: a bounded wait gave up", word);
            return CSRSPMM_B200_ERR_DEVICE_WAIT;
        }
        if (word & (kStatusBadTile | kStatusColClamped)) {
            set_last_error("device status word 0x%x: malformed CSR (row_ptr or col_idx)", word);
            return CSRSPMM_B200_ERR_INVALID_CSR;
        }
    }
    return CSRSPMM_B200_OK;
}

size_t csrspmm_b200_workspace_bytes(const csrspmm_b200_args* args)
{
    if (args != nullptr && args->struct_size == sizeof(csrspmm_b200_args) && schedule_applies(args))
        return scheduled_workspace_bytes(args);
    return worst_case_workspace(args);
}

int csrspmm_b200_select_kernel(const csrspmm_b200_args* args)
{
    Plan plan;
    int status = make_plan(args, &plan);
    if (status != CSRSPMM_B200_OK) return -status;
    if (schedule_applies(args)) return CSRSPMM_B200_KERNEL_SCHEDULED;
    return plan.kernel;
}

size_t csrspmm_b200_host_arena_bytes(const csrspmm_b200_args* a)
{
    if (check_args(a, false) != CSRSPMM_B200_OK) return 0;
    const size_t vbytes = a->value_format == CSRSPMM_B200_VALUES_E2M1 ? (size_t)(a->nnz + 1) / 2
                                                                      : (size_t)a->nnz * 4;
    size_t total = 0;
    total += align256(((size_t)a->M + 1) * 4);
    total += align256((size_t)a->nnz * 4);
    total += align256(vbytes);
    total += align256((size_t)a->Kd * (size_t)a->Nd * 4);
    total += align256((size_t)a->M * (size_t)a->Nd * 4);
    total += align256(worst_case_workspace(a, true));  // row blocks share it
    total += 256;  // status word
    return total;
}

int csrspmm_b200_spmm_host(const csrspmm_b200_args* a, void* device_arena, size_t device_arena_bytes,
                           csrspmm_b200_stream_t stream)
{
    int status = check_args(a, true);
    if (status != CSRSPMM_B200_OK) return status;
    if (a->M == 0 || a->Nd == 0) return CSRSPMM_B200_OK;
    if (a->row_ptr_base != 0) {
        set_last_error("spmm_host: row_ptr_base must be 0 (pass the whole matrix)");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const size_t need = csrspmm_b200_host_arena_bytes(a);
    char* arena = static_cast<char*>(device_arena);
    bool owned = false;
    if (arena == nullptr) {
        CUDA_TRY(cudaMallocAsync(reinterpret_cast<void**>(&arena), need, st));
        owned = true;
    } else if (device_arena_bytes < need || (reinterpret_cast<uintptr_t>(arena) & 255u) != 0) {
        set_last_error("device arena of %zu bytes: need %zu bytes, 256-byte aligned",
                       device_arena_bytes, need);
        return CSRSPMM_B200_ERR_WORKSPACE;
    }

    const bool e2m1 = a->value_format == CSRSPMM_B200_VALUES_E2M1;
    const size_t vbytes = e2m1 ? (size_t)(a->nnz + 1) / 2 : (size_t)a->nnz * 4;
    const size_t rp_bytes = ((size_t)a->M + 1) * 4, ci_bytes = (size_t)a->nnz * 4;
    const size_t c_bytes = (size_t)a->M * (size_t)a->Nd * 4;
    const size_t ws_bytes = worst_case_workspace(a, true);  // enough for every row block below
    char* cur = arena;
    int32_t* d_rp = reinterpret_cast<int32_t*>(cur); cur += align256(rp_bytes);
    int32_t* d_ci = reinterpret_cast<int32_t*>(cur); cur += align256(ci_bytes);
    char* d_va = cur; cur += align256(vbytes);
    float* d_B = reinterpret_cast<float*>(cur); cur += align256((size_t)a->Kd * (size_t)a->Nd * 4);
    float* d_C = reinterpret_cast<float*>(cur); cur += align256(c_bytes);
    void* d_ws = cur; cur += align256(ws_bytes);
    int32_t* d_status = reinterpret_cast<int32_t*>(cur);

    // A may already be on the device (kept there by the caller between products on one matrix, where
    // only B changes): each of its three arrays that is device memory is used in place, not copied.
    const bool rp_dev = on_device(a->row_ptr), ci_dev = on_device(a->col_idx), va_dev = on_device(a->values);
    if (rp_dev) d_rp = const_cast<int32_t*>(a->row_ptr);
    if (ci_dev) d_ci = const_cast<int32_t*>(a->col_idx);
    if (va_dev) d_va = const_cast<char*>(static_cast<const char*>(a->values));

    const int panels = column_panel_layout(a->Kd, a->Nd, 0, nullptr, nullptr);
    if (panels > 1) {
        // A first, on the caller's stream; the panels of B follow it on the same stream
        int word = 0;
        cudaError_t e = cudaMemsetAsync(d_status, 0, 4, st);
        if (e == cudaSuccess && !rp_dev) e = cudaMemcpyAsync(d_rp, a->row_ptr, rp_bytes, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess && a->nnz > 0 && !ci_dev) e = cudaMemcpyAsync(d_ci, a->col_idx, ci_bytes, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess && a->nnz > 0 && !va_dev) e = cudaMemcpyAsync(d_va, a->values, vbytes, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) {
            set_last_error("spmm_host: upload of A failed: %s", cudaGetErrorString(e));
            status = CSRSPMM_B200_ERR_CUDA;
        } else {
            const HostBuffers hb = {d_rp, d_ci, d_va, d_B, d_C, d_ws, align256(ws_bytes), d_status};
            status = spmm_host_panels(a, hb, panels, st, &word);
        }
        if (owned) {
            cudaFreeAsync(arena, st);
            cudaStreamSynchronize(st);
        }
        if (status != CSRSPMM_B200_OK) return status;
        if (word & kStatusWaitTimeout) {
            set_last_error("device status word 0x%x: a bounded wait gave up", word);
            return CSRSPMM_B200_ERR_DEVICE_WAIT;
        }
        if (word != 0) {
            set_last_error("device status word 0x%x: malformed CSR (row_ptr or col_idx)", word);
            return CSRSPMM_B200_ERR_INVALID_CSR;
        }
        return CSRSPMM_B200_OK;
    }

    // C goes back in row blocks on a second stream while the next block is being computed, so
    // the device->host copy of a large C hides the kernel time (and vice versa).
    constexpr int kMaxBlocks = 8;
    int blocks = (c_bytes >= ((size_t)64 << 20) && a->M >= 64) ? kMaxBlocks : 1;
    int32_t bounds[kMaxBlocks + 1] = {0};
    bounds[1] = a->M;
    // the row blocks are cut on the host: a row_ptr that lives on the device is read back once (4 bytes per row)
    const int32_t* h_rp = a->row_ptr;
    int32_t* h_rp_copy = nullptr;
    if (blocks > 1 && rp_dev) {
        h_rp_copy = static_cast<int32_t*>(std::malloc(rp_bytes));
        if (h_rp_copy == nullptr || cudaMemcpy(h_rp_copy, a->row_ptr, rp_bytes, cudaMemcpyDeviceToHost) != cudaSuccess) {
            cudaGetLastError();
            blocks = 1;
        }
        h_rp = h_rp_copy;
    }
    if (blocks > 1 && csrspmm_b200_partition_rows(a->M, h_rp, blocks, 1.0, bounds) != CSRSPMM_B200_OK) blocks = 1;
    if (blocks > 1 && e2m1)  // packed values can only be offset by whole bytes
        for (int k = 1; k < blocks; ++k)
            if (h_rp[bounds[k]] & 1) blocks = 1;
    if (blocks == 1) bounds[1] = a->M;

    cudaStream_t copy_stream = nullptr;
    cudaEvent_t done[kMaxBlocks] = {};
    int events = 0;
    auto cleanup = [&]() {
        // also the way out of every failure below: nothing may still be copying into or out of the
        // arena, or into this frame's `word`, when they go away (errors of these waits are ignored)
        cudaStreamSynchronize(st);
        if (copy_stream) cudaStreamSynchronize(copy_stream);
        std::free(h_rp_copy);
        h_rp_copy = nullptr;
        for (int k = 0; k < events; ++k) cudaEventDestroy(done[k]);
        if (copy_stream) cudaStreamDestroy(copy_stream);
        if (owned) cudaFreeAsync(arena, st);
    };
#define CUDA_TRY_HOST(expr)                                                                 \
    do {                                                                                    \
        cudaError_t e__ = (expr);                                                           \
        if (e__ != cudaSuccess) {                                                           \
            set_last_error("%s failed: %s", #expr, cudaGetErrorString(e__));                \
            cleanup();                                                                      \
            return CSRSPMM_B200_ERR_CUDA;                                                   \
        }                                                                                   \
    } while (0)

    if (blocks > 1) {
        CUDA_TRY_HOST(cudaStreamCreateWithFlags(&copy_stream, cudaStreamNonBlocking));
        for (; events < blocks; ++events) CUDA_TRY_HOST(cudaEventCreateWithFlags(&done[events], cudaEventDisableTiming));
    }
    CUDA_TRY_HOST(cudaMemsetAsync(d_status, 0, 4, st));
    if (!rp_dev) CUDA_TRY_HOST(cudaMemcpyAsync(d_rp, a->row_ptr, rp_bytes, cudaMemcpyHostToDevice, st));
    if (a->nnz > 0) {
        if (!ci_dev) CUDA_TRY_HOST(cudaMemcpyAsync(d_ci, a->col_idx, ci_bytes, cudaMemcpyHostToDevice, st));
        if (!va_dev) CUDA_TRY_HOST(cudaMemcpyAsync(d_va, a->values, vbytes, cudaMemcpyHostToDevice, st));
    }
    if (a->Kd > 0) {
        // B rows are packed on the device (ldb = Nd) whatever the host stride is
        CUDA_TRY_HOST(cudaMemcpy2DAsync(d_B, (size_t)a->Nd * 4, a->B, (size_t)a->ldb * 4,
                                        (size_t)a->Nd * 4, (size_t)a->Kd, cudaMemcpyHostToDevice, st));
    }
    if (a->beta != 0.0f) {
        CUDA_TRY_HOST(cudaMemcpy2DAsync(d_C, (size_t)a->Nd * 4, a->C, (size_t)a->ldc * 4,
                                        (size_t)a->Nd * 4, (size_t)a->M, cudaMemcpyHostToDevice, st));
    }
    for (int k = 0; k < blocks; ++k) {
        const int32_t r0 = bounds[k], r1 = bounds[k + 1];
        if (r1 <= r0) continue;
        // (one block: the whole matrix, and row_ptr may be device memory that the host cannot read)
        const int32_t j0 = blocks > 1 ? h_rp[r0] : 0, j1 = blocks > 1 ? h_rp[r1] : (int32_t)a->nnz;
        csrspmm_b200_args d = *a;
        d.M = r1 - r0;
        d.nnz = (int64_t)j1 - j0;
        d.row_ptr = d_rp + r0;
        d.row_ptr_base = j0;
        d.col_idx = d_ci + j0;
        d.values = e2m1 ? static_cast<const void*>(d_va + j0 / 2) : static_cast<const void*>(d_va + (size_t)j0 * 4);
        d.B = d_B;
        d.ldb = a->Nd;
        d.C = d_C + (size_t)r0 * (size_t)a->Nd;
        d.ldc = a->Nd;
        d.workspace = d_ws;
        d.workspace_bytes = align256(ws_bytes);
        d.status_word = d_status;
        status = enqueue(&d, st);
        if (status != CSRSPMM_B200_OK) {
            cleanup();
            return status;
        }
        cudaStream_t out_stream = st;
        if (blocks > 1) {
            CUDA_TRY_HOST(cudaEventRecord(done[k], st));
            CUDA_TRY_HOST(cudaStreamWaitEvent(copy_stream, done[k], 0));
            out_stream = copy_stream;
        }
        CUDA_TRY_HOST(cudaMemcpy2DAsync(a->C + (size_t)r0 * (size_t)a->ldc, (size_t)a->ldc * 4, d.C, (size_t)a->Nd * 4,
                                        (size_t)a->Nd * 4, (size_t)(r1 - r0), cudaMemcpyDeviceToHost, out_stream));
    }
    int word = 0;
    CUDA_TRY_HOST(cudaMemcpyAsync(&word, d_status, 4, cudaMemcpyDeviceToHost, st));
    CUDA_TRY_HOST(cudaStreamSynchronize(st));
    if (copy_stream) CUDA_TRY_HOST(cudaStreamSynchronize(copy_stream));
    cleanup();
    if (owned) CUDA_TRY(cudaStreamSynchronize(st));
    if (word & kStatusWaitTimeout) {
        set_last_error("device status word 0x%x: a bounded wait gave up", word);
        return CSRSPMM_B200_ERR_DEVICE_WAIT;
    }
    if (word != 0) {
        set_last_error("device status word 0x%x: malformed CSR (row_ptr or col_idx)", word);
        return CSRSPMM_B200_ERR_INVALID_CSR;
    }
    return CSRSPMM_B200_OK;
#undef CUDA_TRY_HOST
}

int csrspmm_b200_column_panels(int32_t Kd, int32_t Nd, int requested, int32_t* first_col, int32_t* width)
{
    if (Kd < 0 || Nd < 0) return 0;
    return column_panel_layout(Kd, Nd, requested, first_col, width);
}

int csrspmm_b200_copy_rows(void* dst, size_t dst_pitch_bytes, const void* src, size_t src_pitch_bytes,
                           size_t width_bytes, size_t rows, int to_host, csrspmm_b200_stream_t stream)
{
    if (width_bytes == 0 || rows == 0) return CSRSPMM_B200_OK;
    if (dst == nullptr || src == nullptr || dst_pitch_bytes < width_bytes || src_pitch_bytes < width_bytes) {
        set_last_error("copy_rows: null pointer or pitch smaller than the row width");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    CUDA_TRY(cudaMemcpy2DAsync(dst, dst_pitch_bytes, src, src_pitch_bytes, width_bytes, rows,
                               to_host ? cudaMemcpyDeviceToHost : cudaMemcpyHostToDevice,
                               reinterpret_cast<cudaStream_t>(stream)));
    return CSRSPMM_B200_OK;
}

int csrspmm_b200_validate_csr_device(int32_t M, int32_t Kd, int64_t nnz, const int32_t* row_ptr,
                                     const int32_t* col_idx, uint32_t* problems,
                                     csrspmm_b200_stream_t stream)
{
    if (M < 0 || Kd < 0 || nnz < 0 || row_ptr == nullptr || (nnz > 0 && col_idx == nullptr) ||
        problems == nullptr) {
        set_last_error("validate_csr_device: bad argument");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    unsigned* d_flags = nullptr;
    CUDA_TRY(cudaMallocAsync(reinterpret_cast<void**>(&d_flags), sizeof(unsigned), st));
    CUDA_TRY(cudaMemsetAsync(d_flags, 0, sizeof(unsigned), st));
    const int threads = 256;
    long long blocks = ((long long)M + threads - 1) / threads;
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 32) blocks = 148 * 32;
    validate_csr_kernel<<<(unsigned)blocks, threads, 0, st>>>(M, Kd, nnz, row_ptr, col_idx, d_flags);
    CUDA_TRY(cudaGetLastError());
    unsigned flags = 0;
    CUDA_TRY(cudaMemcpyAsync(&flags, d_flags, sizeof(unsigned), cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaFreeAsync(d_flags, st));
    CUDA_TRY(cudaStreamSynchronize(st));
    *problems = flags;
    if (flags & 15u) {
        set_last_error("CSR validation failed, problem bits 0x%x", flags);
        return CSRSPMM_B200_ERR_INVALID_CSR;
    }
    return CSRSPMM_B200_OK;
}

int csrspmm_b200_row_stats_device(int32_t M, const int32_t* row_ptr, int64_t stats[4],
                                  csrspmm_b200_stream_t stream)
{
    if (M < 0 || row_ptr == nullptr || stats == nullptr) {
        set_last_error("row_stats_device: bad argument");
        return CSRSPMM_B200_ERR_BAD_ARG;
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int first = 0, last = 0;
    CUDA_TRY(cudaMemcpyAsync(&first, row_ptr, 4, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaMemcpyAsync(&last, row_ptr + M, 4, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaStreamSynchronize(st));
    const long long nnz = (long long)last - first;
    const long long mean = M > 0 ? nnz / M : 0;
    unsigned long long* d_stats = nullptr;
    CUDA_TRY(cudaMallocAsync(reinterpret_cast<void**>(&d_stats), 4 * sizeof(unsigned long long), st));
    CUDA_TRY(cudaMemsetAsync(d_stats, 0, 4 * sizeof(unsigned long long), st));
    const int threads = 256;
    long long blocks = ((long long)M + threads - 1) / threads;
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 16) blocks = 148 * 16;
    row_stats_kernel<<<(unsigned)blocks, threads, 0, st>>>(M, row_ptr, 32 * (mean + 1), d_stats);
    CUDA_TRY(cudaGetLastError());
    unsigned long long h[4] = {0, 0, 0, 0};
    CUDA_TRY(cudaMemcpyAsync(h, d_stats, sizeof(h), cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaFreeAsync(d_stats, st));
    CUDA_TRY(cudaStreamSynchronize(st));
    for (int k = 0; k < 4; ++k) stats[k] = (int64_t)h[k];
    return CSRSPMM_B200_OK;
}

}  // extern "C"
