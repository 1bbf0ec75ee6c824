// csrspmm_b200_spmm_noalloc: the merge-path SpMM with its scratch inside the library image.
//
// Who this is for.  csrspmm_b200_spmm needs a few bytes of device scratch per CTA for the split
// kernels; it takes them from the caller's workspace or, failing that, from cudaMallocAsync.  Some
// hosts of this library can do neither: a process whose own memory manager claimed the whole
// device at start-up (a later cudaMalloc or pool allocation fails, or comes back after a
// device-wide synchronisation it cannot afford), a plug-in called from inside somebody else's
// runtime that forbids allocation calls on its threads, or a control loop with a hard deadline
// per call that must never enter the allocator.  Such a caller already owns A, B and C; the only
// thing it cannot provide on the spot is the scratch.  This entry point therefore carries a fixed
// scratch array in the library's device image and calls no allocation routine of any kind.
//
// Limits and rules.
//   * The array is CSRSPMM_B200_NOALLOC_SCRATCH_BYTES (8 MiB) per device and exists on every GPU
//     that loads the library, until the process ends.  A problem that needs more (one int32 plus
//     one row of Nd floats per CTA of the merge kernel, i.e. per 512 to 3072 merge-path items) is
//     refused with ERR_WORKSPACE and a message that states both numbers; nothing is launched.
//   * It always runs the merge-path kernel (args.kernel, args.workspace, args.workspace_bytes and
//     args.schedule are ignored).
//   * All calls on one device share the one array.  It keeps whatever the previous call left, and
//     that is harmless: every slot the fix-up kernel reads (one carry row index per CTA, and the
//     carry values of the CTAs whose index is valid) is rewritten by the same call's main kernel
//     first, so nothing has to start at zero and nothing is cleared.  Two calls that run on the
//     GPU at the same time (different streams, or different host threads) would overwrite each
//     other's carries: callers must not let calls on the same device overlap.
//   * The first call on each device looks the array's device address up (cudaGetSymbolAddress,
//     with that device current) and caches it; make that first call before starting any stream
//     capture on that device.
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>

#include "csrspmm_b200.h"
#include "launch.h"
#include "plan.h"

using namespace csrspmm_b200;

namespace {

// Lives in device memory of every GPU this library is loaded on.  In host code this name is only
// a handle for cudaGetSymbolAddress, never an address a kernel could use.
static __device__ __align__(256) unsigned char g_noalloc_scratch[CSRSPMM_B200_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
void* g_scratch_address[kMaxDevices] = {};  // per device ordinal, filled on first use

int scratch_of_current_device(void** out)
{
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) {
        set_last_error("cudaGetDevice failed: %s", cudaGetErrorString(e));
        return CSRSPMM_B200_ERR_CUDA;
    }
    if (device < 0 || device >= kMaxDevices) {
        set_last_error("device ordinal %d outside the supported range [0, %d)", device, kMaxDevices);
        return CSRSPMM_B200_ERR_NO_DEVICE;
    }
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_address[device] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            set_last_error("cudaGetSymbolAddress(scratch) failed on device %d: %s", device,
                           cudaGetErrorString(e));
            return CSRSPMM_B200_ERR_CUDA;
        }
        g_scratch_address[device] = ptr;
    }
    *out = g_scratch_address[device];
    return CSRSPMM_B200_OK;
}

}  // namespace

extern "C" int csrspmm_b200_spmm_noalloc(const csrspmm_b200_args* args, csrspmm_b200_stream_t stream)
{
    int status = check_args(args, true);
    if (status != CSRSPMM_B200_OK) return status;
    if (args->M == 0 || args->Nd == 0) return CSRSPMM_B200_OK;

    csrspmm_b200_args a = *args;
    a.kernel = CSRSPMM_B200_KERNEL_MERGE;
    a.workspace = nullptr;
    a.workspace_bytes = 0;
    a.schedule = nullptr;  // a schedule's scratch would not fit the fixed array's contract
    Plan plan;
    status = make_plan(&a, &plan);
    if (status != CSRSPMM_B200_OK) return status;
    if (plan.workspace_bytes > (size_t)CSRSPMM_B200_NOALLOC_SCRATCH_BYTES) {
        set_last_error("csrspmm_b200_spmm_noalloc: this problem (M + nnz = %lld, Nd = %d) needs %zu bytes of "
                       "scratch but the built-in array holds %zu; use csrspmm_b200_spmm with a workspace",
                       plan.num_items, a.Nd, plan.workspace_bytes, (size_t)CSRSPMM_B200_NOALLOC_SCRATCH_BYTES);
        return CSRSPMM_B200_ERR_WORKSPACE;
    }
    void* scratch = nullptr;
    status = scratch_of_current_device(&scratch);
    if (status != CSRSPMM_B200_OK) return status;

    // same parameter block, same kernel dispatch and same fix-up as csrspmm_b200_spmm's merge path
    SpmmParams p;
    fill_params(&a, plan, &p);
    set_carry_scratch(plan, scratch, &p);

    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    cudaError_t err = launch_merge_kernel(p, plan, a.value_format == CSRSPMM_B200_VALUES_E2M1, st);
    if (err == cudaSuccess) err = launch_fixup_kernel(p, plan, st);
    if (err != cudaSuccess) {
        set_last_error("csrspmm_b200_spmm_noalloc: kernel launch failed: %s", cudaGetErrorString(err));
        return CSRSPMM_B200_ERR_CUDA;
    }
    return CSRSPMM_B200_OK;
}
