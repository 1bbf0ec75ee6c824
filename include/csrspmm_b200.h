/*
 * csrspmm_b200 -- C ABI of the sm_100a CSR x dense SpMM kernel library.
 *
 *     C[M x Nd] = alpha * A[M x Kd, CSR] * B[Kd x Nd] + beta * C        (fp32, int32 indices,
 *                                                                        row-major dense)
 *
 * This is the boundary the reference's host layer would bind instead of launching its own
 * src/device kernels.  Plain pointers and sizes only: no C++ types, no exceptions, no exit().
 * Every function returns a csrspmm_b200_status (0 = ok) unless stated otherwise.
 *
 * What each entry point stands in for in the reference (paths within the reference project):
 *   csrspmm_b200_spmm           the six launchers src/host/spmm_launcher.cu:11-171 and the
 *                               kernels they start (src/device/csrspmm_naive.cu:11-39,
 *                               csrspmm_naive_smem.cu:5-44, csrspmm_warp_per_row.cu:13-48,
 *                               csrspmm_warp_per_row_fp4.cu:9-65,
 *                               csrspmm_warp_per_row_smem.cu:11-62,
 *                               csrspmm_warp_per_row_smem_fp4.cu:11-84)
 *   csrspmm_b200_spmm_sync      csrspmm::spmm, src/csrspmm.cpp:28-75 (launch, then
 *                               cudaGetLastError + cudaDeviceSynchronize)
 *   csrspmm_b200_spmm_host      the host round trip the reference's callers spell out by hand:
 *                               csr_host2device / dense_host2device / spmm / dense_device2host
 *                               (tests/test_csrspmm.cu:80-92, benchmarks/bench_csrspmm.cu:84-91)
 *   csrspmm_b200_select_kernel  the (stub) auto-selection in src/csrspmm.cpp:34-40
 *   csrspmm_b200_dense2csr_count/_fill, _csr2dense   csrspmm::dense2csr / csr2dense,
 *                               src/host/csr_utils.cpp:70-145, on device-resident matrices
 *   csrspmm_b200_schedule_create/_destroy/_info   the per-matrix analysis the reference's spmm()
 *                               leaves as a stub (src/csrspmm.cpp:34-40: both branches pick Naive)
 *   validate / row_stats / partition_rows / e2m1_*   no counterpart in the reference
 */
#ifndef CSRSPMM_B200_H
#define CSRSPMM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CSRSPMM_B200_ABI_VERSION 2

/* Same handle type as cudaStream_t; NULL is the legacy default stream. */
typedef struct CUstream_st* csrspmm_b200_stream_t;

typedef enum csrspmm_b200_status {
    CSRSPMM_B200_OK = 0,
    CSRSPMM_B200_ERR_BAD_ARG = 1,      /* null pointer, negative size, bad enum, bad struct_size */
    CSRSPMM_B200_ERR_INVALID_CSR = 2,  /* validation found a malformed matrix */
    CSRSPMM_B200_ERR_UNSUPPORTED = 3,  /* a forced kernel cannot run this shape/alignment */
    CSRSPMM_B200_ERR_CUDA = 4,         /* a CUDA call failed; see csrspmm_b200_last_error */
    CSRSPMM_B200_ERR_DEVICE_WAIT = 5,  /* a bounded device-side wait gave up (status word set) */
    CSRSPMM_B200_ERR_WORKSPACE = 6,    /* caller's workspace is too small or misaligned */
    CSRSPMM_B200_ERR_NO_DEVICE = 7     /* no usable sm_100 device */
} csrspmm_b200_status;

/* Which of the reference's entry points the caller is serving (same order as
 * csrspmm::Algorithm, include/csrspmm/csrspmm.h:10-17).  Recorded for diagnostics; every value
 * computes the same C with the same automatically chosen kernel. */
typedef enum csrspmm_b200_entry {
    CSRSPMM_B200_ENTRY_NAIVE = 0,
    CSRSPMM_B200_ENTRY_NAIVE_SMEM = 1,
    CSRSPMM_B200_ENTRY_WARP_PER_ROW = 2,
    CSRSPMM_B200_ENTRY_WARP_PER_ROW_FP4 = 3,
    CSRSPMM_B200_ENTRY_WARP_PER_ROW_SMEM = 4,
    CSRSPMM_B200_ENTRY_WARP_PER_ROW_SMEM_FP4 = 5
} csrspmm_b200_entry;

typedef enum csrspmm_b200_kernel {
    CSRSPMM_B200_KERNEL_AUTO = 0,
    CSRSPMM_B200_KERNEL_ROW = 1,    /* lane group per row; sequential accumulation per output */
    CSRSPMM_B200_KERNEL_MERGE = 2,  /* merge-path split over (rows + nnz); carries + fix-up */
    CSRSPMM_B200_KERNEL_TMA = 3,    /* merge-path split, B rows staged through shared memory by
                                       bulk async copies (needs the 16-byte-aligned layout) */
    CSRSPMM_B200_KERNEL_SCHEDULED = 4 /* answer of csrspmm_b200_select_kernel only, never an input: the
                                       product will run under args.schedule (pieces, slot sums, merge-path
                                       kernel over the other rows) */
} csrspmm_b200_kernel;

typedef enum csrspmm_b200_value_format {
    CSRSPMM_B200_VALUES_F32 = 0,
    CSRSPMM_B200_VALUES_E2M1 = 1 /* two 4-bit codes per byte, element j in byte j/2 (even j = low
                                    nibble); value = magnitude(code) * value_scale */
} csrspmm_b200_value_format;

/* All pointers are DEVICE pointers (csrspmm_b200_spmm, _sync) or HOST pointers (_spmm_host). */
typedef struct csrspmm_b200_args {
    uint32_t struct_size; /* sizeof(csrspmm_b200_args), checked */
    int32_t M;            /* rows of A and C */
    int32_t Kd;           /* columns of A = rows of B */
    int32_t Nd;           /* columns of B and C */
    int64_t nnz;          /* stored non-zeros, < 2^31 */
    const int32_t* row_ptr; /* M + 1 */
    const int32_t* col_idx; /* nnz */
    const void* values;     /* nnz floats, or (nnz+1)/2 bytes for E2M1 */
    int32_t value_format;   /* csrspmm_b200_value_format */
    float value_scale;      /* E2M1 only */
    const float* B;
    int64_t ldb; /* elements between consecutive rows of B; the reference's layout is ldb == Nd */
    float* C;
    int64_t ldc;
    float alpha;
    float beta;         /* C is not read when beta == 0 */
    int32_t entry;      /* csrspmm_b200_entry */
    int32_t kernel;     /* csrspmm_b200_kernel; AUTO unless pinned */
    int32_t max_row_nnz; /* longest row if known, else 0 (a hint, never trusted for bounds) */
    int32_t row_ptr_base; /* subtracted from every row_ptr entry; 0 for a whole matrix.  To multiply
                             rows [r0, r1) of a larger matrix without re-basing its offsets pass
                             row_ptr + r0, col_idx + row_ptr[r0], values + row_ptr[r0] (F32 values),
                             M = r1 - r0, nnz = row_ptr[r1] - row_ptr[r0], row_ptr_base = row_ptr[r0] */
    void* workspace;        /* device scratch for the split kernels, or NULL: the library then
                               takes it from the stream-ordered allocator for this call */
    size_t workspace_bytes; /* size of workspace when it is not NULL */
    int32_t* status_word;   /* optional device int32 the kernels OR error bits into */
    const struct csrspmm_b200_schedule* schedule; /* optional: a schedule built for this matrix by
                               csrspmm_b200_schedule_create (device-pointer entry points only); NULL
                               multiplies without one */
} csrspmm_b200_args;

int csrspmm_b200_abi_version(void);
const char* csrspmm_b200_status_string(int status);
/* Text of the most recent failure on the calling thread ("" if none). */
const char* csrspmm_b200_last_error(void);

/* Asynchronous: enqueue the SpMM on `stream` and return.  Device pointers.  With CSRSPMM_VALIDATE=1
 * in the environment the CSR structure is first checked on the device (one extra kernel and a
 * stream synchronisation) and a malformed matrix is refused with ERR_INVALID_CSR. */
int csrspmm_b200_spmm(const csrspmm_b200_args* args, csrspmm_b200_stream_t stream);

/* As above, then wait for the stream and report launch/execution errors and the status word. */
int csrspmm_b200_spmm_sync(const csrspmm_b200_args* args, csrspmm_b200_stream_t stream);

/* Host pointers in `args` (workspace/status_word ignored).  Copies A and B (and C when
 * beta != 0) to the current device, runs the SpMM, copies C back and waits.  When
 * device_arena is NULL the device buffers are allocated and released inside the call; else
 * the arena (>= csrspmm_b200_host_arena_bytes(args) bytes, 256-byte aligned) is used.
 * row_ptr, col_idx and values may each be DEVICE memory instead (a matrix the caller keeps on the GPU
 * between products, where only B changes): such an array is used in place and not copied.
 * Copies and kernels overlap: a B of 256 MiB or more with Nd >= 256 is processed in column panels
 * of 128 columns between a first and a last panel of 64 (panel q+1 of B arrives and panel q-1 of C leaves while panel q is multiplied;
 * CSRSPMM_HOST_PANELS=<n> in the environment sets the number of panels, 1 = none); otherwise a
 * large C goes back in row blocks while the next block is computed.  Either way every element of
 * C is the same sequential sum as in one unsplit product. */
int csrspmm_b200_spmm_host(const csrspmm_b200_args* args, void* device_arena,
                           size_t device_arena_bytes, csrspmm_b200_stream_t stream);
size_t csrspmm_b200_host_arena_bytes(const csrspmm_b200_args* args);

/* No counterpart in the reference.  The column panels csrspmm_b200_spmm_host cuts a product of
 * these sizes into: returns their number (1 = unsplit, at most CSRSPMM_B200_MAX_PANELS) and, when
 * the arrays are given, each panel's first column and width.  requested > 0 asks for that many
 * panels instead of the rule; widths are multiples of 32 columns except possibly the last. */
#define CSRSPMM_B200_MAX_PANELS 16
int csrspmm_b200_column_panels(int32_t Kd, int32_t Nd, int requested, int32_t* first_col, int32_t* width);

/* No counterpart in the reference (its dense_host2device / dense_device2host,
 * src/host/dense_utils.cpp, copy whole packed matrices).  Asynchronous copy of `rows` rows of
 * `width_bytes` bytes between host and device, each side with its own pitch -- what a caller
 * needs to move one column panel of a row-major matrix.  to_host = 0: src is host memory, dst
 * device memory; to_host = 1: the other way.  Pinned host memory makes it truly asynchronous. */
int csrspmm_b200_copy_rows(void* dst, size_t dst_pitch_bytes, const void* src, size_t src_pitch_bytes,
                           size_t width_bytes, size_t rows, int to_host, csrspmm_b200_stream_t stream);

/* No counterpart in the reference.  The same product as csrspmm_b200_spmm for callers that cannot
 * obtain device memory at call time -- a process whose memory manager already owns the whole GPU,
 * a plug-in whose host forbids allocation calls, a loop that must never enter the allocator.  It
 * always runs the merge-path kernel and keeps that kernel's scratch in a fixed array inside the
 * library's device image (CSRSPMM_B200_NOALLOC_SCRATCH_BYTES per GPU, held until the process
 * ends), so it calls no allocation routine at all.  args.kernel / workspace / workspace_bytes /
 * schedule are ignored.  A problem whose scratch (an int32 and a row of Nd floats per CTA of the merge kernel, i.e. per 512..3072 of M + nnz)
 * does not fit is refused with ERR_WORKSPACE and nothing is launched.  Every call on a device
 * shares the one array: the previous call's contents are harmless (every slot that is read is
 * rewritten first by the same call), but two calls running on the GPU at the same time corrupt
 * each other -- do not overlap them.  The first call on each device looks up the array's device
 * address; make it before any stream capture on that device. */
#define CSRSPMM_B200_NOALLOC_SCRATCH_BYTES (8u << 20)
int csrspmm_b200_spmm_noalloc(const csrspmm_b200_args* args, csrspmm_b200_stream_t stream);

/* No counterpart in the reference (a locality pass for operands far larger than L2).  The same
 * product as csrspmm_b200_spmm, computed in passes over panels of `panel_rows` columns of A (= rows
 * of B), so that each slab of B is read from HBM once and then served from L2: pass t takes, for
 * every row, the stored entries from where pass t-1 stopped up to the first one whose column index
 * is not below (t+1)*panel_rows.  Each pass re-reads and re-writes the running sums of the rows
 * it touches; on B200 that cost has so far matched or exceeded the HBM traffic saved (level with
 * csrspmm_b200_spmm at best, on long even rows and a B of several times L2; slower elsewhere), so
 * AUTO never picks it and it stays an explicit choice.  Columns need not be sorted
 * (sorted columns give each pass exactly its panel).  Every output accumulates its products in
 * stored order, so the result is bit-identical to the whole-row kernel's.  Device pointers;
 * args.kernel is ignored; args.workspace (256-byte aligned, csrspmm_b200_tiled_workspace_bytes
 * bytes: one int32 per row, plus M x Nd floats when beta != 0) or NULL to let the call take it
 * from cudaMallocAsync.  panel_rows = 0 asks for the library's choice
 * (csrspmm_b200_tiled_panel_rows: a slab of 64 MiB; 0 when B is not larger than that, in which
 * case the call is a single whole-row pass). */
int32_t csrspmm_b200_tiled_panel_rows(const csrspmm_b200_args* args);
size_t csrspmm_b200_tiled_workspace_bytes(const csrspmm_b200_args* args);
int csrspmm_b200_spmm_tiled(const csrspmm_b200_args* args, int32_t panel_rows, csrspmm_b200_stream_t stream);

/* Scratch the split kernels need for this problem (0 for the row kernel).  Depends only on
 * sizes, never on matrix contents. */
size_t csrspmm_b200_workspace_bytes(const csrspmm_b200_args* args);

/* The kernel AUTO resolves to for these arguments (host-only logic, no CUDA call);
 * returns a csrspmm_b200_kernel, or a negative csrspmm_b200_status on bad arguments.
 * The environment variable CSRSPMM_FORCE_KERNEL=row|merge|tma overrides AUTO. */
int csrspmm_b200_select_kernel(const csrspmm_b200_args* args);

/* ---- per-matrix schedule ---------------------------------------------------------------------
 * Stands where the reference's spmm() has a stub that inspects nothing (src/csrspmm.cpp:34-40).
 * For a matrix whose B is several times larger than L2 the gather of B rows is what the product
 * costs, and rows long enough to hold several entries per L2-sized slab of B can take that gather
 * from L2 instead of HBM if their work is ordered by slab.  A schedule is that ordering, built once
 * per matrix from row_ptr and col_idx (never the values) on the device:
 *   - rows of `long_row_threshold` entries or more are "long"; the columns of every long row must
 *     be ascending (else the schedule is built empty and changes nothing);
 *   - each long row is cut at the slab boundaries (slabs of `slab_rows` columns of A = rows of B)
 *     and every cut piece again into pieces of at most `piece_nnz` entries; the pieces are listed
 *     slab by slab, so that CTAs resident together gather from the same slab of B;
 *   - a product with args.schedule set runs three kernels: the pieces (each one sequential fp32
 *     sum into its own slot of scratch), the per-row sum of the slots in stored order (no atomics:
 *     the result is the same on every run), and the merge-path kernel over the remaining rows.
 * Left to itself (no threshold in the options) the library schedules nothing -- the schedule comes back
 * empty and products run as without one -- when it would not pay: B fits one slab, rows of B under 1 KB
 * (there the short rows, not the bytes, set the time), or scheduled rows that together name each row of B
 * fewer than 1.5 times (no re-use to win; typical of a row block of a matrix cut across many GPUs).
 * The schedule holds device memory (csrspmm_b200_schedule_info.device_bytes) on the device that
 * was current at creation and must be used there.  It describes the sparsity pattern only: keep it
 * as long as row_ptr and col_idx are unchanged (values, B, C, alpha, beta and Nd may change; Nd
 * only moves the slab size away from the one planned).  A call whose M, Kd or nnz differ from the
 * schedule's is refused with ERR_BAD_ARG.  args.kernel must be AUTO or MERGE and args.row_ptr_base
 * 0; with AUTO the schedule is left aside when the rows are known to be even (args.max_row_nnz close to
 * the mean), where the whole-row kernel is the better choice.  Scratch: csrspmm_b200_workspace_bytes(args) with args.schedule set.  Thread-safe for
 * concurrent products as long as each has its own workspace. */
struct csrspmm_b200_schedule;
typedef struct csrspmm_b200_schedule csrspmm_b200_schedule;

typedef struct csrspmm_b200_schedule_options {
    uint32_t struct_size;       /* sizeof(csrspmm_b200_schedule_options) */
    int32_t long_row_threshold; /* rows of this many entries or more are scheduled; 0 = choose */
    int32_t slab_rows;          /* rows of B per slab; 0 = choose (about 32 MiB of B) */
    int32_t piece_nnz;          /* longest piece one lane group accumulates; 0 = choose, at most 512 */
} csrspmm_b200_schedule_options;

typedef struct csrspmm_b200_schedule_info {
    uint32_t struct_size; /* set by the caller: sizeof(csrspmm_b200_schedule_info) */
    int32_t M, Kd, Nd;
    int64_t nnz;
    int32_t long_row_threshold, slab_rows, num_slabs, piece_nnz;
    int32_t long_rows;     /* rows the schedule covers (0: an empty schedule, plain kernels run) */
    int64_t long_nnz;      /* their entries */
    int64_t pieces;        /* work items = scratch slots of Nd floats each */
    int32_t columns_sorted; /* 0 when a long row with unsorted columns emptied the schedule */
    size_t device_bytes;   /* device memory the schedule keeps */
    double build_ms;       /* wall time of csrspmm_b200_schedule_create */
} csrspmm_b200_schedule_info;

/* Device row_ptr / col_idx in args (values, B, C are not touched; Nd and ldb size the slabs).
 * options may be NULL.  Synchronous: returns when the schedule is complete.  The environment
 * variables CSRSPMM_SCHED_THRESHOLD, CSRSPMM_SCHED_SLAB_MIB and CSRSPMM_SCHED_PIECE override
 * zero fields of the options. */
int csrspmm_b200_schedule_create(const csrspmm_b200_args* args, const csrspmm_b200_schedule_options* options,
                                 csrspmm_b200_schedule** out, csrspmm_b200_stream_t stream);
int csrspmm_b200_schedule_destroy(csrspmm_b200_schedule* schedule);
int csrspmm_b200_schedule_info_get(const csrspmm_b200_schedule* schedule, csrspmm_b200_schedule_info* info);

/* ---- CSR validation (new; the reference validates nothing) ---------------------------------- */

#define CSRSPMM_B200_CSR_BAD_ROWPTR0 1u    /* row_ptr[0] != 0 */
#define CSRSPMM_B200_CSR_BAD_ROWPTR_END 2u /* row_ptr[M] != nnz */
#define CSRSPMM_B200_CSR_NOT_MONOTONE 4u   /* row_ptr[i+1] < row_ptr[i] */
#define CSRSPMM_B200_CSR_COL_RANGE 8u      /* col_idx[j] < 0 or >= Kd */
#define CSRSPMM_B200_CSR_COL_UNSORTED 16u  /* columns of a row not strictly ascending (allowed
                                              by the kernels; reported, not an error) */

/* Host arrays.  *problems receives the OR of the bits above.  Returns ERR_INVALID_CSR when any
 * of the first four bits is set. */
int csrspmm_b200_validate_csr_host(int32_t M, int32_t Kd, int64_t nnz, const int32_t* row_ptr,
                                   const int32_t* col_idx, uint32_t* problems);
/* Device arrays; runs a checking kernel on `stream` and waits for it. */
int csrspmm_b200_validate_csr_device(int32_t M, int32_t Kd, int64_t nnz, const int32_t* row_ptr,
                                     const int32_t* col_idx, uint32_t* problems,
                                     csrspmm_b200_stream_t stream);

/* Device row_ptr -> stats[0] = longest row, stats[1] = empty rows, stats[2] = rows longer than
 * 32 * (mean + 1), stats[3] = nnz held by those rows.  Waits for the stream. */
int csrspmm_b200_row_stats_device(int32_t M, const int32_t* row_ptr, int64_t stats[4],
                                  csrspmm_b200_stream_t stream);

/* ---- dense <-> CSR on the device --------------------------------------------------------------
 * Same results as the reference's host-only csrspmm::dense2csr / csr2dense
 * (src/host/csr_utils.cpp:70-145): entries with fabs(v) > tol are kept, columns ascending,
 * max_row_nnz = longest row; the way back zero-fills and scatters.  All pointers are device
 * pointers, `ld` is the leading dimension of the dense matrix in elements.
 * Two steps because the caller owns the buffers: _count fills row_ptr (H + 1 entries) and
 * returns nnz (it waits for the stream); the caller allocates col_idx / values; _fill writes
 * them (asynchronous). */
int csrspmm_b200_dense2csr_count(int32_t H, int32_t W, const float* dense, int64_t ld, float tol,
                                 int32_t* row_ptr, int64_t* nnz_out, int32_t* max_row_nnz_out,
                                 csrspmm_b200_stream_t stream);
int csrspmm_b200_dense2csr_fill(int32_t H, int32_t W, const float* dense, int64_t ld, float tol,
                                const int32_t* row_ptr, int32_t* col_idx, float* values,
                                csrspmm_b200_stream_t stream);
int csrspmm_b200_csr2dense(int32_t H, int32_t W, const int32_t* row_ptr, const int32_t* col_idx,
                           const float* values, float* dense, int64_t ld, csrspmm_b200_stream_t stream);

/* ---- multi-GPU row partition (new) ------------------------------------------------------------
 * Contiguous row blocks [bounds[g], bounds[g+1]) for g < parts with near-equal cost, where the
 * cost of a row is its nnz + row_weight (row_weight = 1 balances B-row reads against C-row
 * writes; 0 balances nnz alone).  Host row_ptr.  A row is never split. */
int csrspmm_b200_partition_rows(int32_t M, const int32_t* row_ptr, int32_t parts,
                                double row_weight, int32_t* bounds);

/* ---- e2m1 value codec (new; the reference's "Fp4" kernels take fp32 values) -------------------
 * Host buffers.  scale = max|v| / 6 (1 when all zero); encode rounds v/scale to the nearest of
 * {0, .5, 1, 1.5, 2, 3, 4, 6}, ties to the even code, saturating, sign kept. */
float csrspmm_b200_e2m1_scale(int64_t n, const float* values);
int csrspmm_b200_e2m1_encode(int64_t n, const float* values, float scale, uint8_t* packed);
int csrspmm_b200_e2m1_decode(int64_t n, const uint8_t* packed, float scale, float* values);
/* The same codec for arrays in device memory (same codes bit for bit).  _scale_device waits for the
 * stream and writes the scale to host memory; _encode_device and _decode_device are asynchronous. */
int csrspmm_b200_e2m1_scale_device(int64_t n, const float* values, float* scale_out, csrspmm_b200_stream_t stream);
int csrspmm_b200_e2m1_encode_device(int64_t n, const float* values, float scale, uint8_t* packed,
                                    csrspmm_b200_stream_t stream);
int csrspmm_b200_e2m1_decode_device(int64_t n, const uint8_t* packed, float scale, float* values,
                                    csrspmm_b200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* CSRSPMM_B200_H */
