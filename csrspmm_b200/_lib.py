"""ctypes binding of libcsrspmm_b200.so (the C ABI declared in include/csrspmm_b200.h).

The library is mandatory: there is no Python or CPU fallback for any compute entry point.
Loading fails loudly when the shared object has not been built.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

PKG = Path(__file__).resolve().parent
# CSRSPMM_B200_LIBRARY points at another build of the same library (kernel tuning experiments)
LIB_PATH = Path(os.environ.get("CSRSPMM_B200_LIBRARY") or PKG / "lib" / "libcsrspmm_b200.so")

ABI_VERSION = 2
OK = 0
ERR_BAD_ARG, ERR_INVALID_CSR, ERR_UNSUPPORTED, ERR_CUDA, ERR_DEVICE_WAIT, ERR_WORKSPACE, ERR_NO_DEVICE = range(1, 8)

ENTRY_NAIVE, ENTRY_NAIVE_SMEM, ENTRY_WARP_PER_ROW, ENTRY_WARP_PER_ROW_FP4, ENTRY_WARP_PER_ROW_SMEM, \
    ENTRY_WARP_PER_ROW_SMEM_FP4 = range(6)
KERNEL_AUTO, KERNEL_ROW, KERNEL_MERGE, KERNEL_TMA, KERNEL_SCHEDULED = range(5)
KERNEL_NAMES = {KERNEL_AUTO: "auto", KERNEL_ROW: "row", KERNEL_MERGE: "merge", KERNEL_TMA: "tma", KERNEL_SCHEDULED: "scheduled"}
KERNEL_IDS = {v: k for k, v in KERNEL_NAMES.items() if k != KERNEL_SCHEDULED}  # "scheduled" is an answer, never an input
VALUES_F32, VALUES_E2M1 = 0, 1
NOALLOC_SCRATCH_BYTES = 8 << 20

CSR_BAD_ROWPTR0, CSR_BAD_ROWPTR_END, CSR_NOT_MONOTONE, CSR_COL_RANGE, CSR_COL_UNSORTED = 1, 2, 4, 8, 16

# every symbol include/csrspmm_b200.h declares
EXPORTED_SYMBOLS = (
    "csrspmm_b200_abi_version", "csrspmm_b200_status_string", "csrspmm_b200_last_error",
    "csrspmm_b200_spmm", "csrspmm_b200_spmm_sync", "csrspmm_b200_spmm_host", "csrspmm_b200_spmm_noalloc",
    "csrspmm_b200_host_arena_bytes", "csrspmm_b200_workspace_bytes", "csrspmm_b200_select_kernel",
    "csrspmm_b200_validate_csr_host", "csrspmm_b200_validate_csr_device",
    "csrspmm_b200_row_stats_device", "csrspmm_b200_partition_rows", "csrspmm_b200_e2m1_scale",
    "csrspmm_b200_e2m1_encode", "csrspmm_b200_e2m1_decode", "csrspmm_b200_dense2csr_count",
    "csrspmm_b200_dense2csr_fill", "csrspmm_b200_csr2dense", "csrspmm_b200_copy_rows", "csrspmm_b200_column_panels",
    "csrspmm_b200_e2m1_scale_device", "csrspmm_b200_e2m1_encode_device", "csrspmm_b200_e2m1_decode_device",
    "csrspmm_b200_spmm_tiled", "csrspmm_b200_tiled_workspace_bytes", "csrspmm_b200_tiled_panel_rows",
    "csrspmm_b200_schedule_create", "csrspmm_b200_schedule_destroy", "csrspmm_b200_schedule_info_get",
)


class Args(C.Structure):
    """Mirror of ``csrspmm_b200_args``."""
    _fields_ = [
        ("struct_size", C.c_uint32),
        ("M", C.c_int32),
        ("Kd", C.c_int32),
        ("Nd", C.c_int32),
        ("nnz", C.c_int64),
        ("row_ptr", C.c_void_p),
        ("col_idx", C.c_void_p),
        ("values", C.c_void_p),
        ("value_format", C.c_int32),
        ("value_scale", C.c_float),
        ("B", C.c_void_p),
        ("ldb", C.c_int64),
        ("C", C.c_void_p),
        ("ldc", C.c_int64),
        ("alpha", C.c_float),
        ("beta", C.c_float),
        ("entry", C.c_int32),
        ("kernel", C.c_int32),
        ("max_row_nnz", C.c_int32),
        ("row_ptr_base", C.c_int32),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("status_word", C.c_void_p),
        ("schedule", C.c_void_p),
    ]


class ScheduleOptions(C.Structure):
    """Mirror of ``csrspmm_b200_schedule_options``."""
    _fields_ = [("struct_size", C.c_uint32), ("long_row_threshold", C.c_int32), ("slab_rows", C.c_int32),
                ("piece_nnz", C.c_int32)]


class ScheduleInfo(C.Structure):
    """Mirror of ``csrspmm_b200_schedule_info``."""
    _fields_ = [("struct_size", C.c_uint32), ("M", C.c_int32), ("Kd", C.c_int32), ("Nd", C.c_int32),
                ("nnz", C.c_int64), ("long_row_threshold", C.c_int32), ("slab_rows", C.c_int32),
                ("num_slabs", C.c_int32), ("piece_nnz", C.c_int32), ("long_rows", C.c_int32),
                ("long_nnz", C.c_int64), ("pieces", C.c_int64), ("columns_sorted", C.c_int32),
                ("device_bytes", C.c_size_t), ("build_ms", C.c_double)]


class LibraryMissing(RuntimeError):
    pass


class SpmmError(RuntimeError):
    def __init__(self, status: int, where: str):
        L = lib()
        msg = L.csrspmm_b200_status_string(status).decode()
        detail = L.csrspmm_b200_last_error().decode()
        super().__init__(f"{where}: {msg} (status {status}): {detail}")
        self.status = status


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise LibraryMissing(
            f"{LIB_PATH} is missing: build it with `python -m csrspmm_b200.build` "
            "(there is no fallback path)")
    L = C.CDLL(str(LIB_PATH))
    L.csrspmm_b200_abi_version.restype = C.c_int
    L.csrspmm_b200_status_string.argtypes = [C.c_int]
    L.csrspmm_b200_status_string.restype = C.c_char_p
    L.csrspmm_b200_last_error.restype = C.c_char_p
    for name in ("csrspmm_b200_spmm", "csrspmm_b200_spmm_sync", "csrspmm_b200_spmm_noalloc"):
        fn = getattr(L, name)
        fn.argtypes = [C.POINTER(Args), C.c_void_p]
        fn.restype = C.c_int
    L.csrspmm_b200_spmm_host.argtypes = [C.POINTER(Args), C.c_void_p, C.c_size_t, C.c_void_p]
    L.csrspmm_b200_spmm_host.restype = C.c_int
    L.csrspmm_b200_e2m1_scale_device.argtypes = [C.c_int64, C.c_void_p, C.POINTER(C.c_float), C.c_void_p]
    L.csrspmm_b200_e2m1_scale_device.restype = C.c_int
    L.csrspmm_b200_e2m1_encode_device.argtypes = [C.c_int64, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p]
    L.csrspmm_b200_e2m1_encode_device.restype = C.c_int
    L.csrspmm_b200_e2m1_decode_device.argtypes = [C.c_int64, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p]
    L.csrspmm_b200_e2m1_decode_device.restype = C.c_int
    L.csrspmm_b200_spmm_tiled.argtypes = [C.POINTER(Args), C.c_int32, C.c_void_p]
    L.csrspmm_b200_spmm_tiled.restype = C.c_int
    L.csrspmm_b200_tiled_workspace_bytes.argtypes = [C.POINTER(Args)]
    L.csrspmm_b200_tiled_workspace_bytes.restype = C.c_size_t
    L.csrspmm_b200_tiled_panel_rows.argtypes = [C.POINTER(Args)]
    L.csrspmm_b200_tiled_panel_rows.restype = C.c_int32
    L.csrspmm_b200_column_panels.argtypes = [C.c_int32, C.c_int32, C.c_int, C.c_void_p, C.c_void_p]
    L.csrspmm_b200_column_panels.restype = C.c_int
    L.csrspmm_b200_copy_rows.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                         C.c_int, C.c_void_p]
    L.csrspmm_b200_copy_rows.restype = C.c_int
    L.csrspmm_b200_host_arena_bytes.argtypes = [C.POINTER(Args)]
    L.csrspmm_b200_host_arena_bytes.restype = C.c_size_t
    L.csrspmm_b200_workspace_bytes.argtypes = [C.POINTER(Args)]
    L.csrspmm_b200_workspace_bytes.restype = C.c_size_t
    L.csrspmm_b200_select_kernel.argtypes = [C.POINTER(Args)]
    L.csrspmm_b200_select_kernel.restype = C.c_int
    L.csrspmm_b200_validate_csr_host.argtypes = [C.c_int32, C.c_int32, C.c_int64, C.c_void_p, C.c_void_p,
                                                 C.POINTER(C.c_uint32)]
    L.csrspmm_b200_validate_csr_host.restype = C.c_int
    L.csrspmm_b200_validate_csr_device.argtypes = [C.c_int32, C.c_int32, C.c_int64, C.c_void_p, C.c_void_p,
                                                   C.POINTER(C.c_uint32), C.c_void_p]
    L.csrspmm_b200_validate_csr_device.restype = C.c_int
    L.csrspmm_b200_row_stats_device.argtypes = [C.c_int32, C.c_void_p, C.POINTER(C.c_int64), C.c_void_p]
    L.csrspmm_b200_row_stats_device.restype = C.c_int
    L.csrspmm_b200_partition_rows.argtypes = [C.c_int32, C.c_void_p, C.c_int32, C.c_double, C.c_void_p]
    L.csrspmm_b200_partition_rows.restype = C.c_int
    L.csrspmm_b200_e2m1_scale.argtypes = [C.c_int64, C.c_void_p]
    L.csrspmm_b200_e2m1_scale.restype = C.c_float
    L.csrspmm_b200_e2m1_encode.argtypes = [C.c_int64, C.c_void_p, C.c_float, C.c_void_p]
    L.csrspmm_b200_e2m1_encode.restype = C.c_int
    L.csrspmm_b200_e2m1_decode.argtypes = [C.c_int64, C.c_void_p, C.c_float, C.c_void_p]
    L.csrspmm_b200_e2m1_decode.restype = C.c_int
    L.csrspmm_b200_dense2csr_count.argtypes = [C.c_int32, C.c_int32, C.c_void_p, C.c_int64, C.c_float, C.c_void_p,
                                               C.POINTER(C.c_int64), C.POINTER(C.c_int32), C.c_void_p]
    L.csrspmm_b200_dense2csr_count.restype = C.c_int
    L.csrspmm_b200_dense2csr_fill.argtypes = [C.c_int32, C.c_int32, C.c_void_p, C.c_int64, C.c_float, C.c_void_p,
                                              C.c_void_p, C.c_void_p, C.c_void_p]
    L.csrspmm_b200_dense2csr_fill.restype = C.c_int
    L.csrspmm_b200_csr2dense.argtypes = [C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                         C.c_void_p]
    L.csrspmm_b200_csr2dense.restype = C.c_int
    L.csrspmm_b200_schedule_create.argtypes = [C.POINTER(Args), C.POINTER(ScheduleOptions), C.POINTER(C.c_void_p),
                                               C.c_void_p]
    L.csrspmm_b200_schedule_create.restype = C.c_int
    L.csrspmm_b200_schedule_destroy.argtypes = [C.c_void_p]
    L.csrspmm_b200_schedule_destroy.restype = C.c_int
    L.csrspmm_b200_schedule_info_get.argtypes = [C.c_void_p, C.POINTER(ScheduleInfo)]
    L.csrspmm_b200_schedule_info_get.restype = C.c_int
    if L.csrspmm_b200_abi_version() != ABI_VERSION:
        raise LibraryMissing(f"{LIB_PATH} has ABI version {L.csrspmm_b200_abi_version()}, expected {ABI_VERSION}")
    _lib = L
    return L


def make_args(M, Kd, Nd, nnz, row_ptr=0, col_idx=0, values=0, B=0, Cptr=0, *, ldb=None, ldc=None,
              alpha=1.0, beta=0.0, entry=ENTRY_NAIVE, kernel=KERNEL_AUTO, max_row_nnz=0,
              value_format=VALUES_F32, value_scale=1.0, workspace=0, workspace_bytes=0,
              status_word=0, row_ptr_base=0, schedule=0) -> Args:
    a = Args()
    a.struct_size = C.sizeof(Args)
    a.M, a.Kd, a.Nd, a.nnz = int(M), int(Kd), int(Nd), int(nnz)
    a.row_ptr, a.col_idx, a.values = row_ptr or None, col_idx or None, values or None
    a.value_format, a.value_scale = int(value_format), float(value_scale)
    a.B, a.ldb = B or None, int(Nd if ldb is None else ldb)
    a.C, a.ldc = Cptr or None, int(Nd if ldc is None else ldc)
    a.alpha, a.beta = float(alpha), float(beta)
    a.entry, a.kernel, a.max_row_nnz = int(entry), int(kernel), int(max_row_nnz)
    a.row_ptr_base = int(row_ptr_base)
    a.workspace, a.workspace_bytes = workspace or None, int(workspace_bytes)
    a.status_word = status_word or None
    a.schedule = schedule or None
    return a


def check(status: int, where: str) -> None:
    if status != OK:
        raise SpmmError(status, where)
