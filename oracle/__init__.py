"""CPU oracle for the CSR x dense SpMM path.  TEST INFRASTRUCTURE ONLY.

Python face of ``oracle/spmm_oracle.c`` (the restatement of the reference kernels' arithmetic,
``src/device/csrspmm_naive.cu:27-38``) and, when it has been built, of ``oracle/_ref`` (the
reference's own ``src/host/csr_utils.cpp`` and ``src/host/dense_utils.cpp`` compiled unmodified
behind ``oracle/ref_shim.cpp``).

Nothing in the product package imports this module.  Its users are the test-suite, the smoke
check and the benchmark's CPU-baseline legs.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libspmm_oracle.so"
_REF_PATH = _HERE / "_ref" / "libcsrspmm_ref_host.so"
_REF_GPU_PATH = _HERE / "_ref" / "libcsrspmm_ref_gpu.so"

_i32p = C.POINTER(C.c_int32)
_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)
_u8p = C.POINTER(C.c_uint8)


def build(with_ref: bool | None = None) -> None:
    """Compile the oracle (and the reference cross-check when its checkout is present)."""
    targets = ["all"]
    # the reference checkout: CSRSPMM_REFERENCE, else a checkout next to this repository
    ref_root = os.environ.get("CSRSPMM_REFERENCE") or str(_HERE.parents[1] / "reference")
    if with_ref is None:
        with_ref = Path(ref_root, "src", "host", "dense_utils.cpp").exists()
    if with_ref:
        targets.append("ref")
        targets.append("refgpu")
        if (_HERE.parent / "csrspmm_b200" / "lib" / "libcsrspmm_b200.so").exists():
            targets.append("dropin")
            targets.append("pyext")
    subprocess.run(["make", "-s", "-C", str(_HERE), f"REFERENCE={ref_root}", *targets], check=True)


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            build()
        L = C.CDLL(str(_LIB_PATH))
        L.oracle_spmm_f32.argtypes = [C.c_int, C.c_int, C.c_int, _i32p, _i32p, _f32p, _f32p, C.c_int64,
                                      _f32p, C.c_int64, C.c_float, C.c_float, C.c_int, C.c_int]
        L.oracle_spmm_f32.restype = None
        L.oracle_spmm_f64.argtypes = [C.c_int, C.c_int, _i32p, _i32p, _f32p, _f32p, C.c_int64, _f32p,
                                      C.c_int64, C.c_float, C.c_float, _f64p, _f64p, C.c_int]
        L.oracle_spmm_f64.restype = None
        L.oracle_spmm_rows_f32.argtypes = [C.c_int, _i32p, C.c_int, _i32p, _i32p, _f32p, _f32p,
                                           C.c_int64, _f32p, C.c_int64, C.c_float, C.c_float,
                                           C.c_int, _f32p]
        L.oracle_spmm_rows_f32.restype = None
        L.oracle_dense2csr_count.argtypes = [C.c_int, C.c_int, _f32p, C.c_float]
        L.oracle_dense2csr_count.restype = C.c_int64
        L.oracle_dense2csr_fill.argtypes = [C.c_int, C.c_int, _f32p, C.c_float, _i32p, _i32p, _f32p]
        L.oracle_dense2csr_fill.restype = C.c_int
        L.oracle_csr2dense.argtypes = [C.c_int, C.c_int, _i32p, _i32p, _f32p, _f32p]
        L.oracle_csr2dense.restype = None
        L.oracle_e2m1_encode_one.argtypes = [C.c_float, C.c_float]
        L.oracle_e2m1_encode_one.restype = C.c_uint8
        L.oracle_e2m1_decode_one.argtypes = [C.c_uint8, C.c_float]
        L.oracle_e2m1_decode_one.restype = C.c_float
        L.oracle_e2m1_scale.argtypes = [C.c_int64, _f32p]
        L.oracle_e2m1_scale.restype = C.c_float
        L.oracle_e2m1_encode.argtypes = [C.c_int64, _f32p, C.c_float, _u8p]
        L.oracle_e2m1_encode.restype = None
        L.oracle_e2m1_decode.argtypes = [C.c_int64, _u8p, C.c_float, _f32p]
        L.oracle_e2m1_decode.restype = None
        L.oracle_max_threads.restype = C.c_int
        _lib = L
    return _lib


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def max_threads() -> int:
    """Host threads the oracle may use: the cores this process is allowed on.  Not OpenMP's own default,
    which a launcher may have capped through OMP_NUM_THREADS (torch.distributed.run sets it to 1); the
    parallel regions take their thread count explicitly, so the cap does not apply to them."""
    try:
        return max(len(os.sched_getaffinity(0)), 1)
    except AttributeError:
        return max(os.cpu_count() or 1, int(lib().oracle_max_threads()))


def spmm(row_ptr, col_idx, values, B, C_in=None, alpha=1.0, beta=0.0, *, fused=True, ncols=None,
         threads=1, out=None) -> np.ndarray:
    """alpha*A*B + beta*C_in in fp32, each output accumulated sequentially in stored order.

    ``fused=True`` accumulates with fmaf (what the GPU kernels do); ``fused=False`` rounds the
    product and the sum separately (what the reference's ``dense_gemm_cpu`` does when built
    without contraction).  With ``beta == 0`` the old C is never read, as in
    ``src/device/csrspmm_naive.cu:38``; columns >= ncols keep the contents of C_in (or zero).
    """
    row_ptr, col_idx, values, B = _i32(row_ptr), _i32(col_idx), _f32(values), _f32(B)
    M, Nd = row_ptr.shape[0] - 1, B.shape[1]
    if out is not None:  # timing runs: write into a caller buffer that is already paged in
        if out.dtype != np.float32 or out.shape != (M, Nd) or not out.flags.c_contiguous:
            raise ValueError("out must be a C-contiguous float32 array of shape (M, Nd)")
        if C_in is not None:
            out[...] = C_in
    else:
        out = np.zeros((M, Nd), np.float32) if C_in is None else _f32(C_in).copy()
    if beta != 0.0 and C_in is None:
        raise ValueError("beta != 0 needs C_in")
    lib().oracle_spmm_f32(M, Nd, Nd if ncols is None else int(ncols), _p(row_ptr, _i32p),
                          _p(col_idx, _i32p), _p(values, _f32p), _p(B, _f32p), B.shape[1],
                          _p(out, _f32p), Nd, float(alpha), float(beta), 0 if fused else 1,
                          int(threads))
    return out


def spmm_f64(row_ptr, col_idx, values, B, C_in=None, alpha=1.0, beta=0.0, threads=1):
    """The same product carried in double.  Returns (result, magnitude) where magnitude is
    |alpha|*sum|a*b| + |beta*C_in|, the scale for judging a re-associated fp32 sum."""
    row_ptr, col_idx, values, B = _i32(row_ptr), _i32(col_idx), _f32(values), _f32(B)
    M, Nd = row_ptr.shape[0] - 1, B.shape[1]
    out = np.empty((M, Nd), np.float64)
    mag = np.empty((M, Nd), np.float64)
    cold = _f32(C_in) if C_in is not None else None
    if beta != 0.0 and cold is None:
        raise ValueError("beta != 0 needs C_in")
    lib().oracle_spmm_f64(M, Nd, _p(row_ptr, _i32p), _p(col_idx, _i32p), _p(values, _f32p),
                          _p(B, _f32p), B.shape[1], _p(cold, _f32p) if cold is not None else None,
                          Nd, float(alpha), float(beta), _p(out, _f64p), _p(mag, _f64p), int(threads))
    return out, mag


def spmm_rows(rows, row_ptr, col_idx, values, B, C_in=None, alpha=1.0, beta=0.0, fused=True):
    """Oracle result for the listed rows only (len(rows) x Nd)."""
    rows = _i32(rows)
    row_ptr, col_idx, values, B = _i32(row_ptr), _i32(col_idx), _f32(values), _f32(B)
    Nd = B.shape[1]
    out = np.zeros((rows.shape[0], Nd), np.float32)
    cold = _f32(C_in) if C_in is not None else None
    if beta != 0.0 and cold is None:
        raise ValueError("beta != 0 needs C_in")
    lib().oracle_spmm_rows_f32(rows.shape[0], _p(rows, _i32p), Nd, _p(row_ptr, _i32p),
                               _p(col_idx, _i32p), _p(values, _f32p), _p(B, _f32p), B.shape[1],
                               _p(cold, _f32p) if cold is not None else None, Nd, float(alpha),
                               float(beta), 0 if fused else 1, _p(out, _f32p))
    return out


def dense2csr(dense, tol=0.0):
    """(row_ptr, col_idx, values, max_row_nnz) following src/host/csr_utils.cpp:85-110."""
    dense = _f32(dense)
    H, W = dense.shape
    nnz = int(lib().oracle_dense2csr_count(H, W, _p(dense, _f32p), float(tol)))
    row_ptr = np.empty(H + 1, np.int32)
    col_idx = np.empty(nnz, np.int32)
    values = np.empty(nnz, np.float32)
    mx = lib().oracle_dense2csr_fill(H, W, _p(dense, _f32p), float(tol), _p(row_ptr, _i32p),
                                     _p(col_idx, _i32p), _p(values, _f32p))
    return row_ptr, col_idx, values, int(mx)


def csr2dense(H, W, row_ptr, col_idx, values) -> np.ndarray:
    row_ptr, col_idx, values = _i32(row_ptr), _i32(col_idx), _f32(values)
    out = np.empty((H, W), np.float32)
    lib().oracle_csr2dense(H, W, _p(row_ptr, _i32p), _p(col_idx, _i32p), _p(values, _f32p),
                           _p(out, _f32p))
    return out


# ---- e2m1 codec (defined by this library; no counterpart in the reference) -------------------

E2M1_MAGNITUDES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)


def e2m1_scale(values) -> float:
    values = _f32(values)
    return float(lib().oracle_e2m1_scale(values.shape[0], _p(values, _f32p)))


def e2m1_encode(values, scale) -> np.ndarray:
    values = _f32(values)
    packed = np.zeros((values.shape[0] + 1) // 2, np.uint8)
    lib().oracle_e2m1_encode(values.shape[0], _p(values, _f32p), float(scale), _p(packed, _u8p))
    return packed


def e2m1_decode(packed, n, scale) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty(int(n), np.float32)
    lib().oracle_e2m1_decode(int(n), _p(packed, _u8p), float(scale), _p(out, _f32p))
    return out


def e2m1_encode_one(v, scale=1.0) -> int:
    return int(lib().oracle_e2m1_encode_one(float(v), float(scale)))


def e2m1_decode_one(code, scale=1.0) -> float:
    return float(lib().oracle_e2m1_decode_one(int(code), float(scale)))


# ---- the reference's own host code (oracle/_ref), when built ----------------------------------

class Reference:
    """The reference's dense2csr / csr2dense / dense_gemm_cpu / dense_compare, run on the CPU."""

    def __init__(self):
        path = _REF_PATH
        if not path.exists():
            raise FileNotFoundError(f"{path} not built (needs the reference checkout: make -C oracle ref)")
        L = C.CDLL(str(path))
        L.ref_dense2csr.argtypes = [C.c_int, C.c_int, _f32p, C.c_float, C.POINTER(_i32p),
                                    C.POINTER(_i32p), C.POINTER(_f32p), C.POINTER(C.c_int)]
        L.ref_dense2csr.restype = C.c_int
        L.ref_free.argtypes = [C.c_void_p]
        L.ref_csr2dense.argtypes = [C.c_int, C.c_int, C.c_int, _i32p, _i32p, _f32p, _f32p]
        L.ref_dense_gemm_cpu.argtypes = [C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, _f32p,
                                         _f32p, _f32p]
        L.ref_dense_compare.argtypes = [C.c_int, C.c_int, _f32p, _f32p, C.c_float]
        L.ref_dense_compare.restype = C.c_int
        L.ref_compression_ratio.argtypes = [C.c_int, C.c_int, C.c_int]
        L.ref_compression_ratio.restype = C.c_float
        self.L = L

    @staticmethod
    def available() -> bool:
        return _REF_PATH.exists()

    def dense2csr(self, dense, tol=0.0):
        dense = _f32(dense)
        H, W = dense.shape
        rp, ci, va, mx = _i32p(), _i32p(), _f32p(), C.c_int(0)
        nnz = self.L.ref_dense2csr(H, W, _p(dense, _f32p), float(tol), C.byref(rp), C.byref(ci),
                                   C.byref(va), C.byref(mx))
        row_ptr = np.ctypeslib.as_array(rp, (H + 1,)).copy()
        col_idx = np.ctypeslib.as_array(ci, (nnz,)).copy() if nnz else np.empty(0, np.int32)
        values = np.ctypeslib.as_array(va, (nnz,)).copy() if nnz else np.empty(0, np.float32)
        for ptr in (rp, ci, va):
            self.L.ref_free(C.cast(ptr, C.c_void_p))
        return row_ptr, col_idx, values, int(mx.value)

    def csr2dense(self, H, W, row_ptr, col_idx, values):
        row_ptr, col_idx, values = _i32(row_ptr), _i32(col_idx), _f32(values)
        out = np.empty((H, W), np.float32)
        self.L.ref_csr2dense(H, W, values.shape[0], _p(row_ptr, _i32p), _p(col_idx, _i32p),
                             _p(values, _f32p), _p(out, _f32p))
        return out

    def dense_gemm_cpu(self, A, B, C_in, alpha, beta):
        A, B = _f32(A), _f32(B)
        out = _f32(C_in).copy()
        self.L.ref_dense_gemm_cpu(A.shape[0], A.shape[1], B.shape[1], float(alpha), float(beta),
                                  _p(A, _f32p), _p(B, _f32p), _p(out, _f32p))
        return out

    def dense_compare(self, A, B, tol=1e-4) -> bool:
        A, B = _f32(A), _f32(B)
        return bool(self.L.ref_dense_compare(A.shape[0], A.shape[1], _p(A, _f32p), _p(B, _f32p),
                                             float(tol)))

    def compression_ratio(self, H, W, nnz) -> float:
        return float(self.L.ref_compression_ratio(H, W, nnz))


class ReferenceGpu:
    """The reference's own GPU kernels (recompiled for sm_100a, oracle/_ref/libcsrspmm_ref_gpu.so),
    launched on torch CUDA tensors through oracle/ref_gpu_shim.cu.  Legacy default stream."""

    ALGOS = {"Naive": 0, "WarpPerRow": 2, "WarpPerRowFp4": 3, "WarpPerRowSmem": 4, "WarpPerRowSmemFp4": 5}

    def __init__(self):
        if not _REF_GPU_PATH.exists():
            raise FileNotFoundError(f"{_REF_GPU_PATH} not built (needs the reference checkout: make -C oracle refgpu)")
        self.L = C.CDLL(str(_REF_GPU_PATH))
        self.L.ref_gpu_spmm.argtypes = [C.c_int] * 5 + [C.c_void_p] * 3 + [C.c_int] + [C.c_void_p] * 2 + [C.c_float] * 2
        self.L.ref_gpu_spmm.restype = C.c_int

    @staticmethod
    def available() -> bool:
        return _REF_GPU_PATH.exists()

    def spmm(self, algo, row_ptr, col_idx, values, B, C_out, alpha=1.0, beta=0.0, max_row_nnz=0) -> int:
        """Enqueue C_out = alpha*A*B + beta*C_out with the reference kernel `algo`.  Returns 0, or -2
        when the reference cannot run this shape (32-bit offsets, shared memory, alignment)."""
        M, Kd, Nd = row_ptr.numel() - 1, B.shape[0], B.shape[1]
        return int(self.L.ref_gpu_spmm(self.ALGOS[algo], M, Kd, Nd, col_idx.numel(), row_ptr.data_ptr(),
                                       col_idx.data_ptr(), values.data_ptr(), int(max_row_nnz), B.data_ptr(),
                                       C_out.data_ptr(), float(alpha), float(beta)))
