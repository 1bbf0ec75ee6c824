"""Torch-tensor face of the C ABI: the five ops of the reference's ``torch_csrspmm`` package plus
a general ``spmm`` with in-place C, strides, packed e2m1 values and a pinned kernel.

The reference's ops are pybind wrappers that fill the two POD views from ``data_ptr()`` and call
``csrspmm::launch_*`` on the legacy default stream without a device guard
(torch_csrspmm/torch_csrspmm_naive.cpp:11-58 and its four siblings).  Here the same arguments go
through ``csrspmm_b200_spmm`` on torch's *current* stream of the tensors' device, and a failed
call raises instead of returning an unwritten C.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

_ENTRY = {
    "naive": _lib.ENTRY_NAIVE,
    "naive_smem": _lib.ENTRY_NAIVE_SMEM,
    "warp_per_row": _lib.ENTRY_WARP_PER_ROW,
    "warp_per_row_fp4": _lib.ENTRY_WARP_PER_ROW_FP4,
    "warp_per_row_smem": _lib.ENTRY_WARP_PER_ROW_SMEM,
    "warp_per_row_smem_fp4": _lib.ENTRY_WARP_PER_ROW_SMEM_FP4,
}


def _check_csr(row_ptr, col_idx, values, B, packed: bool):
    # same wording as the reference's TORCH_CHECKs (torch_csrspmm/torch_csrspmm_naive.cpp:19-26)
    if not row_ptr.is_cuda:
        raise RuntimeError("A_row_ptr must be a CUDA tensor")
    if not col_idx.is_cuda:
        raise RuntimeError("A_col_idx must be a CUDA tensor")
    if not values.is_cuda:
        raise RuntimeError("A_values must be a CUDA tensor")
    if not B.is_cuda:
        raise RuntimeError("B must be a CUDA tensor")
    if row_ptr.dtype != torch.int32:
        raise RuntimeError("A_row_ptr must be int32")
    if col_idx.dtype != torch.int32:
        raise RuntimeError("A_col_idx must be int32")
    if packed:
        if values.dtype != torch.uint8:
            raise RuntimeError("packed A_values must be uint8")
    elif values.dtype != torch.float32:
        raise RuntimeError("A_values must be float32")
    if B.dtype != torch.float32:
        raise RuntimeError("B must be float32")
    if B.dim() != 2 or row_ptr.dim() != 1 or col_idx.dim() != 1 or values.dim() != 1 or row_ptr.numel() < 1:
        raise RuntimeError("expected 1-D row_ptr/col_idx/values and 2-D B")
    if not (row_ptr.is_contiguous() and col_idx.is_contiguous() and values.is_contiguous()):
        raise RuntimeError("row_ptr, col_idx and values must be contiguous")
    if B.stride(1) != 1 and B.size(1) > 1:
        raise RuntimeError("B must be row-major (unit stride along its columns)")
    dev = B.device
    if not (row_ptr.device == dev and col_idx.device == dev and values.device == dev):
        raise RuntimeError("all tensors must be on the same device")


def workspace_bytes(M: int, Kd: int, Nd: int, nnz: int) -> int:
    """Scratch the split kernels need for a problem of these sizes."""
    a = _lib.make_args(M, Kd, Nd, nnz)
    return int(_lib.lib().csrspmm_b200_workspace_bytes(C.byref(a)))


class Schedule:
    """A per-matrix schedule (``csrspmm_b200_schedule_create``): the long rows of one sparsity pattern cut
    into pieces ordered by slab of B, so that their gather is served from L2.  Built once from the CUDA
    tensors ``row_ptr`` and ``col_idx``; valid while they are unchanged (values and B may change).  Pass it
    to ``spmm`` / ``SpmmCall`` as ``schedule=``.  ``Kd`` and ``Nd`` are the sizes of the B it will multiply
    (they size the slabs).  ``threshold`` / ``slab_rows`` / ``piece_nnz`` of 0 let the library choose."""

    def __init__(self, row_ptr, col_idx, Kd: int, Nd: int, *, ldb: int | None = None, threshold: int = 0,
                 slab_rows: int = 0, piece_nnz: int = 0):
        if not (row_ptr.is_cuda and col_idx.is_cuda and row_ptr.dtype == torch.int32 and col_idx.dtype == torch.int32):
            raise RuntimeError("a schedule is built from int32 CUDA row_ptr and col_idx")
        self.L = _lib.lib()
        self.device = row_ptr.device
        M, n = row_ptr.numel() - 1, col_idx.numel()
        a = _lib.make_args(M, int(Kd), int(Nd), n, row_ptr.data_ptr(), col_idx.data_ptr(), ldb=ldb or Nd)
        opt = _lib.ScheduleOptions(C.sizeof(_lib.ScheduleOptions), int(threshold), int(slab_rows), int(piece_nnz))
        handle = C.c_void_p(None)
        with torch.cuda.device(self.device):
            st = C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
            _lib.check(self.L.csrspmm_b200_schedule_create(C.byref(a), C.byref(opt), C.byref(handle), st),
                       "csrspmm_b200_schedule_create")
        self.handle = handle.value
        self._keep = (row_ptr, col_idx)

    def info(self) -> dict:
        i = _lib.ScheduleInfo()
        i.struct_size = C.sizeof(_lib.ScheduleInfo)
        _lib.check(self.L.csrspmm_b200_schedule_info_get(C.c_void_p(self.handle), C.byref(i)), "csrspmm_b200_schedule_info_get")
        return {k: getattr(i, k) for k, _ in _lib.ScheduleInfo._fields_ if k != "struct_size"}

    @property
    def active(self) -> bool:
        """False when the schedule is empty (no long rows, B fits one slab, or unsorted columns)."""
        return self.info()["long_rows"] > 0

    def close(self):
        if getattr(self, "handle", None):
            self.L.csrspmm_b200_schedule_destroy(C.c_void_p(self.handle))
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def spmm(row_ptr, col_idx, values, B, C_out=None, alpha=1.0, beta=0.0, *, entry="naive", kernel="auto",
         max_row_nnz=0, e2m1_scale=None, nnz=None, workspace=None, status_word=None, sync=False, schedule=None):
    """C_out = alpha * A @ B + beta * C_out on the current stream; returns C_out.

    C_out is allocated (uninitialised) when omitted, which requires beta == 0.  With
    ``e2m1_scale`` set, ``values`` holds packed 4-bit codes (uint8, two per byte) and ``nnz``
    gives the element count.  ``kernel`` pins "row", "merge" or "tma".  ``workspace`` is an
    optional uint8 tensor of at least ``workspace_bytes(...)`` bytes; without it the scratch comes
    from torch's caching allocator.  ``sync=True`` waits and raises on device-side errors.
    ``schedule`` is an optional ``Schedule`` built for this matrix.
    """
    packed = e2m1_scale is not None
    _check_csr(row_ptr, col_idx, values, B, packed)
    M = row_ptr.numel() - 1
    Kd, Nd = B.size(0), B.size(1)
    n = int(col_idx.numel() if nnz is None else nnz)
    if not packed and values.numel() != n:
        raise RuntimeError("values and col_idx differ in length")
    if packed and values.numel() < (n + 1) // 2:
        raise RuntimeError("packed values too short")
    if C_out is None:
        if beta != 0.0:
            raise RuntimeError("beta != 0 needs C_out")
        C_out = torch.empty((M, Nd), dtype=torch.float32, device=B.device)
    else:
        if not C_out.is_cuda or C_out.dtype != torch.float32 or C_out.shape != (M, Nd) or C_out.device != B.device:
            raise RuntimeError("C_out must be a float32 CUDA tensor of shape (M, Nd) on B's device")
        if C_out.stride(1) != 1 and Nd > 1:
            raise RuntimeError("C_out must be row-major")
    L = _lib.lib()
    ldb = B.stride(0) if Kd > 1 else Nd
    ldc = C_out.stride(0) if M > 1 else Nd
    a = _lib.make_args(M, Kd, Nd, n, row_ptr.data_ptr(), col_idx.data_ptr(), values.data_ptr(), B.data_ptr(),
                       C_out.data_ptr(), ldb=max(ldb, Nd), ldc=max(ldc, Nd), alpha=alpha, beta=beta,
                       entry=_ENTRY[entry] if isinstance(entry, str) else int(entry),
                       kernel=_lib.KERNEL_IDS[kernel] if isinstance(kernel, str) else int(kernel),
                       max_row_nnz=max_row_nnz,
                       value_format=_lib.VALUES_E2M1 if packed else _lib.VALUES_F32,
                       value_scale=float(e2m1_scale) if packed else 1.0,
                       status_word=status_word.data_ptr() if status_word is not None else 0,
                       schedule=schedule.handle if schedule is not None else 0)
    with torch.cuda.device(B.device):
        if M > 0 and Nd > 0:
            chosen = L.csrspmm_b200_select_kernel(C.byref(a))
            if chosen < 0:
                raise _lib.SpmmError(-chosen, "csrspmm_b200_select_kernel")
            if chosen != _lib.KERNEL_ROW:
                need = int(L.csrspmm_b200_workspace_bytes(C.byref(a)))
                if workspace is None or workspace.numel() * workspace.element_size() < need:
                    workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=B.device)
                a.workspace = workspace.data_ptr()
                a.workspace_bytes = workspace.numel() * workspace.element_size()
        stream = torch.cuda.current_stream(B.device).cuda_stream
        fn = L.csrspmm_b200_spmm_sync if sync else L.csrspmm_b200_spmm
        _lib.check(fn(C.byref(a), C.c_void_p(stream)), "csrspmm_b200_spmm")
        if workspace is not None:
            workspace.record_stream(torch.cuda.current_stream(B.device))
    return C_out


def spmm_tiled(row_ptr, col_idx, values, B, C_out=None, alpha=1.0, beta=0.0, *, panel_rows=0, e2m1_scale=None,
               nnz=None, workspace=None, status_word=None):
    """The same product as ``spmm`` in passes over column panels of A whose slab of B (``panel_rows`` rows;
    0 = the library's 64 MiB choice) stays in L2 (``csrspmm_b200_spmm_tiled``).  Opt-in: it pays when rows
    hold several non-zeros per panel and B is several times L2.  Bit-identical to the whole-row kernel."""
    packed = e2m1_scale is not None
    _check_csr(row_ptr, col_idx, values, B, packed)
    M, Kd, Nd = row_ptr.numel() - 1, B.size(0), B.size(1)
    n = int(col_idx.numel() if nnz is None else nnz)
    if C_out is None:
        if beta != 0.0:
            raise RuntimeError("beta != 0 needs C_out")
        C_out = torch.empty((M, Nd), dtype=torch.float32, device=B.device)
    elif not C_out.is_cuda or C_out.dtype != torch.float32 or C_out.shape != (M, Nd) or C_out.device != B.device:
        raise RuntimeError("C_out must be a float32 CUDA tensor of shape (M, Nd) on B's device")
    L = _lib.lib()
    a = _lib.make_args(M, Kd, Nd, n, row_ptr.data_ptr(), col_idx.data_ptr(), values.data_ptr(), B.data_ptr(),
                       C_out.data_ptr(), ldb=max(B.stride(0) if Kd > 1 else Nd, Nd),
                       ldc=max(C_out.stride(0) if M > 1 else Nd, Nd), alpha=alpha, beta=beta,
                       value_format=_lib.VALUES_E2M1 if packed else _lib.VALUES_F32,
                       value_scale=float(e2m1_scale) if packed else 1.0,
                       status_word=status_word.data_ptr() if status_word is not None else 0)
    with torch.cuda.device(B.device):
        need = int(L.csrspmm_b200_tiled_workspace_bytes(C.byref(a)))
        if workspace is None or workspace.numel() * workspace.element_size() < need:
            workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=B.device)
        a.workspace = workspace.data_ptr()
        a.workspace_bytes = workspace.numel() * workspace.element_size()
        stream = torch.cuda.current_stream(B.device)
        _lib.check(L.csrspmm_b200_spmm_tiled(C.byref(a), int(panel_rows), C.c_void_p(stream.cuda_stream)),
                   "csrspmm_b200_spmm_tiled")
        workspace.record_stream(stream)
    return C_out


def tiled_panel_rows(Kd: int, Nd: int, ldb: int | None = None) -> int:
    """Rows of B per panel that ``spmm_tiled`` chooses by itself (0: B is no larger than one slab)."""
    a = _lib.make_args(1, Kd, Nd, 0, ldb=ldb or Nd)
    return int(_lib.lib().csrspmm_b200_tiled_panel_rows(C.byref(a)))


class SpmmCall:
    """A prepared SpMM: argument block, kernel choice and scratch fixed once, so that each call is
    a single trip through the C ABI.  For tight launch loops (benchmarks, repeated products with the
    same operands); keeps its tensors alive."""

    def __init__(self, row_ptr, col_idx, values, B, C_out, alpha=1.0, beta=0.0, *, entry="naive", kernel="auto",
                 max_row_nnz=0, e2m1_scale=None, nnz=None, workspace=None, status_word=None, schedule=None):
        packed = e2m1_scale is not None
        _check_csr(row_ptr, col_idx, values, B, packed)
        M, Kd, Nd = row_ptr.numel() - 1, B.size(0), B.size(1)
        n = int(col_idx.numel() if nnz is None else nnz)
        if C_out.shape != (M, Nd) or C_out.dtype != torch.float32 or C_out.device != B.device:
            raise RuntimeError("C_out must be a float32 CUDA tensor of shape (M, Nd) on B's device")
        self.device = B.device
        self.L = _lib.lib()
        self.args = _lib.make_args(
            M, Kd, Nd, n, row_ptr.data_ptr(), col_idx.data_ptr(), values.data_ptr(), B.data_ptr(), C_out.data_ptr(),
            ldb=max(B.stride(0) if Kd > 1 else Nd, Nd), ldc=max(C_out.stride(0) if M > 1 else Nd, Nd), alpha=alpha,
            beta=beta, entry=_ENTRY[entry], kernel=_lib.KERNEL_IDS[kernel], max_row_nnz=max_row_nnz,
            value_format=_lib.VALUES_E2M1 if packed else _lib.VALUES_F32,
            value_scale=float(e2m1_scale) if packed else 1.0,
            status_word=status_word.data_ptr() if status_word is not None else 0,
            schedule=schedule.handle if schedule is not None else 0)
        self.kernel = "row"
        self.launches = 0
        if M > 0 and Nd > 0:
            k = self.L.csrspmm_b200_select_kernel(C.byref(self.args))
            if k < 0:
                raise _lib.SpmmError(-k, "csrspmm_b200_select_kernel")
            self.kernel = _lib.KERNEL_NAMES[k]
            # scheduled: pieces, slot sums, merge-path over the other rows, fix-up
            self.launches = 1 if k == _lib.KERNEL_ROW else (4 if k == _lib.KERNEL_SCHEDULED else 2)
            if k != _lib.KERNEL_ROW:
                need = int(self.L.csrspmm_b200_workspace_bytes(C.byref(self.args)))
                if workspace is None or workspace.numel() * workspace.element_size() < need:
                    workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=B.device)
                self.args.workspace = workspace.data_ptr()
                self.args.workspace_bytes = workspace.numel() * workspace.element_size()
        self.workspace = workspace  # scratch of the split kernels (None for the row kernel); may be shared
        self._keep = (row_ptr, col_idx, values, B, C_out, workspace, status_word, schedule)
        self._ref = C.byref(self.args)
        self.out = C_out

    def __call__(self):
        """Enqueue on the current stream of the operands' device (which must be the current device)."""
        st = self.L.csrspmm_b200_spmm(self._ref, C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        if st != _lib.OK:
            raise _lib.SpmmError(st, "csrspmm_b200_spmm")
        return self.out


def selected_kernel(M, Kd, Nd, nnz, *, entry="naive", max_row_nnz=0, kernel="auto", aligned=True) -> str:
    """Name of the kernel AUTO picks for these sizes (host-only, needs no GPU)."""
    a = _lib.make_args(M, Kd, Nd, nnz, B=256 if aligned else 4, Cptr=256 if aligned else 4,
                       entry=_ENTRY[entry], kernel=_lib.KERNEL_IDS[kernel], max_row_nnz=max_row_nnz)
    k = _lib.lib().csrspmm_b200_select_kernel(C.byref(a))
    if k < 0:
        raise _lib.SpmmError(-k, "csrspmm_b200_select_kernel")
    return _lib.KERNEL_NAMES[k]


# ---- the reference's five ops (torch_csrspmm/__init__.py:10-23): new C = alpha * A @ B ---------------
# The reference allocates C as zeros when beta != 0 and computes alpha*A*B + beta*0
# (torch_csrspmm/torch_csrspmm_naive.cpp:32-34); the product with zero is skipped here, which
# changes nothing but the sign of an exact zero.

_ROW_STATS_CACHE: dict = {}


def _longest_row_hint(row_ptr) -> int:
    """Longest row of the matrix behind this row_ptr tensor, measured once (one small kernel and a
    host read) and remembered per (address, length, version).  It only steers the kernel choice, so
    a stale entry -- another matrix later placed at the same address -- costs speed, never
    correctness."""
    key = (row_ptr.data_ptr(), row_ptr.numel(), row_ptr._version, row_ptr.device.index)
    hit = _ROW_STATS_CACHE.get(key)
    if hit is None:
        if len(_ROW_STATS_CACHE) >= 64:
            _ROW_STATS_CACHE.pop(next(iter(_ROW_STATS_CACHE)))
        hit = row_stats(row_ptr)["max_row_nnz"] if row_ptr.numel() > 1 else 0
        _ROW_STATS_CACHE[key] = hit
    return hit


def _op(entry, row_ptr, col_idx, values, B, alpha, beta, max_row_nnz=0):
    del beta
    if row_ptr.is_cuda and row_ptr.dtype == torch.int32:
        # measured, not believed: three of the reference's five ops carry no such argument, and a stale value
        # passed to the other two would send a skewed matrix to the whole-row kernel
        max_row_nnz = _longest_row_hint(row_ptr)
    return spmm(row_ptr, col_idx, values, B, None, float(alpha), 0.0, entry=entry, max_row_nnz=int(max_row_nnz))


def csrspmm_naive(A_rowptr, A_colidx, A_values, B, alpha, beta):
    return _op("naive", A_rowptr, A_colidx, A_values, B, alpha, beta)


def csrspmm_warp_per_row(A_rowptr, A_colidx, A_values, B, alpha, beta):
    return _op("warp_per_row", A_rowptr, A_colidx, A_values, B, alpha, beta)


def csrspmm_warp_per_row_smem(A_rowptr, A_colidx, A_values, A_max_row_nnz, B, alpha, beta):
    return _op("warp_per_row_smem", A_rowptr, A_colidx, A_values, B, alpha, beta, A_max_row_nnz)


def csrspmm_warp_per_row_fp4(A_rowptr, A_colidx, A_values, B, alpha, beta):
    return _op("warp_per_row_fp4", A_rowptr, A_colidx, A_values, B, alpha, beta)


def csrspmm_warp_per_row_smem_fp4(A_rowptr, A_colidx, A_values, A_max_row_nnz, B, alpha, beta):
    return _op("warp_per_row_smem_fp4", A_rowptr, A_colidx, A_values, B, alpha, beta, A_max_row_nnz)


# ---- helpers over the host-only / utility entry points -----------------------------------------------

def e2m1_quantize(values_f32):
    """fp32 tensor/array -> (packed uint8 tensor, scale) with the library's codec.  A CUDA tensor is
    encoded on its device and the packed tensor stays there; anything else is encoded on the host."""
    import numpy as np
    if isinstance(values_f32, torch.Tensor) and values_f32.is_cuda:
        v = values_f32.detach().to(torch.float32).contiguous()
        n = v.numel()
        L = _lib.lib()
        scale = C.c_float(1.0)
        packed = torch.empty((n + 1) // 2, dtype=torch.uint8, device=v.device)
        with torch.cuda.device(v.device):
            st = C.c_void_p(torch.cuda.current_stream(v.device).cuda_stream)
            _lib.check(L.csrspmm_b200_e2m1_scale_device(n, v.data_ptr(), C.byref(scale), st), "e2m1_scale_device")
            _lib.check(L.csrspmm_b200_e2m1_encode_device(n, v.data_ptr(), scale.value, packed.data_ptr(), st),
                       "e2m1_encode_device")
        return packed, float(scale.value)
    v = np.ascontiguousarray(values_f32.detach().cpu().numpy() if isinstance(values_f32, torch.Tensor)
                             else values_f32, dtype=np.float32)
    L = _lib.lib()
    scale = float(L.csrspmm_b200_e2m1_scale(v.shape[0], v.ctypes.data))
    packed = np.zeros((v.shape[0] + 1) // 2, np.uint8)
    _lib.check(L.csrspmm_b200_e2m1_encode(v.shape[0], v.ctypes.data, scale, packed.ctypes.data), "e2m1_encode")
    return torch.from_numpy(packed), scale


def e2m1_dequantize(packed, n, scale):
    """Packed codes -> fp32 values (on the device for a CUDA tensor, else on the host)."""
    import numpy as np
    if isinstance(packed, torch.Tensor) and packed.is_cuda:
        out = torch.empty(int(n), dtype=torch.float32, device=packed.device)
        with torch.cuda.device(packed.device):
            st = C.c_void_p(torch.cuda.current_stream(packed.device).cuda_stream)
            _lib.check(_lib.lib().csrspmm_b200_e2m1_decode_device(int(n), packed.contiguous().data_ptr(), float(scale),
                                                                  out.data_ptr(), st), "e2m1_decode_device")
        return out
    pk = np.ascontiguousarray(packed.cpu().numpy() if isinstance(packed, torch.Tensor) else packed, dtype=np.uint8)
    out = np.empty(int(n), np.float32)
    _lib.check(_lib.lib().csrspmm_b200_e2m1_decode(int(n), pk.ctypes.data, float(scale), out.ctypes.data),
               "e2m1_decode")
    return torch.from_numpy(out)


def validate_csr(row_ptr, col_idx, Kd: int) -> int:
    """Checks a CSR structure (host or CUDA int32 tensors); returns the problem bits and raises
    SpmmError(ERR_INVALID_CSR) when the matrix cannot be multiplied safely."""
    M = row_ptr.numel() - 1
    flags = C.c_uint32(0)
    L = _lib.lib()
    if row_ptr.is_cuda:
        with torch.cuda.device(row_ptr.device):
            st = L.csrspmm_b200_validate_csr_device(M, Kd, col_idx.numel(), row_ptr.data_ptr(), col_idx.data_ptr(),
                                                    C.byref(flags),
                                                    C.c_void_p(torch.cuda.current_stream(row_ptr.device).cuda_stream))
    else:
        st = L.csrspmm_b200_validate_csr_host(M, Kd, col_idx.numel(), row_ptr.data_ptr(), col_idx.data_ptr(),
                                              C.byref(flags))
    _lib.check(st, "csrspmm_b200_validate_csr")
    return int(flags.value)


def row_stats(row_ptr) -> dict:
    """Longest row, empty rows, rows longer than 32*(mean+1) and their nnz, from a CUDA row_ptr."""
    out = (C.c_int64 * 4)()
    with torch.cuda.device(row_ptr.device):
        st = _lib.lib().csrspmm_b200_row_stats_device(row_ptr.numel() - 1, row_ptr.data_ptr(), out,
                                                      C.c_void_p(torch.cuda.current_stream(row_ptr.device).cuda_stream))
    _lib.check(st, "csrspmm_b200_row_stats_device")
    return dict(max_row_nnz=int(out[0]), empty_rows=int(out[1]), long_rows=int(out[2]), long_rows_nnz=int(out[3]))


def spmm_host(row_ptr, col_idx, values, B, C_host, alpha=1.0, beta=0.0, *, entry="naive", kernel="auto",
              max_row_nnz=0, arena=None, device=None):
    """End-to-end call on HOST tensors (ideally pinned): copies A and B in, multiplies, copies C
    back into C_host and waits.  ``arena`` is an optional CUDA uint8 tensor to stage in.  row_ptr, col_idx
    and values may be CUDA tensors instead (a matrix kept on the GPU between products): they are then used
    in place and only B goes up."""
    M = row_ptr.numel() - 1
    Kd, Nd = B.shape
    a = _lib.make_args(M, Kd, Nd, col_idx.numel(), row_ptr.data_ptr(), col_idx.data_ptr(), values.data_ptr(),
                       B.data_ptr(), C_host.data_ptr(), ldb=B.stride(0) if Kd > 1 else Nd,
                       ldc=C_host.stride(0) if M > 1 else Nd, alpha=alpha, beta=beta, entry=_ENTRY[entry],
                       kernel=_lib.KERNEL_IDS[kernel], max_row_nnz=max_row_nnz)
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        st = _lib.lib().csrspmm_b200_spmm_host(C.byref(a), arena.data_ptr() if arena is not None else None,
                                               arena.numel() if arena is not None else 0, C.c_void_p(stream))
    _lib.check(st, "csrspmm_b200_spmm_host")
    return C_host


def copy_rows(dst: torch.Tensor, src: torch.Tensor) -> None:
    """Asynchronous strided copy between a host matrix and a CUDA matrix of the same shape, on the
    current stream of the CUDA side.  Either side may be a column slice of a wider row-major matrix
    (rows keep their pitch), which ``Tensor.copy_`` would first repack on the host."""
    if dst.shape != src.shape or dst.dim() != 2 or dst.dtype != src.dtype or dst.is_cuda == src.is_cuda:
        raise RuntimeError("copy_rows wants two 2-D tensors of one shape and dtype, one on the host and one on a GPU")
    rows, cols = dst.shape
    if rows == 0 or cols == 0:
        return
    if (cols > 1 and (dst.stride(1) != 1 or src.stride(1) != 1)):
        raise RuntimeError("copy_rows wants unit stride along the rows")
    es = dst.element_size()
    dpitch = (dst.stride(0) if rows > 1 else cols) * es
    spitch = (src.stride(0) if rows > 1 else cols) * es
    dev = dst.device if dst.is_cuda else src.device
    with torch.cuda.device(dev):
        st = _lib.lib().csrspmm_b200_copy_rows(dst.data_ptr(), dpitch, src.data_ptr(), spitch, cols * es, rows,
                                               0 if dst.is_cuda else 1,
                                               C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    _lib.check(st, "csrspmm_b200_copy_rows")


def host_arena_bytes(M, Kd, Nd, nnz) -> int:
    a = _lib.make_args(M, Kd, Nd, nnz)
    return int(_lib.lib().csrspmm_b200_host_arena_bytes(C.byref(a)))


# ---- dense <-> CSR on the device (csrspmm::dense2csr / csr2dense for device-resident matrices) ----------

def dense2csr(dense: torch.Tensor, tol: float = 0.0):
    """CUDA float32 matrix -> (row_ptr, col_idx, values, max_row_nnz), the arrays the reference's host
    ``dense2csr`` would produce (entries with |v| > tol, ascending columns), built on the device."""
    if not dense.is_cuda or dense.dtype != torch.float32 or dense.dim() != 2 or (dense.stride(1) != 1 and dense.size(1) > 1):
        raise RuntimeError("dense must be a row-major float32 CUDA matrix")
    H, W = dense.shape
    ld = dense.stride(0) if H > 1 else max(W, 1)
    L = _lib.lib()
    row_ptr = torch.empty(H + 1, dtype=torch.int32, device=dense.device)
    nnz, mx = C.c_int64(0), C.c_int32(0)
    with torch.cuda.device(dense.device):
        stream = C.c_void_p(torch.cuda.current_stream(dense.device).cuda_stream)
        _lib.check(L.csrspmm_b200_dense2csr_count(H, W, dense.data_ptr(), max(ld, W), float(tol), row_ptr.data_ptr(),
                                                  C.byref(nnz), C.byref(mx), stream), "csrspmm_b200_dense2csr_count")
        col_idx = torch.empty(nnz.value, dtype=torch.int32, device=dense.device)
        values = torch.empty(nnz.value, dtype=torch.float32, device=dense.device)
        if nnz.value > 0:
            _lib.check(L.csrspmm_b200_dense2csr_fill(H, W, dense.data_ptr(), max(ld, W), float(tol), row_ptr.data_ptr(),
                                                     col_idx.data_ptr(), values.data_ptr(), stream),
                       "csrspmm_b200_dense2csr_fill")
    return row_ptr, col_idx, values, int(mx.value)


def csr2dense(row_ptr: torch.Tensor, col_idx: torch.Tensor, values: torch.Tensor, shape) -> torch.Tensor:
    """CSR arrays on a CUDA device -> dense float32 matrix of the given shape."""
    H, W = int(shape[0]), int(shape[1])
    out = torch.empty((H, W), dtype=torch.float32, device=row_ptr.device)
    with torch.cuda.device(row_ptr.device):
        stream = C.c_void_p(torch.cuda.current_stream(row_ptr.device).cuda_stream)
        _lib.check(_lib.lib().csrspmm_b200_csr2dense(H, W, row_ptr.data_ptr(), col_idx.data_ptr(), values.data_ptr(),
                                                     out.data_ptr(), max(W, 1), stream), "csrspmm_b200_csr2dense")
    return out
