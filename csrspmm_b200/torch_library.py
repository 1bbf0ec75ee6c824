"""``torch.library`` registration of the SpMM, with a gradient for B, and a small CSR holder.

The reference's Python ops are plain pybind functions (torch_csrspmm/binding.cpp:26-32): opaque to
``torch.compile``, no ``out=``, no autograd, ``beta`` only ever multiplying a fresh zero tensor
(torch_csrspmm/torch_csrspmm_naive.cpp:32-34).  This module adds, on top of the same C ABI:

* ``torch.ops.csrspmm_b200.spmm(row_ptr, col_idx, values, B, alpha, kernel)`` -> new C, with a fake
  (meta) implementation so it traces, and an autograd formula for B:
  ``dB = alpha * A^T @ dC`` (A^T built once per matrix as a CSR, by a stable sort on the device);
* ``torch.ops.csrspmm_b200.spmm_(row_ptr, col_idx, values, B, C, alpha, beta, kernel)`` -> in place
  ``C = alpha * A @ B + beta * C`` (the reference's full semantics);
* ``CsrMatrix``: keeps the three arrays, the longest row (so AUTO can pick the row kernel), the cached
  transpose and, per dense width, the matrix's schedule (``csrspmm_b200_schedule_create``) together.

Gradients with respect to the stored values of A (a sampled dense-dense product) are not provided.
"""
from __future__ import annotations

import torch

from . import ops


def transpose_csr(row_ptr: torch.Tensor, col_idx: torch.Tensor, values: torch.Tensor, Kd: int):
    """CSR of A^T (Kd x M) from the CSR of A (M x Kd), on the arrays' device.  Entries of a column
    keep their row order (stable sort), so the result has ascending, distinct column indices
    whenever A has no repeated entry."""
    M = row_ptr.numel() - 1
    lens = (row_ptr[1:] - row_ptr[:-1]).long()
    rows = torch.repeat_interleave(torch.arange(M, device=row_ptr.device, dtype=torch.int32), lens)
    order = torch.sort(col_idx.long(), stable=True).indices
    t_col = rows[order].contiguous()
    t_val = values[order].contiguous()
    counts = torch.bincount(col_idx.long(), minlength=Kd)
    t_rp = torch.zeros(Kd + 1, dtype=torch.int32, device=row_ptr.device)
    t_rp[1:] = torch.cumsum(counts, 0).to(torch.int32)
    return t_rp, t_col, t_val


@torch.library.custom_op("csrspmm_b200::spmm", mutates_args=(), device_types="cuda")
def spmm_op(row_ptr: torch.Tensor, col_idx: torch.Tensor, values: torch.Tensor, B: torch.Tensor, alpha: float,
            kernel: str) -> torch.Tensor:
    return ops.spmm(row_ptr, col_idx, values, B.contiguous(), None, alpha, 0.0, kernel=kernel)


@spmm_op.register_fake
def _spmm_fake(row_ptr, col_idx, values, B, alpha, kernel):
    return B.new_empty((row_ptr.shape[0] - 1, B.shape[1]))


@torch.library.custom_op("csrspmm_b200::spmm_", mutates_args=("C",), device_types="cuda")
def spmm_inplace_op(row_ptr: torch.Tensor, col_idx: torch.Tensor, values: torch.Tensor, B: torch.Tensor,
                    C: torch.Tensor, alpha: float, beta: float, kernel: str) -> None:
    ops.spmm(row_ptr, col_idx, values, B, C, alpha, beta, kernel=kernel)


def _setup_context(ctx, inputs, output):
    row_ptr, col_idx, values, B, alpha, kernel = inputs
    ctx.save_for_backward(row_ptr, col_idx, values)
    ctx.Kd, ctx.alpha, ctx.kernel = B.shape[0], alpha, kernel
    ctx.values_need_grad = values.requires_grad


def _backward(ctx, grad_C):
    if ctx.values_need_grad:
        raise RuntimeError("csrspmm_b200::spmm has no gradient for the stored values of A")
    row_ptr, col_idx, values = ctx.saved_tensors
    t_rp, t_ci, t_va = transpose_csr(row_ptr, col_idx, values, ctx.Kd)
    dB = spmm_op(t_rp, t_ci, t_va, grad_C.contiguous(), ctx.alpha, ctx.kernel)
    return None, None, None, dB, None, None


spmm_op.register_autograd(_backward, setup_context=_setup_context)


class CsrMatrix:
    """A CSR matrix on a CUDA device together with what repeated products need: the longest row
    (lets AUTO choose the whole-row kernel when rows are even) and, on first use, the transpose."""

    def __init__(self, row_ptr: torch.Tensor, col_idx: torch.Tensor, values: torch.Tensor, shape, validate: bool = False):
        self.row_ptr, self.col_idx, self.values = row_ptr, col_idx, values
        self.shape = (int(shape[0]), int(shape[1]))
        if row_ptr.numel() != self.shape[0] + 1:
            raise ValueError("row_ptr must have shape[0] + 1 entries")
        if validate:
            ops.validate_csr(row_ptr, col_idx, self.shape[1])
        self.max_row_nnz = ops.row_stats(row_ptr)["max_row_nnz"] if row_ptr.is_cuda else 0
        self._t = None
        self._schedules = {}  # dense width -> ops.Schedule or None (built on first use, kept with the matrix)

    def schedule(self, Nd: int):
        """The per-matrix schedule for a B of ``Nd`` columns, built on first use (a few milliseconds) and kept;
        None when the library finds nothing worth scheduling for this matrix and width."""
        Nd = int(Nd)
        if Nd not in self._schedules:
            sched = None
            if self.row_ptr.is_cuda and self.nnz > 0:
                sched = ops.Schedule(self.row_ptr, self.col_idx, self.shape[1], Nd)
                if not sched.active:
                    sched.close()
                    sched = None
            self._schedules[Nd] = sched
        return self._schedules[Nd]

    @property
    def nnz(self) -> int:
        return int(self.col_idx.numel())

    def t(self) -> "CsrMatrix":
        if self._t is None:
            rp, ci, va = transpose_csr(self.row_ptr, self.col_idx, self.values, self.shape[1])
            self._t = CsrMatrix(rp, ci, va, (self.shape[1], self.shape[0]))
            self._t._t = self
        return self._t

    def matmul(self, B: torch.Tensor, alpha: float = 1.0, *, out: torch.Tensor | None = None, beta: float = 0.0,
               kernel: str = "auto") -> torch.Tensor:
        """alpha * A @ B (+ beta * out).  Differentiable in B when ``out`` is None."""
        if out is None and B.requires_grad:
            return _CsrMatmul.apply(self, B, float(alpha), kernel)
        return ops.spmm(self.row_ptr, self.col_idx, self.values, B, out, alpha, beta, kernel=kernel,
                        max_row_nnz=self.max_row_nnz, schedule=self.schedule(B.shape[1]) if kernel == "auto" else None)

    __matmul__ = matmul


class _CsrMatmul(torch.autograd.Function):
    """A @ B with the cached transpose for the backward product."""

    @staticmethod
    def forward(ctx, A: CsrMatrix, B: torch.Tensor, alpha: float, kernel: str):
        ctx.A, ctx.alpha, ctx.kernel = A, alpha, kernel
        return ops.spmm(A.row_ptr, A.col_idx, A.values, B.contiguous(), None, alpha, 0.0, kernel=kernel,
                        max_row_nnz=A.max_row_nnz, schedule=A.schedule(B.shape[1]) if kernel == "auto" else None)

    @staticmethod
    def backward(ctx, grad_C):
        At = ctx.A.t()
        dB = ops.spmm(At.row_ptr, At.col_idx, At.values, grad_C.contiguous(), None, ctx.alpha, 0.0, kernel=ctx.kernel,
                      max_row_nnz=At.max_row_nnz, schedule=At.schedule(grad_C.shape[1]) if ctx.kernel == "auto" else None)
        return None, dB, None, None
