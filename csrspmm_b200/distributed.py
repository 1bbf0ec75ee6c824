"""Row-partitioned multi-GPU SpMM: one process per GPU, A and C sharded by rows, B replicated.

The reference is single-GPU (its launchers never select a device, src/host/spmm_launcher.cu), so
this module has no counterpart there.  Rows of C depend only on the same rows of A and on all
of B, so the product needs no exchange: the matrix is cut into contiguous row blocks of
near-equal cost (non-zeros + rows, found by binary search on ``row_ptr`` in the C library), each
rank keeps its block of A re-based to local offsets (column indices unchanged) and a full copy of
B that is broadcast ONCE, outside any timed region, and every rank multiplies its block with the
single-GPU kernels.  C stays sharded.  ``torch.distributed`` (NCCL on GPUs, gloo on CPU for the
host-logic tests) provides the broadcast, the barrier and the max-over-ranks reduction of times.

When the operands start in HOST memory (``ShardedHostSpmm``) there is one real exchange: each rank
uploads only 1/N of B over PCIe and the slices are all-gathered over NVLink, instead of every
rank pulling all of B through its own PCIe link.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib


def partition_rows(row_ptr, parts: int, row_weight: float = 1.0) -> np.ndarray:
    """bounds[g] .. bounds[g+1] = rows of part g.  ``row_ptr`` is a host array/tensor.  The cost of
    a row is its nnz + row_weight: with the default weight a row of C written counts like a
    row of B read, which is what the traffic is."""
    rp = np.ascontiguousarray(row_ptr.cpu().numpy() if isinstance(row_ptr, torch.Tensor) else row_ptr,
                              dtype=np.int32)
    bounds = np.zeros(parts + 1, np.int32)
    st = _lib.lib().csrspmm_b200_partition_rows(rp.shape[0] - 1, rp.ctypes.data, int(parts), float(row_weight),
                                                bounds.ctypes.data)
    _lib.check(st, "csrspmm_b200_partition_rows")
    return bounds


@dataclass
class Shard:
    """Rows [row_lo, row_hi) of A with offsets re-based to zero; column indices untouched."""
    rank: int
    world: int
    row_lo: int
    row_hi: int
    row_ptr: object
    col_idx: object
    values: object
    max_row_nnz: int

    @property
    def rows(self) -> int:
        return self.row_hi - self.row_lo

    @property
    def nnz(self) -> int:
        return int(self.col_idx.shape[0])


def take_shard(row_ptr, col_idx, values, bounds, rank: int) -> Shard:
    """Slice of a CSR matrix (numpy arrays or torch tensors on any device) for one rank."""
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    rp = row_ptr[lo:hi + 1]
    j0, j1 = int(rp[0]), int(rp[-1])
    local_rp = rp - rp[0]
    if isinstance(local_rp, torch.Tensor):
        local_rp = local_rp.to(torch.int32).contiguous()
        lens = local_rp[1:] - local_rp[:-1]
        mx = int(lens.max().item()) if hi > lo else 0
        ci, va = col_idx[j0:j1].contiguous(), values[j0:j1].contiguous()
    else:
        local_rp = np.ascontiguousarray(local_rp, dtype=np.int32)
        mx = int(np.diff(local_rp).max()) if hi > lo else 0
        ci, va = np.ascontiguousarray(col_idx[j0:j1]), np.ascontiguousarray(values[j0:j1])
    return Shard(rank, len(bounds) - 1, lo, hi, local_rp, ci, va, mx)


def replicate(t: torch.Tensor, src: int = 0) -> torch.Tensor:
    """Broadcast a tensor that every rank has already allocated with the same shape."""
    import torch.distributed as dist
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.broadcast(t, src=src)
    return t


def max_over_ranks(seconds: float, device) -> float:
    """Job time of a step that every rank timed on its own device."""
    import torch.distributed as dist
    t = torch.tensor([seconds], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, device) -> float:
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def column_panels(Kd: int, Nd: int, panels: int | None = None):
    """[(first column, width)] of the column panels a host round trip is cut into, as the C library
    lays them out.  ``panels`` None applies its rule (a B of 256 MiB or more with Nd >= 256: panels
    of 128 columns between a first and a last panel of 64; CSRSPMM_HOST_PANELS in the environment overrides); widths are
    multiples of 32 columns except possibly the last."""
    first = np.zeros(16, np.int32)
    width = np.zeros(16, np.int32)
    n = _lib.lib().csrspmm_b200_column_panels(int(Kd), int(Nd), int(panels or 0), first.ctypes.data, width.ctypes.data)
    if n < 1:
        raise ValueError("csrspmm_b200_column_panels: negative size")
    return [(int(first[k]), int(width[k])) for k in range(n)]


class ShardedHostSpmm:
    """End-to-end product from HOST memory on several GPUs: every rank uploads only its own part.

    Rank g holds, in pinned host memory, its row block of A and rows [g*Kd/world, (g+1)*Kd/world)
    of B.  One ``run()`` = upload the block of A and the slice of B, all-gather the slices over
    NVLink into the full device copy of B (the one exchange this path has: each byte of B
    crosses PCIe once instead of once per GPU), multiply, download the block of C.  With a
    single rank there is no exchange and this is the plain host round trip.

    A wide product runs in column panels (``column_panels``): C[:, panel] needs B[:, panel] only,
    so while panel q is gathered and multiplied, panel q+1 of the B slice is still arriving over
    PCIe and panel q-1 of C is already leaving -- uploads, NVLink exchange, kernels and downloads of
    different panels run at the same time, each stage on its own stream.  On the device each panel of B and
    of C is stored contiguously; every element of C is the same sum as in the unsplit product.

    ``keep_matrix=True`` uploads the block of A once, here, and keeps it on the device: ``run()`` then moves
    only B and C (repeated products on one matrix, where only B changes).
    """

    def __init__(self, shard_host: "Shard", B_slice_host: torch.Tensor, Kd: int, device, kernel: str = "auto",
                 panels: int | None = None, keep_matrix: bool = False):
        import torch.distributed as dist
        from . import ops
        self.dist, self.ops, self.dev = dist, ops, torch.device(device)
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        if Kd % self.world != 0 or B_slice_host.shape[0] * self.world != Kd:
            raise ValueError("Kd must be divisible by the number of ranks and B_slice_host hold Kd/world rows")
        self.h_rp, self.h_ci, self.h_va, self.h_B = shard_host.row_ptr, shard_host.col_idx, shard_host.values, B_slice_host
        Nd, rows = B_slice_host.shape[1], shard_host.rows
        d = self.dev
        self.d_rp = torch.empty(rows + 1, dtype=torch.int32, device=d)
        self.d_ci = torch.empty(shard_host.nnz, dtype=torch.int32, device=d)
        self.d_va = torch.empty(shard_host.nnz, dtype=torch.float32, device=d)
        self.C_host = torch.empty((rows, Nd), dtype=torch.float32, pin_memory=True)
        self.slice_rows = Kd // self.world
        self.panels = column_panels(Kd, Nd, panels)
        flat_B = torch.empty(Kd * Nd, dtype=torch.float32, device=d)
        flat_C = torch.empty(rows * Nd, dtype=torch.float32, device=d)
        self.d_B = [flat_B[Kd * c0:Kd * (c0 + w)].view(Kd, w) for c0, w in self.panels]
        self.d_C = [flat_C[rows * c0:rows * (c0 + w)].view(rows, w) for c0, w in self.panels]
        self.calls, ws = [], None
        for Bq, Cq in zip(self.d_B, self.d_C):  # widest panel first, so its scratch serves the others
            call = ops.SpmmCall(self.d_rp, self.d_ci, self.d_va, Bq, Cq, 1.0, 0.0, kernel=kernel,
                                max_row_nnz=shard_host.max_row_nnz, workspace=ws)
            ws = call.workspace if ws is None else ws
            self.calls.append(call)
        with torch.cuda.device(d):
            self.s_up, self.s_gather, self.s_mul, self.s_down = (torch.cuda.Stream(d) for _ in range(4))
            self.ev_up = [torch.cuda.Event() for _ in self.panels]
            self.ev_gather = [torch.cuda.Event() for _ in self.panels]
            self.ev_mul = [torch.cuda.Event() for _ in self.panels]
        self.keep_matrix = bool(keep_matrix)
        if self.keep_matrix:
            self.d_rp.copy_(self.h_rp)
            self.d_ci.copy_(self.h_ci)
            self.d_va.copy_(self.h_va)
            torch.cuda.synchronize(d)
        self.h2d_bytes = (0 if self.keep_matrix else (rows + 1) * 4 + shard_host.nnz * 8) + self.slice_rows * Nd * 4
        self.d2h_bytes = rows * Nd * 4
        self.exchange_bytes = (Kd - self.slice_rows) * Nd * 4  # received over NVLink per rank

    def run(self) -> torch.Tensor:
        k0, k1 = self.rank * self.slice_rows, (self.rank + 1) * self.slice_rows
        self.s_up.wait_stream(torch.cuda.current_stream(self.dev))
        if not self.keep_matrix:
            with torch.cuda.stream(self.s_up):
                self.d_rp.copy_(self.h_rp, non_blocking=True)
                self.d_ci.copy_(self.h_ci, non_blocking=True)
                self.d_va.copy_(self.h_va, non_blocking=True)
        for q, (c0, w) in enumerate(self.panels):
            mine = self.d_B[q][k0:k1]
            with torch.cuda.stream(self.s_up):
                self.ops.copy_rows(mine, self.h_B[:, c0:c0 + w])
                self.ev_up[q].record()
            ready = self.ev_up[q]
            if self.world > 1:
                with torch.cuda.stream(self.s_gather):
                    self.s_gather.wait_event(self.ev_up[q])
                    self.dist.all_gather_into_tensor(self.d_B[q], mine)  # in place: slice g already sits at offset g
                    self.ev_gather[q].record()
                ready = self.ev_gather[q]
            with torch.cuda.stream(self.s_mul):
                self.s_mul.wait_event(ready)
                self.calls[q]()
                self.ev_mul[q].record()
            with torch.cuda.stream(self.s_down):
                self.s_down.wait_event(self.ev_mul[q])
                self.ops.copy_rows(self.C_host[:, c0:c0 + w], self.d_C[q])
        self.s_down.synchronize()  # the last download follows every other stage
        return self.C_host


def partition_imbalance(row_ptr, bounds, row_weight: float = 1.0) -> float:
    """max part cost / mean part cost (1.0 = perfect)."""
    rp = np.asarray(row_ptr.cpu().numpy() if isinstance(row_ptr, torch.Tensor) else row_ptr, dtype=np.int64)
    b = np.asarray(bounds, dtype=np.int64)
    cost = (rp[b[1:]] - rp[b[:-1]]) + row_weight * (b[1:] - b[:-1])
    return float(cost.max() / max(cost.mean(), 1e-30))
