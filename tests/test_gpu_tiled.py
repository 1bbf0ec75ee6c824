"""csrspmm_b200_spmm_tiled: the product in column panels (a locality pass for B far larger than L2).
Every output still accumulates in stored order, so results are compared bit for bit with the sequential
oracle and with the whole-row kernel."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from csrspmm_b200 import _lib, generators as G, ops

pytestmark = pytest.mark.gpu


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def arrays(p):
    return p.row_ptr, p.col_idx, p.values, p.B


@pytest.mark.parametrize("Nd", [1, 3, 4, 20, 64, 100, 128, 256, 512, 600, 1100])
@pytest.mark.parametrize("panel_rows", [1, 7, 64, 500, 5000])
def test_tiled_equals_oracle_bit_for_bit(cuda_lib, Nd, panel_rows):
    p = G.random_csr(700, 900, Nd, 0.03, seed=Nd + panel_rows)
    want = oracle.spmm(*arrays(p), fused=True, threads=4)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = ops.spmm_tiled(*(dev(x) for x in arrays(p)), panel_rows=panel_rows, status_word=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert np.array_equal(got.cpu().numpy(), want)


@pytest.mark.parametrize("alpha,beta", [(1.0, 0.5), (2.0, -1.0), (0.0, 0.75), (-0.5, 0.0)])
def test_tiled_alpha_beta_keep_c_old_until_the_last_pass(cuda_lib, alpha, beta):
    p = G.random_csr(1200, 800, 96, 0.02, seed=3)
    C0 = np.random.default_rng(1).standard_normal((p.M, p.Nd)).astype(np.float32)
    want = oracle.spmm(*arrays(p), C0.copy(), alpha, beta, fused=True, threads=4)
    Cd = dev(C0)
    ops.spmm_tiled(*(dev(x) for x in arrays(p)), Cd, alpha, beta, panel_rows=100)
    assert np.array_equal(Cd.cpu().numpy(), want)
    # and with padded leading dimensions (ldb, ldc > Nd); the padding of C is left alone
    Bp = torch.zeros(p.Kd, p.Nd + 4, device="cuda")
    Bp[:, :p.Nd] = dev(p.B)
    Cp = torch.full((p.M, p.Nd + 8), 9.0, device="cuda")
    Cp[:, :p.Nd] = dev(C0)
    ops.spmm_tiled(dev(p.row_ptr), dev(p.col_idx), dev(p.values), Bp[:, :p.Nd], Cp[:, :p.Nd], alpha, beta, panel_rows=100)
    assert np.array_equal(Cp[:, :p.Nd].cpu().numpy(), want) and bool((Cp[:, p.Nd:] == 9.0).all())


def test_tiled_unsorted_repeated_columns_empty_and_long_rows(cuda_lib):
    """Stored order is taken as it comes: an entry is consumed by the first pass that reaches it."""
    rng = np.random.default_rng(8)
    lens = np.where(rng.random(2000) < 0.3, 0, rng.integers(1, 40, 2000))
    lens[17], lens[1999] = 3000, 1500
    p = G.random_csr(2000, 4000, 64, 0.0, seed=5, lengths=lens)
    ci = p.col_idx.copy()
    for r in range(0, 2000, 3):  # shuffle every third row, plant repeats
        s, e = p.row_ptr[r], p.row_ptr[r + 1]
        if e - s > 2:
            seg = ci[s:e]
            rng.shuffle(seg)
            seg[1] = seg[0]
    want = oracle.spmm(p.row_ptr, ci, p.values, p.B, fused=True, threads=4)
    for panel_rows in (128, 1000, 10_000):
        got = ops.spmm_tiled(dev(p.row_ptr), dev(ci), dev(p.values), dev(p.B), panel_rows=panel_rows)
        assert np.array_equal(got.cpu().numpy(), want)


def test_tiled_matches_row_kernel_on_packed_values_and_a_row_block(cuda_lib):
    p = G.make("cfg4_fp4", scale=32)
    packed, scale = ops.e2m1_quantize(p.values)
    rp, ci, B = dev(p.row_ptr), dev(p.col_idx), dev(p.B)
    want = ops.spmm(rp, ci, packed.cuda(), B, kernel="row", e2m1_scale=scale, nnz=p.nnz, sync=True)
    got = ops.spmm_tiled(rp, ci, packed.cuda(), B, panel_rows=300, e2m1_scale=scale, nnz=p.nnz)
    assert torch.equal(got, want)
    # rows [r0, r1) of the matrix through offset pointers (args.row_ptr_base), C ABI directly
    va = dev(p.values)
    whole = ops.spmm(rp, ci, va, B, kernel="row", sync=True)
    r0, r1 = 100, 1500
    j0, j1 = int(p.row_ptr[r0]), int(p.row_ptr[r1])
    out = torch.zeros(r1 - r0, p.Nd, device="cuda")
    a = _lib.make_args(r1 - r0, p.Kd, p.Nd, j1 - j0, rp.data_ptr() + 4 * r0, ci.data_ptr() + 4 * j0,
                       va.data_ptr() + 4 * j0, B.data_ptr(), out.data_ptr(), row_ptr_base=j0)
    assert cuda_lib.csrspmm_b200_spmm_tiled(C.byref(a), 256, None) == _lib.OK, cuda_lib.csrspmm_b200_last_error()
    torch.cuda.synchronize()
    assert torch.equal(out, whole[r0:r1])


def test_tiled_workspace_and_argument_errors(cuda_lib):
    p = G.random_csr(300, 400, 32, 0.05, seed=2)
    t = [dev(x) for x in arrays(p)]
    out = torch.zeros(p.M, p.Nd, device="cuda")
    a = _lib.make_args(p.M, p.Kd, p.Nd, p.nnz, *(x.data_ptr() for x in t), out.data_ptr(), beta=0.5)
    need = cuda_lib.csrspmm_b200_tiled_workspace_bytes(C.byref(a))
    assert need >= (p.M + 1) * 4 + p.M * p.Nd * 4
    small = torch.empty(256, dtype=torch.uint8, device="cuda")
    a.workspace, a.workspace_bytes = small.data_ptr(), 256
    assert cuda_lib.csrspmm_b200_spmm_tiled(C.byref(a), 50, None) == _lib.ERR_WORKSPACE
    assert cuda_lib.csrspmm_b200_spmm_tiled(C.byref(a), -1, None) == _lib.ERR_BAD_ARG
    assert ops.tiled_panel_rows(1 << 22, 512) == 32768 and ops.tiled_panel_rows(1000, 512) == 0
    # a malformed column index is clamped and reported, never dereferenced
    bad = t[1].clone()
    bad[5] = 10 ** 6
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.spmm_tiled(t[0], bad, t[2], t[3], panel_rows=64, status_word=status)
    torch.cuda.synchronize()
    assert int(status.item()) & 2
