"""csrspmm_b200_spmm_noalloc -- the entry point for hosts that cannot allocate device memory when
they call (their memory manager owns the whole GPU, or their runtime forbids allocation calls):
the merge-path SpMM with its scratch in a fixed array inside the library.  Checked against the
ordinary entry point (bit for bit: same kernel, same tiles, same summation order) and against the
CPU oracle on back-to-back calls that share that array, plus the size limit.

Collected last on purpose (file name), so a run that stops at the first failure has already run
every other test; it does not depend on them and passes in a fresh process too."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from csrspmm_b200 import _lib, generators as G, ops

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-5, 1e-6


def _dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def _args(p, t, C_out, alpha, beta, **kw):
    return _lib.make_args(p.M, p.Kd, p.Nd, p.nnz, t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(),
                          C_out.data_ptr(), alpha=alpha, beta=beta, **kw)


def test_noalloc_matches_the_ordinary_entry_point_twice_in_a_row(cuda_lib):
    L = cuda_lib
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # two different problems, both with rows long enough to be split across CTAs (carries in use);
    # the second is wider and smaller, so it reuses the front of the array the first one filled
    probs = [G.make("cfg3_powerlaw", scale=32), G.random_csr(300, 9000, 256, 0.0, seed=77,
                                                             lengths=np.r_[np.full(6, 4000), np.arange(294) % 23])]
    work = []
    for i, p in enumerate(probs):
        t = [_dev(x) for x in (p.row_ptr, p.col_idx, p.values, p.B)]
        C0 = np.random.default_rng(i).standard_normal((p.M, p.Nd), dtype=np.float32)
        want, got = _dev(C0), _dev(C0)
        ws = torch.empty(int(L.csrspmm_b200_workspace_bytes(C.byref(_args(p, t, want, 1.0, 0.0)))), dtype=torch.uint8,
                         device="cuda")
        ref_args = _args(p, t, want, 1.25, 0.5, kernel=_lib.KERNEL_MERGE, workspace=ws.data_ptr(),
                         workspace_bytes=ws.numel())
        assert L.csrspmm_b200_spmm(C.byref(ref_args), stream) == _lib.OK, L.csrspmm_b200_last_error()
        work.append((p, t, want, got, ws))
    torch.cuda.synchronize()
    # the two no-alloc calls, one right after the other on the same stream, no host sync between
    for p, t, want, got, ws in work:
        st = L.csrspmm_b200_spmm_noalloc(C.byref(_args(p, t, got, 1.25, 0.5)), stream)
        assert st == _lib.OK, L.csrspmm_b200_last_error()
    torch.cuda.synchronize()
    for i, (p, t, want, got, ws) in enumerate(work):
        assert torch.isfinite(got).all()
        assert torch.equal(got, want), float((got - want).abs().max())  # same kernel, same tiles, same order
        C0 = np.random.default_rng(i).standard_normal((p.M, p.Nd), dtype=np.float32)
        f64, mag = oracle.spmm_f64(p.row_ptr, p.col_idx, p.values, p.B, C0, 1.25, 0.5, threads=4)
        assert (np.abs(got.cpu().numpy() - f64) <= RTOL * mag + ATOL).all()


@pytest.mark.parametrize("case", ["ragged_width", "several_column_passes", "packed_e2m1"])
def test_noalloc_on_other_layouts(cuda_lib, case):
    """A dense width that is not a multiple of 4 (scalar instantiation), one above 512 (several passes over
    the columns, carries as wide as the row) and packed 4-bit values: bit-identical to the ordinary merge
    call and within the accumulation-order bound of the oracle."""
    L = cuda_lib
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    Nd = {"ragged_width": 30, "several_column_passes": 1040, "packed_e2m1": 128}[case]
    p = G.random_csr(400, 6000, Nd, 0.0, seed=Nd, lengths=np.r_[np.full(3, 3000), np.arange(397) % 40])
    values = p.values
    kw = {}
    t = [_dev(x) for x in (p.row_ptr, p.col_idx, p.values, p.B)]
    if case == "packed_e2m1":
        packed, scale = ops.e2m1_quantize(p.values)
        values = oracle.e2m1_decode(packed.numpy(), p.nnz, scale)
        t[2] = packed.cuda()
        kw = dict(value_format=_lib.VALUES_E2M1, value_scale=scale)
    want = torch.empty(p.M, Nd, device="cuda")
    got = torch.empty(p.M, Nd, device="cuda")
    ws = torch.empty(int(L.csrspmm_b200_workspace_bytes(C.byref(_args(p, t, want, 1.0, 0.0)))), dtype=torch.uint8, device="cuda")
    ref_args = _args(p, t, want, 0.75, 0.0, kernel=_lib.KERNEL_MERGE, workspace=ws.data_ptr(), workspace_bytes=ws.numel(), **kw)
    assert L.csrspmm_b200_spmm(C.byref(ref_args), stream) == _lib.OK, L.csrspmm_b200_last_error()
    for _ in range(2):  # the second call finds the first one's carries in the array
        assert L.csrspmm_b200_spmm_noalloc(C.byref(_args(p, t, got, 0.75, 0.0, **kw)), stream) == _lib.OK, L.csrspmm_b200_last_error()
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    f64, mag = oracle.spmm_f64(p.row_ptr, p.col_idx, values, p.B, None, 0.75, 0.0, threads=4)
    assert (np.abs(got.cpu().numpy() - f64) <= RTOL * mag + ATOL).all()


def test_noalloc_on_every_visible_device(cuda_lib):
    """The array's address is looked up per device: the call works on each GPU of the box, not only device 0."""
    L = cuda_lib
    p = G.make("cfg3_powerlaw", scale=256)
    for d in range(torch.cuda.device_count()):
        with torch.cuda.device(d):
            t = [torch.from_numpy(np.ascontiguousarray(x)).cuda(d) for x in (p.row_ptr, p.col_idx, p.values, p.B)]
            got = torch.empty(p.M, p.Nd, device=f"cuda:{d}")
            stream = C.c_void_p(torch.cuda.current_stream(d).cuda_stream)
            assert L.csrspmm_b200_spmm_noalloc(C.byref(_args(p, t, got, 1.0, 0.0)), stream) == _lib.OK, L.csrspmm_b200_last_error()
            torch.cuda.synchronize(d)
            f64, mag = oracle.spmm_f64(p.row_ptr, p.col_idx, p.values, p.B, threads=4)
            assert (np.abs(got.cpu().numpy() - f64) <= RTOL * mag + ATOL).all()


def test_noalloc_refuses_problems_beyond_its_array(cuda_lib):
    L = cuda_lib
    p = G.random_csr(64, 64, 512, 0.1, seed=5)
    t = [_dev(x) for x in (p.row_ptr, p.col_idx, p.values, p.B)]
    out = torch.zeros(p.M, p.Nd, device="cuda")
    a = _args(p, t, out, 1.0, 0.0)
    a.M, a.nnz = 64, 40_000_000  # sizes only: the call is refused before anything is read or launched
    assert L.csrspmm_b200_workspace_bytes(C.byref(a)) > _lib.NOALLOC_SCRATCH_BYTES
    assert L.csrspmm_b200_spmm_noalloc(C.byref(a), None) == _lib.ERR_WORKSPACE
    msg = L.csrspmm_b200_last_error().decode()
    assert str(_lib.NOALLOC_SCRATCH_BYTES) in msg and "scratch" in msg
    torch.cuda.synchronize()
    assert not out.any()
