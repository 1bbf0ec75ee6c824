"""Failure detection on the device without a fault: the bulk-copy kernel's bounded waits.

Every wait on a row copy in spmm_tma_kernel is bounded.  Here the bound of the first wait is set to
zero attempts (CSRSPMM_TEST_WAIT_LIMIT, a test hook read by the C ABI), so every warp that has a row
in flight "times out" at once: it must report the timeout in the status word, wait (with the full
bound) for the copies it had started, publish nothing, and return.  Nothing hangs, traps or faults,
the context stays usable, and csrspmm_b200_spmm_sync turns the status word into ERR_DEVICE_WAIT.
"""
import numpy as np
import pytest
import torch

import oracle
from csrspmm_b200 import _lib, generators as G, ops

pytestmark = pytest.mark.gpu


def _dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


@pytest.mark.parametrize("Nd", [64, 512])
def test_wait_that_runs_out_is_reported_and_leaves_the_context_usable(cuda_lib, monkeypatch, Nd):
    p = G.make("cfg3_powerlaw", scale=256, Nd=Nd)
    rp, ci, va, B = (_dev(x) for x in (p.row_ptr, p.col_idx, p.values, p.B))
    good = ops.spmm(rp, ci, va, B, kernel="tma", sync=True)

    monkeypatch.setenv("CSRSPMM_TEST_WAIT_LIMIT", "0")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    C = torch.full((p.M, Nd), 7.0, device="cuda")
    with pytest.raises(_lib.SpmmError) as e:
        ops.spmm(rp, ci, va, B, C, 1.0, 0.0, kernel="tma", status_word=status, sync=True)
    assert e.value.status == _lib.ERR_DEVICE_WAIT
    assert int(status.item()) & 4  # kStatusWaitTimeout
    torch.cuda.synchronize()  # the context is alive: no sticky error
    # a warp that gave up wrote nothing: rows whose entries all lay with such warps still hold the fill
    lens = np.diff(p.row_ptr)
    untouched = (C == 7.0).all(dim=1).cpu().numpy()
    assert untouched[lens > 0].mean() > 0.9
    # the asynchronous entry point reports nothing by itself; the status word does
    status.zero_()
    ops.spmm(rp, ci, va, B, C, 1.0, 0.0, kernel="tma", status_word=status)
    torch.cuda.synchronize()
    assert int(status.item()) & 4

    monkeypatch.delenv("CSRSPMM_TEST_WAIT_LIMIT")
    status.zero_()
    again = ops.spmm(rp, ci, va, B, kernel="tma", status_word=status, sync=True)
    assert int(status.item()) == 0
    assert torch.equal(again, good)
    f64, mag = oracle.spmm_f64(p.row_ptr, p.col_idx, p.values, p.B, threads=4)
    assert (np.abs(again.cpu().numpy() - f64) <= 1e-5 * mag + 1e-6).all()


def test_host_round_trip_reports_the_timeout_too(cuda_lib, monkeypatch):
    p = G.make("cfg3_powerlaw", scale=512, Nd=128)
    h = [torch.from_numpy(np.ascontiguousarray(x)) for x in (p.row_ptr, p.col_idx, p.values, p.B)]
    C_host = torch.zeros(p.M, p.Nd)
    monkeypatch.setenv("CSRSPMM_TEST_WAIT_LIMIT", "0")
    with pytest.raises(_lib.SpmmError) as e:
        ops.spmm_host(*h, C_host, kernel="tma")
    assert e.value.status == _lib.ERR_DEVICE_WAIT
    monkeypatch.delenv("CSRSPMM_TEST_WAIT_LIMIT")
    ops.spmm_host(*h, C_host, kernel="tma")
    f64, mag = oracle.spmm_f64(p.row_ptr, p.col_idx, p.values, p.B, threads=4)
    assert (np.abs(C_host.numpy() - f64) <= 1e-5 * mag + 1e-6).all()
