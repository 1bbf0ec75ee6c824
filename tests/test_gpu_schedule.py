"""The product under a per-matrix schedule (csrspmm_b200_schedule_create + args.schedule) against the
CPU oracle and against the unscheduled kernels, through the C ABI.

Tolerances: a long row is a fixed-order sum of sequential piece sums, so it is judged like the rows
the merge-path kernel cuts: |err| <= 1e-5 * sum|a*b| + 1e-6 against the fp64 oracle; a long row that
fits one piece, and every row the schedule leaves to the merge-path kernel's lane groups whole, equals
the sequential fp32 oracle bit for bit.  Two runs are bit-identical (no atomics).
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from csrspmm_b200 import _lib, generators as G, ops

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 1e-6


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def skewed(M, Kd, Nd, seed, mean=12.0, cap=None, vlo=-1.0, vhi=1.0):
    lens = G.zipf_lengths(np.random.default_rng(seed), M, Kd, 2.0, mean, cap or Kd // 2)
    return G.from_lengths("skewed", lens, Kd, Nd, np.random.default_rng(seed + 1), vlo, vhi, seed)


def check(got, p, C0=None, alpha=1.0, beta=0.0):
    f64, mag = oracle.spmm_f64(p.row_ptr, p.col_idx, p.values, p.B, C0, alpha, beta, threads=4)
    err = np.abs(got.astype(np.float64) - f64)
    assert (err <= RTOL * mag + ATOL).all(), f"worst excess {(err - RTOL * mag - ATOL).max()}"


def run(p, sched, C0=None, alpha=1.0, beta=0.0, kernel="auto", values=None, **kw):
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.spmm(dev(p.row_ptr), dev(p.col_idx), dev(p.values) if values is None else values, dev(p.B),
                   dev(C0) if C0 is not None else None, alpha, beta, kernel=kernel, status_word=status, sync=True,
                   schedule=sched, **kw)
    assert int(status.item()) == 0
    return out.cpu().numpy()


@pytest.mark.parametrize("Nd", [4, 7, 64, 128, 256, 520])
def test_scheduled_product_matches_the_oracle(cuda_lib, Nd):
    """Several slabs, several pieces per slab, rows on both sides of the threshold, empty rows."""
    p = skewed(3000, 4096, Nd, seed=Nd)
    lens = np.diff(p.row_ptr)
    lens_h = lens
    rp, ci = dev(p.row_ptr), dev(p.col_idx)
    s = ops.Schedule(rp, ci, p.Kd, Nd, threshold=24, slab_rows=512, piece_nnz=16)
    info = s.info()
    assert info["num_slabs"] == 8 and info["long_rows"] == int((lens_h >= 24).sum()) and info["columns_sorted"] == 1
    assert info["long_nnz"] == int(lens_h[lens_h >= 24].sum()) and info["pieces"] >= info["long_rows"]
    got = run(p, s)
    check(got, p)
    want = oracle.spmm(p.row_ptr, p.col_idx, p.values, p.B, fused=True, threads=4)
    assert np.isclose(got, want, rtol=RTOL, atol=ATOL).mean() > 0.99
    assert np.array_equal(got, run(p, s))  # fixed summation order
    C0 = np.random.default_rng(5).standard_normal((p.M, Nd), dtype=np.float32)
    check(run(p, s, C0, 1.5, 0.5), p, C0, 1.5, 0.5)
    check(run(p, s, C0, -0.25, 1.0, kernel="merge"), p, C0, -0.25, 1.0)


def test_single_piece_long_rows_are_sequential_sums(cuda_lib):
    """One slab boundary never reached and pieces longer than any row: each long row is one piece, i.e. the
    oracle's sequential fp32 sum."""
    lens = np.full(512, 3, np.int64)
    lens[::7] = 150
    p = G.from_lengths("hubs", lens, 1 << 14, 64, np.random.default_rng(3), -1.0, 1.0, 3)
    p.col_idx[:] = p.col_idx % 4000  # keeps every column inside slab 0 ...
    for r in range(p.M):  # ... and ascending, distinct
        a, b = p.row_ptr[r], p.row_ptr[r + 1]
        p.col_idx[a:b] = np.sort(np.random.default_rng(r).choice(4000, b - a, replace=False))
    s = ops.Schedule(dev(p.row_ptr), dev(p.col_idx), p.Kd, 64, threshold=100, slab_rows=4096, piece_nnz=256)
    assert s.info()["long_rows"] == len(lens[lens >= 100]) and s.info()["pieces"] == s.info()["long_rows"]
    got = run(p, s)
    want = oracle.spmm(p.row_ptr, p.col_idx, p.values, p.B, fused=True, threads=4)
    assert np.array_equal(got[lens >= 100], want[lens >= 100])
    check(got, p)


def test_hub_rows_and_tile_boundaries(cuda_lib):
    """Hub rows far longer than a merge-path tile (tiles wholly inside a scheduled row do nothing), next to
    rows of one entry and empty rows."""
    lens = np.zeros(4000, np.int64)
    lens[1::3] = 1
    lens[2::3] = 5
    lens[[0, 17, 1999, 3999]] = [9000, 70000, 4097, 12345]
    p = G.from_lengths("hubs", lens, 1 << 18, 64, np.random.default_rng(11), 0.0, 1.0, 11)
    s = ops.Schedule(dev(p.row_ptr), dev(p.col_idx), p.Kd, 64, threshold=1000, slab_rows=1 << 14, piece_nnz=64)
    assert s.info()["long_rows"] == 4
    got = run(p, s)
    check(got, p)
    assert np.array_equal(got, run(p, s))
    assert (got[lens == 0] == 0).all()


def test_packed_e2m1_values_under_a_schedule(cuda_lib):
    p = skewed(2048, 8192, 128, seed=21)
    packed, scale = ops.e2m1_quantize(p.values)
    decoded = oracle.e2m1_decode(packed.numpy(), p.nnz, scale)
    s = ops.Schedule(dev(p.row_ptr), dev(p.col_idx), p.Kd, 128, threshold=20, slab_rows=1024, piece_nnz=32)
    assert s.active
    got4 = run(p, s, values=packed.cuda(), e2m1_scale=scale, nnz=p.nnz)
    got = run(p, s, values=dev(decoded))
    assert np.array_equal(got4, got)  # identical in decoded operands
    f64, mag = oracle.spmm_f64(p.row_ptr, p.col_idx, decoded, p.B, threads=4)
    assert (np.abs(got4 - f64) <= 1e-4 * mag + 1e-6).all()


def test_schedule_is_empty_when_it_cannot_help(cuda_lib):
    p = skewed(1024, 2048, 64, seed=2)
    rp, ci = dev(p.row_ptr), dev(p.col_idx)
    one_slab = ops.Schedule(rp, ci, p.Kd, 64)  # B = 512 KiB: one slab
    assert not one_slab.active and one_slab.info()["device_bytes"] == 0
    none_long = ops.Schedule(rp, ci, p.Kd, 64, threshold=1 << 20, slab_rows=256)
    assert not none_long.active
    # unsorted columns inside a long row: the schedule comes back empty, the product is still right
    ci_bad = p.col_idx.copy()
    r = int(np.argmax(np.diff(p.row_ptr)))
    a = p.row_ptr[r]
    ci_bad[a], ci_bad[a + 1] = ci_bad[a + 1], ci_bad[a]
    unsorted = ops.Schedule(rp, dev(ci_bad), p.Kd, 64, threshold=16, slab_rows=256)
    assert not unsorted.active and unsorted.info()["columns_sorted"] == 0
    for s in (one_slab, none_long):
        check(run(p, s), p)


def test_schedule_argument_checks(cuda_lib):
    p = skewed(1024, 4096, 64, seed=4)
    rp, ci, va, B = dev(p.row_ptr), dev(p.col_idx), dev(p.values), dev(p.B)
    s = ops.Schedule(rp, ci, p.Kd, 64, threshold=16, slab_rows=512)
    assert s.active
    with pytest.raises(_lib.SpmmError) as e:  # another matrix
        ops.spmm(rp[:-1].contiguous(), ci, va, B, schedule=s)
    assert e.value.status == _lib.ERR_BAD_ARG
    with pytest.raises(_lib.SpmmError) as e:  # a pinned kernel that cannot honour it
        ops.spmm(rp, ci, va, B, schedule=s, kernel="row")
    assert e.value.status == _lib.ERR_BAD_ARG
    L = _lib.lib()
    a = _lib.make_args(p.M, p.Kd, 64, p.nnz, rp.data_ptr(), ci.data_ptr(), va.data_ptr(), B.data_ptr(),
                       torch.empty(p.M, 64, device="cuda").data_ptr(), schedule=s.handle)
    need = L.csrspmm_b200_workspace_bytes(C.byref(a))
    a.schedule = None
    assert need > L.csrspmm_b200_workspace_bytes(C.byref(a))  # the slots come on top of the carries
    a.schedule = s.handle
    small = torch.empty(need - 256, dtype=torch.uint8, device="cuda")
    a.workspace, a.workspace_bytes = small.data_ptr(), small.numel()
    assert L.csrspmm_b200_spmm(C.byref(a), None) == _lib.ERR_WORKSPACE
    bad = _lib.ScheduleOptions(4, 0, 0, 0)
    h = C.c_void_p(None)
    assert L.csrspmm_b200_schedule_create(C.byref(a), C.byref(bad), C.byref(h), None) == _lib.ERR_BAD_ARG
    info = _lib.ScheduleInfo()
    assert L.csrspmm_b200_schedule_info_get(C.c_void_p(s.handle), C.byref(info)) == _lib.ERR_BAD_ARG  # struct_size unset
    s.close()
    s.close()  # idempotent


def test_prepared_call_with_a_schedule(cuda_lib):
    p = skewed(4096, 8192, 64, seed=9)
    rp, ci, va, B = dev(p.row_ptr), dev(p.col_idx), dev(p.values), dev(p.B)
    s = ops.Schedule(rp, ci, p.Kd, 64, threshold=16, slab_rows=1024, piece_nnz=32)
    out = torch.empty(p.M, 64, device="cuda")
    call = ops.SpmmCall(rp, ci, va, B, out, schedule=s)
    assert call.kernel == "scheduled" and call.launches == 4
    call()
    torch.cuda.synchronize()
    check(out.cpu().numpy(), p)
    first = out.clone()
    call()
    torch.cuda.synchronize()
    assert torch.equal(first, out)


def test_scheduled_product_replayed_from_a_stream_capture(cuda_lib):
    """The pieces kernel hands out work from a counter in the call's scratch; the memset that zeroes it is part
    of the product, so a captured product can be replayed any number of times."""
    p = skewed(4096, 8192, 128, seed=10)
    rp, ci, va, B = dev(p.row_ptr), dev(p.col_idx), dev(p.values), dev(p.B)
    s = ops.Schedule(rp, ci, p.Kd, 128, threshold=16, slab_rows=1024, piece_nnz=32)
    out = torch.empty(p.M, 128, device="cuda")
    call = ops.SpmmCall(rp, ci, va, B, out, schedule=s)
    call()
    torch.cuda.synchronize()
    eager = out.clone()
    g, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            call()
    for _ in range(3):
        out.fill_(float("nan"))
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager)


def test_even_rows_keep_the_whole_row_kernel(cuda_lib):
    """With AUTO and a longest row known to be close to the mean, the whole-row kernel is the better choice and
    a schedule is left aside; csrspmm_b200_select_kernel says which way a call will go."""
    p = G.random_csr(2000, 8192, 64, 0.0, seed=3, lengths=np.full(2000, 40))
    rp, ci, va, B = dev(p.row_ptr), dev(p.col_idx), dev(p.values), dev(p.B)
    s = ops.Schedule(rp, ci, p.Kd, 64, threshold=16, slab_rows=1024)
    assert s.active
    out = torch.empty(p.M, 64, device="cuda")
    assert ops.SpmmCall(rp, ci, va, B, out, schedule=s).kernel == "scheduled"  # row lengths unknown
    known = ops.SpmmCall(rp, ci, va, B, out, schedule=s, max_row_nnz=40)
    assert known.kernel == "row" and known.launches == 1
    known()
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), oracle.spmm(p.row_ptr, p.col_idx, p.values, p.B, fused=True, threads=4))
    assert ops.SpmmCall(rp, ci, va, B, out, schedule=s, max_row_nnz=40, kernel="merge").kernel == "scheduled"


def test_csr_matrix_keeps_its_schedules(cuda_lib):
    from csrspmm_b200.torch_library import CsrMatrix
    p = skewed(4096, 8192, 320, seed=31, mean=40.0)
    A = CsrMatrix(dev(p.row_ptr), dev(p.col_idx), dev(p.values), (p.M, p.Kd))
    assert A.schedule(320) is None and A.schedule(320) is None  # B of 10 MB: one slab, nothing to schedule; asked once
    got = (A @ dev(p.B)).cpu().numpy()
    check(got, p)


def test_cfg3_powerlaw_full_size_under_its_schedule(cuda_lib):
    """BASELINE config 3 at full size under a schedule (threshold given: for rows of B this narrow the
    library would schedule nothing by itself): oracle on a row sample (random rows and the longest ones), row
    sums through an all-ones B over every row, linearity, determinism."""
    from test_gpu_parity import _check_sampled_rows, _sample
    p = G.make("cfg3_powerlaw", device="cuda")
    rp_h = p.row_ptr.cpu().numpy()
    assert not ops.Schedule(p.row_ptr, p.col_idx, p.Kd, p.Nd).active  # 256-byte rows: not worth it
    s = ops.Schedule(p.row_ptr, p.col_idx, p.Kd, p.Nd, threshold=64, slab_rows=(32 << 20) // 256)
    info = s.info()
    assert s.active and info["num_slabs"] == 8 and info["long_nnz"] > p.nnz // 3
    Cd = ops.spmm(p.row_ptr, p.col_idx, p.values, p.B, sync=True, schedule=s)
    rate = _check_sampled_rows(rp_h, p.col_idx, p.values, p.B, Cd, _sample(rp_h, np.random.default_rng(0)))
    assert rate > 0.999
    C2 = ops.spmm(p.row_ptr, p.col_idx, p.values, p.B, None, 2.0, sync=True, schedule=s)
    assert torch.equal(C2, 2.0 * Cd)
    ones = torch.ones(p.Kd, 64, device="cuda")
    Cs = ops.spmm(p.row_ptr, p.col_idx, p.values, ones, sync=True, schedule=s)
    csum = torch.zeros(p.nnz + 1, dtype=torch.float64, device="cuda")
    csum[1:] = torch.cumsum(p.values.double(), 0)
    rowsum = csum[p.row_ptr[1:].long()] - csum[p.row_ptr[:-1].long()]
    assert torch.allclose(Cs[:, 0].double(), rowsum, rtol=1e-5, atol=1e-4)
    assert torch.equal(Cs[:, :1].expand(-1, 64), Cs)
    assert torch.equal(Cd, ops.spmm(p.row_ptr, p.col_idx, p.values, p.B, sync=True, schedule=s))
    # the rows the schedule does not cover are the merge-path kernel's own, bit for bit
    plain = ops.spmm(p.row_ptr, p.col_idx, p.values, p.B, kernel="merge", sync=True)
    short = torch.from_numpy(np.diff(rp_h) < info["long_row_threshold"]).cuda()
    assert torch.equal(Cd[short], plain[short])


def test_cfg5_xl_eighth_size_under_the_librarys_own_schedule(cuda_lib):
    """BASELINE config 5's row-length law and width (Zipf 2.2, mean 32, Nd 512) on 2^19 rows, with the
    threshold, slab and piece length the library picks for 2 KB rows of B."""
    from test_gpu_parity import _check_sampled_rows, _sample
    p = G.make("cfg5_xl", scale=8, device="cuda")
    rp_h = p.row_ptr.cpu().numpy()
    s = ops.Schedule(p.row_ptr, p.col_idx, p.Kd, p.Nd)
    info = s.info()
    assert s.active and info["num_slabs"] == 16 and info["long_row_threshold"] == 128, info  # 8 entries per slab
    Cd = ops.spmm(p.row_ptr, p.col_idx, p.values, p.B, sync=True, schedule=s)
    rate = _check_sampled_rows(rp_h, p.col_idx, p.values, p.B, Cd, _sample(rp_h, np.random.default_rng(1), 4000, 32))
    assert rate > 0.999
    assert torch.equal(Cd, ops.spmm(p.row_ptr, p.col_idx, p.values, p.B, sync=True, schedule=s))
    plain = ops.spmm(p.row_ptr, p.col_idx, p.values, p.B, kernel="merge", sync=True)
    short = torch.from_numpy(np.diff(rp_h) < info["long_row_threshold"]).cuda()
    assert torch.equal(Cd[short], plain[short])


def test_results_do_not_depend_on_which_warp_sums_a_piece(cuda_lib):
    """The pieces are drawn from a ticket counter by whichever warp is free: the draw changes from run to run, no
    sum may."""
    p = skewed(3000, 4096, 64, seed=11, mean=24.0)
    rp, ci, va, B = dev(p.row_ptr), dev(p.col_idx), dev(p.values), dev(p.B)
    sched = ops.Schedule(rp, ci, p.Kd, p.Nd, threshold=32, slab_rows=128, piece_nnz=16)
    assert sched.active
    first = ops.spmm(rp, ci, va, B, schedule=sched, sync=True)
    for _ in range(5):
        assert torch.equal(first, ops.spmm(rp, ci, va, B, schedule=sched, sync=True))
    check(first.cpu().numpy(), p)


@pytest.mark.parametrize("seed", range(8))
def test_random_schedules_match_the_oracle(cuda_lib, seed):
    """Random sizes, widths and schedule parameters (few pieces, many pieces, more pieces than the persistent
    grid has warps, pieces of one entry): every combination against the fp64 oracle and against itself."""
    rng = np.random.default_rng(100 + seed)
    M = int(rng.integers(50, 6000))
    Kd = int(rng.integers(600, 9000))
    Nd = int(rng.choice([1, 4, 12, 32, 64, 100, 128, 256, 516]))
    p = skewed(M, Kd, Nd, seed=200 + seed, mean=float(rng.uniform(4, 40)), cap=Kd)
    threshold = int(rng.choice([2, 8, 33, 200]))
    slab_rows = int(rng.choice([256, 300, 1024, 4096]))
    piece = int(rng.choice([1, 3, 16, 64, 500]))
    rp, ci = dev(p.row_ptr), dev(p.col_idx)
    sched = ops.Schedule(rp, ci, p.Kd, p.Nd, threshold=threshold, slab_rows=slab_rows, piece_nnz=piece)
    C0 = rng.standard_normal((p.M, p.Nd), dtype=np.float32)
    got = run(p, sched if sched.active else None, C0=C0, alpha=0.75, beta=-0.5)
    check(got, p, C0=C0, alpha=0.75, beta=-0.5)
    assert np.array_equal(got, run(p, sched if sched.active else None, C0=C0, alpha=0.75, beta=-0.5))
