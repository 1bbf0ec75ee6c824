"""This library against the reference's OWN GPU kernels, recompiled for sm_100a from the reference
checkout (oracle/_ref/libcsrspmm_ref_gpu.so, see oracle/Makefile target refgpu), on the same device
buffers.  Skipped when that library was not built.

Bit-level expectation: with alpha = 1 and beta = 0 the reference kernels and the row kernel do the
same thing per output element -- one fp32 accumulator, fused multiply-adds in stored order -- so
they must agree exactly.  With other alpha/beta the reference's epilogue may be contracted by its
compiler, and the split kernels re-associate rows they cut: those are held to the
accumulation-order tolerance (rtol 1e-5 / atol 1e-6, or the fp64-magnitude bound for cut rows).

Set CSRSPMM_TIMING_OUT=<file> to also write a timing table (reference kernels vs this library).
"""
import json
import os

import numpy as np
import pytest
import torch

import oracle
from csrspmm_b200 import generators as G, ops

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not oracle.ReferenceGpu.available(),
                                 reason="reference GPU kernels not built (needs the reference checkout)")]

REF_ALGOS = ["Naive", "WarpPerRow", "WarpPerRowFp4", "WarpPerRowSmem", "WarpPerRowSmemFp4"]


def _dev(p):
    return [torch.from_numpy(x).cuda() for x in (p.row_ptr, p.col_idx, p.values, p.B)]


def _problems():
    yield "cfg1_check", G.make("cfg1_check")
    yield "cfg2_medium", G.make("cfg2_medium")
    yield "cfg4_fp4/16", G.make("cfg4_fp4", scale=16)
    yield "cfg3_powerlaw/64", G.make("cfg3_powerlaw", scale=64)
    yield "test_pytorch 256x64x16", G.random_csr(256, 64, 16, 0.3, seed=2, vlo=0.0, vhi=1.0)
    yield "ragged 203x150x100", G.random_csr(203, 150, 100, 0.08, seed=3)


@pytest.mark.parametrize("name,p", list(_problems()), ids=[n for n, _ in _problems()])
def test_results_equal_the_reference_kernels(cuda_lib, name, p):
    ref = oracle.ReferenceGpu()
    rp, ci, va, B = _dev(p)
    mx = int(np.diff(p.row_ptr).max())
    f64, mag = oracle.spmm_f64(p.row_ptr, p.col_idx, p.values, p.B, threads=4)
    ours = {k: ops.spmm(rp, ci, va, B, kernel=k, sync=True) for k in ("row", "merge")}
    if p.Nd % 4 == 0 and p.Nd <= 512:
        ours["tma"] = ops.spmm(rp, ci, va, B, kernel="tma", sync=True)
    ran = 0
    for algo in REF_ALGOS:
        C_ref = torch.full((p.M, p.Nd), float("nan"), device="cuda")
        rc = ref.spmm(algo, rp, ci, va, B, C_ref, 1.0, 0.0, mx)
        if rc == -2:
            continue  # shape outside what this reference kernel can launch
        assert rc == 0
        torch.cuda.synchronize()
        ran += 1
        assert torch.equal(ours["row"], C_ref), f"{algo}: row kernel differs, max {float((ours['row'] - C_ref).abs().max())}"
        for k in ("merge", "tma"):
            if k in ours:
                err = (ours[k] - C_ref).abs().cpu().numpy()
                assert (err <= 2 * (1e-5 * mag + 1e-6)).all(), f"{algo} vs {k}"
    assert ran >= 3
    # alpha, beta != (1, 0): C is read and scaled
    C0 = torch.randn(p.M, p.Nd, device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    C_ref, C_our = C0.clone(), C0.clone()
    assert ref.spmm("WarpPerRow", rp, ci, va, B, C_ref, 1.5, 0.5, mx) == 0
    ops.spmm(rp, ci, va, B, C_our, 1.5, 0.5, kernel="row", sync=True)
    assert torch.allclose(C_our, C_ref, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("scale", [16, 1])
def test_packed_e2m1_against_the_reference_fp4_kernels(cuda_lib, scale):
    """BASELINE config 4 (full size and 1/16): values quantised with this library's e2m1 codec, the DECODED
    fp32 values fed to the reference's own WarpPerRowFp4 / WarpPerRowSmemFp4 GPU kernels
    (src/device/csrspmm_warp_per_row_fp4.cu:9-65, csrspmm_warp_per_row_smem_fp4.cu:11-84: "Fp4" is float4,
    the values are fp32), the packed codes fed to this library.  Identical decoded operands and one fp32
    accumulator per output in stored order on both sides: the whole-row kernel must agree bit for bit, the
    split kernels within rel 1e-4 of the reference kernel (magnitude-scaled, as for every cut row)."""
    ref = oracle.ReferenceGpu()
    p = G.make("cfg4_fp4", scale=scale)
    rp, ci, va, B = _dev(p)
    mx = int(np.diff(p.row_ptr).max())
    packed, e2m1_scale = ops.e2m1_quantize(va)
    decoded = ops.e2m1_dequantize(packed, p.nnz, e2m1_scale)
    assert torch.equal(decoded.cpu(), torch.from_numpy(oracle.e2m1_decode(packed.cpu().numpy(), p.nnz, e2m1_scale)))
    mag = torch.zeros(p.M, p.Nd, device="cuda")  # sum |a*b| per output, for the scaled bound
    ops.spmm(rp, ci, decoded.abs(), B.abs(), mag, kernel="row", max_row_nnz=mx, sync=True)
    for algo in ("WarpPerRowFp4", "WarpPerRowSmemFp4"):
        C_ref = torch.full((p.M, p.Nd), float("nan"), device="cuda")
        assert ref.spmm(algo, rp, ci, decoded, B, C_ref, 1.0, 0.0, mx) == 0
        torch.cuda.synchronize()
        got = ops.spmm(rp, ci, packed, B, kernel="row", max_row_nnz=mx, e2m1_scale=e2m1_scale, nnz=p.nnz, sync=True)
        assert torch.equal(got, C_ref), f"{algo}: packed whole-row kernel differs by {float((got - C_ref).abs().max())}"
        for k in ("merge", "tma"):
            got = ops.spmm(rp, ci, packed, B, kernel=k, e2m1_scale=e2m1_scale, nnz=p.nnz, sync=True)
            assert bool(((got - C_ref).abs() <= 1e-4 * mag + 1e-6).all()), f"{algo} vs packed {k}"
            assert float(torch.isclose(got, C_ref, rtol=1e-4, atol=1e-6).float().mean()) > 0.999


def test_reference_limits_are_not_ours(cuda_lib):
    """Shapes the reference's kernels cannot launch (or would address out of range) run here."""
    ref = oracle.ReferenceGpu()
    p = G.random_csr(8, 40_000, 64, 0.0, seed=4, lengths=np.array([3000, 2, 0, 1537, 9, 0, 1, 20000]))
    rp, ci, va, B = _dev(p)
    C = torch.empty(p.M, p.Nd, device="cuda")
    assert ref.spmm("WarpPerRowSmem", rp, ci, va, B, C, 1.0, 0.0, 20000) == -2  # 640 KB of shared memory
    q = G.random_csr(16, 16, 6, 0.5, seed=5)
    assert ref.spmm("WarpPerRowFp4", *_dev(q), torch.empty(16, 6, device="cuda"), 1.0, 0.0, 16) == -2  # Nd % 4 != 0
    got = ops.spmm(rp, ci, va, B, entry="warp_per_row_smem", max_row_nnz=20000, sync=True).cpu().numpy()
    f64, mag = oracle.spmm_f64(p.row_ptr, p.col_idx, p.values, p.B)
    assert (np.abs(got - f64) <= 1e-5 * mag + 1e-6).all()


def _time(fn, reps=50, warmup=10, flush=None):
    for _ in range(warmup):
        if flush is not None:
            flush.zero_()
        fn()
    torch.cuda.synchronize()
    st = [torch.cuda.Event(enable_timing=True) for _ in range(reps)]
    en = [torch.cuda.Event(enable_timing=True) for _ in range(reps)]
    for i in range(reps):
        if flush is not None:
            flush.zero_()
        st[i].record()
        fn()
        en[i].record()
    torch.cuda.synchronize()
    t = sorted(s.elapsed_time(e) for s, e in zip(st, en))
    return t[len(t) // 2] * 1e3  # us


def _time_back_to_back(fn, reps=200, warmup=20):
    """The reference benchmark's way (benchmarks/bench_csrspmm.cu:93-113): launches one after the other, L2-warm."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def test_timing_table(cuda_lib):
    """Reference kernels (sm_100a build) vs this library on the BASELINE configurations they can run.
    Informational: the table is printed (and written to CSRSPMM_TIMING_OUT); the one assertion is that
    on the power-law configuration, where whole-row mappings stall on the longest rows, this
    library is at least twice as fast as the best reference kernel."""
    ref = oracle.ReferenceGpu()
    table = {}
    for name, make in (("cfg2_medium", lambda: G.make("cfg2_medium", device="cuda")),
                       ("cfg3_powerlaw", lambda: G.make("cfg3_powerlaw", device="cuda")),
                       ("cfg4_fp4", lambda: G.make("cfg4_fp4", device="cuda"))):
        p = make()
        mx = ops.row_stats(p.row_ptr)["max_row_nnz"]
        C = torch.empty(p.M, p.Nd, device="cuda")
        foot = p.nnz * 8 + p.M * 4 + (p.Kd + p.M) * p.Nd * 4
        flush = torch.empty(252 << 20, dtype=torch.uint8, device="cuda") if foot < (252 << 20) else None
        row = {}
        for algo in REF_ALGOS:
            if ref.spmm(algo, p.row_ptr, p.col_idx, p.values, p.B, C, 1.0, 0.0, mx) != 0:
                row["ref " + algo] = None
                continue
            torch.cuda.synchronize()
            reps = 5 if name == "cfg3_powerlaw" else 30
            row["ref " + algo] = _time(lambda: ref.spmm(algo, p.row_ptr, p.col_idx, p.values, p.B, C, 1.0, 0.0, mx), reps, 2,
                                       flush)
        call = ops.SpmmCall(p.row_ptr, p.col_idx, p.values, p.B, C, max_row_nnz=mx)
        row["csrspmm_b200 " + call.kernel] = _time(call, 30, 5, flush)
        table[name] = {"nnz": p.nnz, "max_row_nnz": mx, "us": row}
        del p, C, flush
        torch.cuda.empty_cache()
    # the reference's own benchmark grid (benchmarks/csrspmm_vs_cusparse.sh: 4 shapes x 5 densities,
    # alpha 1, beta 0.5, L2-warm back-to-back launches)
    from csrspmm_b200 import sweep
    grid = {}
    for case, M, N, K in sweep.SHAPES:
        for dens in sweep.DENSITIES:
            q = G.random_csr(M, N, K, dens, seed=M + int(dens * 1000), vlo=-10.0, vhi=10.0)
            rp, ci, va, B = _dev(q)
            mx = int(np.diff(q.row_ptr).max())
            C = torch.randn(M, K, device="cuda")
            row = {}
            for algo in REF_ALGOS:
                if ref.spmm(algo, rp, ci, va, B, C, 1.0, 0.5, mx) == 0:
                    row["ref " + algo] = _time_back_to_back(lambda: ref.spmm(algo, rp, ci, va, B, C, 1.0, 0.5, mx))
                    C.normal_()
            call = ops.SpmmCall(rp, ci, va, B, C, 1.0, 0.5, max_row_nnz=mx)
            row["csrspmm_b200 " + call.kernel] = _time_back_to_back(call)
            grid[f"{case} {M}x{N}.{K} d={dens}"] = row
    table["reference_grid_us"] = grid
    ours = np.array([next(v for k, v in r.items() if k.startswith("csrspmm")) for r in grid.values()])
    best = np.array([min(v for k, v in r.items() if k.startswith("ref")) for r in grid.values()])
    table["reference_grid_mean_speedup_over_best_reference_kernel"] = float(np.mean(best / ours))
    r3 = table["cfg3_powerlaw"]["us"]
    assert 2 * r3["csrspmm_b200 merge"] < min(v for k, v in r3.items() if k.startswith("ref") and v)
    out = os.environ.get("CSRSPMM_TIMING_OUT")
    if out:
        with open(out, "w") as f:
            json.dump(table, f, indent=1)
    print(json.dumps(table))
