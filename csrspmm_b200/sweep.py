"""The reference's benchmark sweep, on this library.

    python -m csrspmm_b200.sweep [--out sweep.csv] [--reps 300] [--warmup 50]
    python -m csrspmm_b200.sweep --torch [--out torch_sweep.csv]     # the Python-op table

Re-creates the pipeline of the reference's ``benchmarks/csrspmm_vs_cusparse.sh`` (4 shapes x 5
densities x {entry points, cuSPARSE} -> CSV with the columns ``case,M,N,K,density,sparsity,lib,algo,
gflops``) and of ``benchmarks/csrspmm_vs_cusparse.py`` (mean GFLOPS and mean speed-up over cuSPARSE
per algorithm), so that B200 numbers can be put next to the RTX 4070 table the reference publishes
(results/vs_cusparse.log).  Same protocol where it matters: alpha = 1, beta = 0.5
(benchmarks/bench_csrspmm.cu:23-24), GFLOPS = 2 * nnz * K / t (:121), cuSPARSE CSR_ALG2 with
row-major B and C (benchmarks/bench_cusparse.cu:42,126-140), L2-warm back-to-back repetitions.
Differences: inputs come from this repository's seeded Bernoulli generator (the reference's
generator is degenerate, src/host/dense_utils.cpp:54-56), the repetitions are timed with CUDA
events without a host synchronisation per call, and every entry point resolves to the same
automatically chosen kernel, so their rows differ by noise only.

``--torch`` re-creates the reference's other table, ``torch_csrspmm/torch_benchmarks.py`` (results in its
results/vs_torchsparse.log): the five Python ops next to ``torch.sparse.mm`` and ``torch.sparse.addmm``
on that script's own problems -- its tuples are (case, M, N, K) with A of M x K and B of K x N, so the dense
width is N in {1024, 2048, 4096, 4096} (:15-20, 30-36) -- built its way (A = (rand < density) * rand, B = rand),
alpha = 1.1, beta = 0.5 (:92-93), wall clock around each call with a device synchronisation, 20 warm-ups and
100 iterations, output allocation included (:47-59), GFLOPS = 2 * nnz * N / t (:62-64).
"""
from __future__ import annotations

import argparse
import csv
import ctypes as C
import sys
from pathlib import Path

import numpy as np

SHAPES = [("small", 512, 1024, 64), ("medium", 1024, 2048, 128), ("large", 4096, 4096, 128), ("XL", 8192, 4096, 256)]
DENSITIES = [0.01, 0.05, 0.10, 0.20, 0.30]
ENTRIES = [("Naive", "naive"), ("WarpPerRow", "warp_per_row"), ("WarpPerRowSmem", "warp_per_row_smem"),
           ("WarpPerRowFp4", "warp_per_row_fp4"), ("WarpPerRowSmemFp4", "warp_per_row_smem_fp4")]


def _time_call(torch, call, reps, warmup):
    for _ in range(warmup):
        call()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        call()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1e3 / reps


def _cusparse_alg2(torch, t, M, Kd, Nd, nnz, C_out, reps, warmup):
    lib_path = Path(__file__).resolve().parent / "lib" / "libcsrspmm_b200_cusparse_cmp.so"
    if not lib_path.exists():
        return None
    L = C.CDLL(str(lib_path))
    fn = L.csrspmm_cmp_cusparse_spmm
    fn.argtypes = [C.c_int, C.c_int, C.c_int, C.c_longlong, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                   C.c_float, C.c_float, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p,
                   C.POINTER(C.c_double), C.POINTER(C.c_size_t)]
    fn.restype = C.c_int
    sec, buf = C.c_double(0.0), C.c_size_t(0)
    rc = fn(M, Kd, Nd, nnz, t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(), C_out.data_ptr(), 1.0,
            0.5, 2, 0, warmup, reps, None, 0, C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(sec),
            C.byref(buf))
    torch.cuda.synchronize()
    return sec.value if rc == 0 else None


def run(out_path: str, reps: int, warmup: int, kernel: str = "auto"):
    import torch

    from . import generators as G, ops

    rows = []
    for case, M, N, K in SHAPES:
        for dens in DENSITIES:
            p = G.random_csr(M, N, K, dens, seed=M + int(dens * 1000), vlo=-10.0, vhi=10.0)
            t = [torch.from_numpy(x).cuda() for x in (p.row_ptr, p.col_idx, p.values, p.B)]
            mx = int(np.diff(p.row_ptr).max())
            C_out = torch.randn(M, K, device="cuda")
            flops = 2.0 * p.nnz * K
            for algo, entry in ENTRIES:
                call = ops.SpmmCall(t[0], t[1], t[2], t[3], C_out, 1.0, 0.5, entry=entry, max_row_nnz=mx, kernel=kernel)
                sec = _time_call(torch, call, reps, warmup)
                rows.append([case, M, N, K, dens, round(1 - dens, 2), "csrspmm_b200", algo, round(flops / sec / 1e9, 2)])
                C_out.normal_()
            sec = _cusparse_alg2(torch, t, M, N, K, p.nnz, C_out, reps, warmup)
            if sec:
                rows.append([case, M, N, K, dens, round(1 - dens, 2), "cuSPARSE", "cuSPARSE", round(flops / sec / 1e9, 2)])
            print(f"{case:6s} density {dens:.2f} nnz {p.nnz:8d} kernel {call.kernel}: "
                  f"{rows[-2][-1]:9.1f} GFLOPS, cuSPARSE {rows[-1][-1] if sec else float('nan'):9.1f}", file=sys.stderr)
    with open(out_path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["case", "M", "N", "K", "density", "sparsity", "lib", "algo", "gflops"])
        w.writerows(rows)
    return rows


def summarize(rows):
    """mean GFLOPS per algorithm and mean speed-up over cuSPARSE at the same (case, density)."""
    base = {(r[0], r[4]): r[8] for r in rows if r[7] == "cuSPARSE"}
    algos = {}
    for r in rows:
        algos.setdefault(r[7], []).append((r[8], r[8] / base[(r[0], r[4])] if (r[0], r[4]) in base else float("nan")))
    out = [(a, float(np.mean([g for g, _ in v])), float(np.nanmean([s for _, s in v]))) for a, v in algos.items()]
    return sorted(out, key=lambda x: -x[1])


def run_torch(out_path: str, iters: int = 100, warmup: int = 20):
    """The Python ops against torch.sparse, the reference's way (torch_csrspmm/torch_benchmarks.py:15-22,47-59,92-93)."""
    import time

    import torch

    import torch_csrspmm as T

    dev = torch.device("cuda")
    alpha, beta = 1.1, 0.5
    gen = torch.Generator(device=dev)
    gen.manual_seed(0)

    def wall(fn):
        for _ in range(warmup):
            fn()
            torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            t0 = time.time()
            fn()
            torch.cuda.synchronize()
            ts.append(time.time() - t0)
        return float(np.mean(ts))

    rows = []
    for case, M, N, K in SHAPES:
        for dens in DENSITIES:
            A = (torch.rand(M, K, device=dev, generator=gen) < dens).float() * torch.rand(M, K, device=dev, generator=gen)
            B = torch.rand(K, N, device=dev, generator=gen)
            Cz = torch.zeros(M, N, device=dev)
            A_csr = A.to_sparse_csr()
            row = A_csr.crow_indices().to(torch.int32)
            col = A_csr.col_indices().to(torch.int32)
            val = A_csr.values()
            mx = int((row[1:] - row[:-1]).max().item())
            nnz = val.numel()
            fns = {
                "torch.mm": lambda: alpha * torch.sparse.mm(A_csr, B) + beta * Cz,
                "torch.addmm": lambda: torch.sparse.addmm(Cz, A_csr, B, beta=beta, alpha=alpha),
                "Naive": lambda: T.csrspmm_naive(row, col, val, B, alpha, beta),
                "WarpPerRow": lambda: T.csrspmm_warp_per_row(row, col, val, B, alpha, beta),
                "WarpPerRowSmem": lambda: T.csrspmm_warp_per_row_smem(row, col, val, mx, B, alpha, beta),
                "WarpPerRowFp4": lambda: T.csrspmm_warp_per_row_fp4(row, col, val, B, alpha, beta),
                "WarpPerRowSmemFp4": lambda: T.csrspmm_warp_per_row_smem_fp4(row, col, val, mx, B, alpha, beta),
            }
            want = alpha * torch.sparse.mm(A_csr, B)
            got = fns["WarpPerRowFp4"]()
            assert torch.allclose(got, want, rtol=1e-4, atol=1e-3), "op result differs from torch.sparse.mm"
            for algo, fn in fns.items():
                sec = wall(fn)
                rows.append([case, M, N, K, dens, round(1 - dens, 2), "torch" if algo.startswith("torch") else "csrspmm_b200",
                             algo, round(2.0 * nnz * N / sec / 1e9, 2)])
            print(f"{case:6s} density {dens:.2f} nnz {nnz:8d}: " +
                  ", ".join(f"{r[7]} {r[8]:.0f}" for r in rows[-len(fns):]), file=sys.stderr)
            del A, B, Cz, A_csr, want, got
    with open(out_path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["case", "M", "N", "K", "density", "sparsity", "lib", "algo", "gflops"])
        w.writerows(rows)
    return rows


def summarize_torch(rows):
    """mean GFLOPS per algorithm and mean speed-up over torch.sparse.mm at the same (case, density), the
    reference's summary (results/vs_torchsparse.log)."""
    base = {(r[0], r[4]): r[8] for r in rows if r[7] == "torch.mm"}
    algos = {}
    for r in rows:
        algos.setdefault(r[7], []).append((r[8], r[8] / base[(r[0], r[4])]))
    out = [(a, float(np.mean([g for g, _ in v])), float(np.mean([s for _, s in v]))) for a, v in algos.items()]
    return sorted(out, key=lambda x: -x[1])


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--torch", action="store_true", help="the Python-op table against torch.sparse instead")
    ap.add_argument("--out", default="csrspmm_vs_cusparse_b200.csv")
    ap.add_argument("--reps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--kernel", default="auto", choices=["auto", "row", "merge", "tma"], help="pin a kernel")
    ns = ap.parse_args(argv)
    if ns.torch:
        rows = run_torch(ns.out if ns.out != "csrspmm_vs_cusparse_b200.csv" else "csrspmm_vs_torchsparse_b200.csv")
        print("========= Summary =========")
        print(f"{'algo':20s} {'mean_gflops':>12s} {'mean_speedup':>13s}")
        for a, g, s in summarize_torch(rows):
            print(f"{a:20s} {g:12.2f} {s:13.4f}")
        return 0
    rows = run(ns.out, ns.reps, ns.warmup, ns.kernel)
    print("========= Summary =========")
    print(f"{'algo':20s} {'mean_gflops':>12s} {'mean_speedup':>13s}")
    for a, g, s in summarize(rows):
        print(f"{a:20s} {g:12.2f} {s:13.4f}")
    for case, *_ in SHAPES:
        ours = [r[8] for r in rows if r[0] == case and r[7] == "WarpPerRowFp4"]
        cus = [r[8] for r in rows if r[0] == case and r[7] == "cuSPARSE"]
        if ours and cus:
            print(f"{case:6s} mean over densities: csrspmm_b200 {np.mean(ours):9.1f}  cuSPARSE {np.mean(cus):9.1f} GFLOPS")
    return 0


if __name__ == "__main__":
    sys.exit(main())
