#!/usr/bin/env python
"""Benchmark of the CSR x dense SpMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--kernel auto|row|merge|tma]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...        # the CPU arm (see below)

One step = one SpMM (C = A*B, alpha 1, beta 0) over the whole workload.  The default workload is
BASELINE config 5 ("cfg5_xl": 2^22 x 2^22, Zipf(2.2) row lengths with mean 32, B 2^22 x 512), the
configuration the 1/2/4/8-GPU metric is defined on; it fits one GPU.  With N > 1 the rows of A
and C are split into N contiguous blocks of equal (nnz + rows), B is broadcast once over NCCL
outside the timed region, and every rank multiplies its block: strong scaling, no collective in
the timed loop.  Rank 0 prints ONE JSON line.

  value / ms_per_step   device time, max over ranks, inputs resident in HBM
  e2e                   the same product through csrspmm_b200_spmm_host (N > 1: through
                        distributed.ShardedHostSpmm): pinned HOST buffers in, host C out, copies
                        inside the timed region, pipelined over column panels (--e2e-panels)
  roofline              compulsory bytes of rank 0's block / its step time, against the measured
                        HBM copy bandwidth in MEASURED_PEAKS.json
  cpu_baseline          the CPU oracle (OpenMP over rows) on a bounded row sample, rank 0, N = 1
  other_workloads       N = 1 only: the other BASELINE configs (kernel time, roofline, cuSPARSE via
                        torch.sparse) measured after the main loop

--impl reference times the CPU restatement of the reference's arithmetic (the reference ships no
host SpMM; see oracle/spmm_oracle.c) on all host threads over a bounded row sample of the same
workload and prints the same line with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

L2_BYTES = 126 * 2 ** 20
FALLBACK_HBM_GBS = 6650.0

# nominal fp32 multiply-add rate of a B200 (148 SMs x 128 lanes x 2 flops at the maximum SM clock): the
# denominator of the "fraction of fp32-FMA peak" reported for compute/L2-bound configurations
FP32_FMA_PEAK_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12


def ncu_traffic(workload, kernel, nnz):
    """DRAM bytes per step (dram__bytes_read.sum + dram__bytes_write.sum over the step's kernels) from
    the ncu captures recorded in profiles/ncu_traffic.json, scaled by the non-zero count when the
    captured case was smaller than (or a different shard of) what is being timed.  Each record names the
    kernel instantiations it was taken from, so a stale record can be told from the launch list."""
    f = ROOT / "profiles" / "ncu_traffic.json"
    try:
        recs = json.loads(f.read_text())["captures"]
    except Exception:
        return None
    for r in recs:
        if r["workload"] == workload.split("/")[0] and r["kernel"] == kernel:
            return {"bytes": r["dram_bytes_per_step"] * (nnz / r["nnz"]), "captured_nnz": r["nnz"],
                    "kernels": r["kernels"], "summary": r["summary"],
                    "lts_throughput_pct": r.get("lts_throughput_pct"), "l2_hit_rate_pct": r.get("l2_hit_rate_pct")}
    return None


def measured_peak():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs
    (read-only queries)."""

    def __init__(self, index: int, period_s: float = 0.05):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    _NAMES = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
              0x80: "hw_power_brake_slowdown"}

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in self._NAMES.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


# ---------------------------------------------------------------------------------------------------

def time_spmm(torch, ops, t, C_out, workspace, kernel, steps, warmup, flush_buf, max_row_nnz=0, e2m1=None,
              schedule=None):
    """Runs warmup + steps SpMMs; returns seconds per step on this device."""
    kw = dict(kernel=kernel, workspace=workspace, max_row_nnz=max_row_nnz, schedule=schedule)
    if e2m1 is not None:
        kw.update(e2m1_scale=e2m1[1], nnz=e2m1[2])
    vals = e2m1[0] if e2m1 is not None else t["values"]
    # argument block prepared once: a step is one call through the C ABI
    step = ops.SpmmCall(t["row_ptr"], t["col_idx"], vals, t["B"], C_out, 1.0, 0.0, **kw)

    for _ in range(warmup):
        if flush_buf is not None:
            flush_buf.zero_()
        step()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        if flush_buf is not None:
            flush_buf.zero_()  # evicts the previous step's lines from L2
        starts[i].record()
        step()
        stops[i].record()
    torch.cuda.synchronize()
    if flush_buf is None:
        total_ms = starts[0].elapsed_time(stops[-1])  # back to back, launch gaps included
    else:
        total_ms = sum(s.elapsed_time(e) for s, e in zip(starts, stops))
    return total_ms / 1e3 / steps


def launch_bound_modes(torch, ops, t, C_out, workspace, kernel, max_row_nnz, flush_buf, reps=100):
    """A small product in the ways a caller can issue it, microseconds per launch over `reps` launches:
    L2-cold (252 MiB written between launches; median and min of per-launch events), L2-warm back to
    back (one event pair around all launches, launch gaps included), the same launches replayed from
    one CUDA graph (launch gaps removed), and warm with beta = 0.5 (C read as well as written)."""
    kw = dict(kernel=kernel, workspace=workspace, max_row_nnz=max_row_nnz)
    step = ops.SpmmCall(t["row_ptr"], t["col_idx"], t["values"], t["B"], C_out, 1.0, 0.0, **kw)
    step_beta = ops.SpmmCall(t["row_ptr"], t["col_idx"], t["values"], t["B"], C_out, 1.0, 0.5, **kw)
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731

    def back_to_back(fn):
        for _ in range(10):
            fn()
        torch.cuda.synchronize()
        e0, e1 = ev(), ev()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    out = {"launches": reps}
    cold = []
    for i in range(reps + 3):
        flush_buf.zero_()
        e0, e1 = ev(), ev()
        e0.record()
        step()
        e1.record()
        cold.append((e0, e1))
    torch.cuda.synchronize()
    cold = sorted(a.elapsed_time(b) * 1e3 for a, b in cold[3:])
    out["cold_us_median"], out["cold_us_min"] = cold[len(cold) // 2], cold[0]
    out["warm_us"] = back_to_back(step)
    out["warm_beta_half_us"] = back_to_back(step_beta)
    g, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for _ in range(reps):
                step()
    out["graph_us"] = back_to_back(g.replay) / reps
    return out


def problem_bytes(G, t, M, Nd, nnz, Kd, value_bytes=4.0):
    touched = G.touched_rows(t["col_idx"], Kd) if nnz else 0
    return G.min_bytes(M, Nd, nnz, touched, 0.0, value_bytes), touched


def tolerance_report(torch, oracle, row_ptr, col_idx, values, B, C_dev, n_random=4096, n_long=64, seed=0):
    """Rows [n_long longest + n_random random] of a device result against the CPU oracle: the strict
    elementwise pass rate at rtol 1e-5 / atol 1e-6 against the sequential fp32 (fused multiply-add) oracle,
    and the worst |err| / (1e-5 * sum|a*b| + 1e-6) against the fp64 oracle (<= 1 means inside the
    accumulation-order bound)."""
    rp_l = row_ptr.cpu().numpy().astype(np.int64)
    M = rp_l.shape[0] - 1
    lens = np.diff(rp_l)
    rows = np.unique(np.concatenate([np.random.default_rng(seed).integers(0, M, n_random), np.argsort(lens)[-n_long:]]))
    idx = np.concatenate([np.arange(rp_l[r], rp_l[r + 1]) for r in rows]) if rows.size else np.zeros(0, np.int64)
    idx_d = torch.from_numpy(idx).to(col_idx.device)
    uniq, inv = torch.unique(col_idx[idx_d].long(), return_inverse=True)
    sub_rp = np.zeros(len(rows) + 1, np.int32)
    np.cumsum(lens[rows], out=sub_rp[1:])
    sub_ci = inv.to(torch.int32).cpu().numpy()
    sub_va = values[idx_d].cpu().numpy()
    sub_B = B[uniq].cpu().numpy() if uniq.numel() else np.zeros((1, B.shape[1]), np.float32)
    th = oracle.max_threads()
    f64, mag = oracle.spmm_f64(sub_rp, sub_ci, sub_va, sub_B, threads=th)
    f32 = oracle.spmm(sub_rp, sub_ci, sub_va, sub_B, fused=True, threads=th)
    got = C_dev[torch.from_numpy(rows).to(C_dev.device)].cpu().numpy()
    bound = 1e-5 * mag + 1e-6
    worst = float((np.abs(got - f64) / bound).max()) if got.size else 0.0
    strict = np.isclose(got, f32, rtol=1e-5, atol=1e-6)
    return {"rows_checked": int(rows.size), "longest_row_checked": int(lens[rows].max()) if rows.size else 0,
            "strict_pass_rate_rtol1e-5_atol1e-6": float(strict.mean()) if strict.size else 1.0,
            "bit_identical_to_fp32_oracle": float((got == f32).mean()) if got.size else 1.0,
            "worst_err_over_bound": worst, "within_bound": bool(worst <= 1.0)}


def copy_ceiling(torch, dev, barrier, D, nbytes=1 << 30, reps=3):
    """What the host link of this box gives with nothing else going on: every rank copies `nbytes` of pinned
    memory up and `nbytes` down at the same time (two streams), all ranks together.  GB/s per rank and
    direction = nbytes / (slowest rank's time for both copies to finish)."""
    h_up = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    h_dn = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    d_up = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    d_dn = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    s1, s2 = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    best = {"both": float("inf"), "up": float("inf"), "down": float("inf")}
    for mode in ("both", "up", "down"):
        for _ in range(reps + 1):
            barrier()
            t0 = time.perf_counter()
            if mode in ("both", "up"):
                with torch.cuda.stream(s1):
                    d_up.copy_(h_up, non_blocking=True)
            if mode in ("both", "down"):
                with torch.cuda.stream(s2):
                    h_dn.copy_(d_dn, non_blocking=True)
            s1.synchronize()
            s2.synchronize()
            best[mode] = min(best[mode], D.max_over_ranks(time.perf_counter() - t0, dev))
    del h_up, h_dn, d_up, d_dn
    g = nbytes / 1e9
    return {"bytes_each_way_per_rank": nbytes, "GBps_per_rank_up_alone": g / best["up"], "GBps_per_rank_down_alone": g / best["down"],
            "GBps_per_rank_each_way_together": g / best["both"]}


def cusparse_via_torch(torch, t, M, Kd, steps, warmup, flush_buf):
    """cuSPARSE CSR SpMM as torch.sparse dispatches it (comparator only)."""
    try:
        A = torch.sparse_csr_tensor(t["row_ptr"], t["col_idx"], t["values"], size=(M, Kd))
        for _ in range(max(warmup, 1)):
            out = torch.sparse.mm(A, t["B"])
        torch.cuda.synchronize()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        for i in range(steps):
            if flush_buf is not None:
                flush_buf.zero_()
            starts[i].record()
            out = torch.sparse.mm(A, t["B"])
            stops[i].record()
        torch.cuda.synchronize()
        del out
        return sum(s.elapsed_time(e) for s, e in zip(starts, stops)) / 1e3 / steps
    except Exception as e:  # comparator is best effort
        return f"unavailable: {type(e).__name__}: {e}"[:200]


def cusparse_direct(torch, t, M, Kd, Nd, nnz, C_out, steps, warmup, flush_buf):
    """cusparseSpMM through the comparator library (csrc/cmp/cusparse_cmp.cu): every CSR algorithm,
    with and without cusparseSpMM_preprocess.  Returns {name: seconds} or a reason string."""
    import ctypes as C
    lib_path = ROOT / "csrspmm_b200" / "lib" / "libcsrspmm_b200_cusparse_cmp.so"
    if not lib_path.exists():
        return "unavailable: comparator library not built"
    try:
        L = C.CDLL(str(lib_path))
        fn = L.csrspmm_cmp_cusparse_spmm
        fn.argtypes = [C.c_int, C.c_int, C.c_int, C.c_longlong, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                       C.c_void_p, C.c_float, C.c_float, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_size_t,
                       C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_size_t)]
        fn.restype = C.c_int
        out = {}
        stream = torch.cuda.current_stream().cuda_stream
        for alg, name in ((0, "default"), (1, "csr_alg1"), (2, "csr_alg2"), (3, "csr_alg3")):
            for pre in (0, 1):
                sec, buf = C.c_double(0.0), C.c_size_t(0)
                rc = fn(M, Kd, Nd, nnz, t["row_ptr"].data_ptr(), t["col_idx"].data_ptr(), t["values"].data_ptr(),
                        t["B"].data_ptr(), C_out.data_ptr(), 1.0, 0.0, alg, pre, warmup, steps,
                        flush_buf.data_ptr() if flush_buf is not None else None,
                        flush_buf.numel() if flush_buf is not None else 0, C.c_void_p(stream), C.byref(sec), C.byref(buf))
                torch.cuda.synchronize()
                out[name + ("+preprocess" if pre else "")] = sec.value if rc == 0 else f"error {rc}"
        return out
    except Exception as e:
        return f"unavailable: {type(e).__name__}: {e}"[:200]


def cusparse_summary(res, flops):
    if not isinstance(res, dict):
        return res
    ok = {k: v for k, v in res.items() if isinstance(v, float) and v > 0}
    if not ok:
        return res
    best = min(ok, key=ok.get)
    return {"best": best, "gflops": flops / ok[best] / 1e9, "us": ok[best] * 1e6,
            "all_us": {k: (round(v * 1e6, 1) if isinstance(v, float) else v) for k, v in res.items()}}


def cpu_sample(torch, G, oracle, prob, sample_rows, threads, repeats=3):
    """Times the CPU oracle on rows [0, sample_rows) of the problem (B complete, on the host)."""
    rp = prob.row_ptr[: sample_rows + 1]
    rp_h = (rp.cpu().numpy() if hasattr(rp, "cpu") else np.asarray(rp)).astype(np.int32)
    n = int(rp_h[-1])
    to_h = (lambda x: x.cpu().numpy()) if hasattr(prob.col_idx, "cpu") else np.asarray
    ci_h, va_h = to_h(prob.col_idx[:n]), to_h(prob.values[:n])
    B_h = to_h(prob.B)
    C_h = np.zeros((sample_rows, prob.Nd), np.float32)
    oracle.spmm(rp_h, ci_h, va_h, B_h, threads=threads, out=C_h)  # untimed: pages in C, warms the caches
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle.spmm(rp_h, ci_h, va_h, B_h, threads=threads, out=C_h)
        best = min(best, time.perf_counter() - t0)
    return 2.0 * n * prob.Nd / best / 1e9, n, best


def sample_rows_for(name, M):
    """Rows of the workload the CPU legs run.  All of them: even config 5 (137 GFLOP, 275 GB of
    gathered rows) is a few seconds per pass on the host cores, so no sub-sampling is needed to
    stay within the time bound; the three timed passes add up to about ten seconds of CPU work."""
    return M


# ---------------------------------------------------------------------------------------------------

def run_reference_arm(ns):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import oracle
    from csrspmm_b200 import generators as G
    device = "cuda" if torch.cuda.is_available() else "cpu"
    prob = G.make(ns.workload, scale=ns.scale, device=device)
    threads = oracle.max_threads()
    rows = sample_rows_for(ns.workload, prob.M)
    # untimed warm-up pass(es), then K timed passes over the sample
    times = []
    rp_h = (prob.row_ptr[: rows + 1].cpu().numpy() if hasattr(prob.row_ptr, "cpu") else prob.row_ptr[: rows + 1]).astype(np.int32)
    n = int(rp_h[-1])
    to_h = (lambda x: x.cpu().numpy()) if hasattr(prob.col_idx, "cpu") else np.asarray
    ci_h, va_h, B_h = to_h(prob.col_idx[:n]), to_h(prob.values[:n]), to_h(prob.B)
    C_h = np.zeros((rows, prob.Nd), np.float32)
    for i in range(max(ns.warmup, 1) + ns.steps):
        t0 = time.perf_counter()
        oracle.spmm(rp_h, ci_h, va_h, B_h, threads=threads, out=C_h)
        if i >= max(ns.warmup, 1):
            times.append(time.perf_counter() - t0)
    sec = float(np.mean(times))
    gflops = 2.0 * n * prob.Nd / sec / 1e9
    sample = f"rows [0, {rows}) of {prob.M} ({n} of {prob.nnz} nnz), B complete on the host"
    line = {
        "impl": "reference", "metric": "SpMM GFLOPS", "value": gflops, "unit": "GFLOPS", "n_gpus": ns.gpus,
        "steps": ns.steps, "warmup": ns.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": prob.name, "M": prob.M, "Kd": prob.Kd, "Nd": prob.Nd, "nnz": prob.nnz,
                   "note": "CPU restatement of the reference kernels' arithmetic (the reference has no host SpMM), "
                           "OpenMP over rows, one step = one pass over the row sample"},
        "cpu_baseline": {"value": gflops, "unit": "GFLOPS", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gflops, "unit": "GFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)
    return 0


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg5_xl")
    ap.add_argument("--scale", type=int, default=1, help="divide M and Kd (for quick runs and ncu captures)")
    ap.add_argument("--kernel", default="auto", choices=["auto", "row", "merge", "tma"])
    ap.add_argument("--no-extras", action="store_true", help="skip e2e, cpu_baseline and other_workloads")
    ap.add_argument("--no-schedule", action="store_true", help="never build a per-matrix schedule (plain AUTO kernel)")
    ap.add_argument("--sched-threshold", type=int, default=0, help="rows of this many entries or more are scheduled (0: the library's choice)")
    ap.add_argument("--sched-slab-mib", type=int, default=0, help="MiB of B per slab of a schedule (0: the library's choice)")
    ap.add_argument("--sched-piece", type=int, default=0, help="longest piece of a scheduled row (0: the library's choice)")
    ap.add_argument("--only-e2e", action="store_true",
                    help="keep e2e but skip the oracle check, cpu_baseline, cuSPARSE and other_workloads")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-copy-ceiling", action="store_true", help="skip the copies-only measurement of the host link")
    ap.add_argument("--e2e-panels", type=int, default=0,
                    help="column panels of the host round trip (0 = the library's rule, 1 = no panels)")
    ns = ap.parse_args(argv)
    ns.warmup = max(ns.warmup, 3) if ns.impl == "ours" else ns.warmup

    if ns.impl == "reference":
        return run_reference_arm(ns)

    import torch
    import torch.distributed as dist
    from csrspmm_b200 import _lib, distributed as D, generators as G, ops

    _lib.lib()  # fail here, loudly, when the CUDA library is missing
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != ns.gpus:
        raise SystemExit(f"--gpus {ns.gpus} but WORLD_SIZE={world}: launch one rank per GPU with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # ---- the workload: generated on rank 0's GPU, replicated once (untimed) ------------------------
    cfg = G.CONFIGS[ns.workload]
    if rank == 0:
        prob = G.make(ns.workload, scale=ns.scale, device=dev)
        sizes = torch.tensor([prob.M, prob.Kd, prob.Nd, prob.nnz], dtype=torch.int64, device=dev)
    else:
        prob, sizes = None, torch.zeros(4, dtype=torch.int64, device=dev)
    if world > 1:
        dist.broadcast(sizes, 0)
    M, Kd, Nd, nnz = (int(x) for x in sizes.tolist())
    if rank == 0:
        row_ptr, col_idx, values, B = prob.row_ptr, prob.col_idx, prob.values, prob.B
    else:
        row_ptr = torch.empty(M + 1, dtype=torch.int32, device=dev)
        col_idx = torch.empty(nnz, dtype=torch.int32, device=dev)
        values = torch.empty(nnz, dtype=torch.float32, device=dev)
        B = torch.empty((Kd, Nd), dtype=torch.float32, device=dev)
    t_bcast = 0.0
    if world > 1:
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for x in (row_ptr, col_idx, values, B):
            D.replicate(x, 0)
        torch.cuda.synchronize()
        t_bcast = time.perf_counter() - t0

    # ---- nnz-balanced row partition (host), this rank's block -----------------------------------
    rp_host = row_ptr.cpu().numpy()
    bounds = D.partition_rows(rp_host, world, 1.0)
    imbalance = D.partition_imbalance(rp_host, bounds, 1.0)
    shard = D.take_shard(row_ptr, col_idx, values, bounds, rank)
    t = {"row_ptr": shard.row_ptr, "col_idx": shard.col_idx, "values": shard.values, "B": B}
    if world > 1:
        del row_ptr, col_idx, values
    my_rows, my_nnz = shard.rows, shard.nnz
    C_out = torch.empty((my_rows, Nd), dtype=torch.float32, device=dev)
    workspace = torch.empty(max(ops.workspace_bytes(my_rows, Kd, Nd, my_nnz), 256), dtype=torch.uint8, device=dev)
    my_bytes, touched = problem_bytes(G, t, my_rows, Nd, my_nnz, Kd)
    footprint = my_nnz * 8 + my_rows * 4 + (Kd + my_rows) * Nd * 4
    flush = footprint < 2 * L2_BYTES
    flush_buf = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev) if flush else None
    chosen = ops.selected_kernel(my_rows, Kd, Nd, my_nnz, kernel=ns.kernel, max_row_nnz=0)
    launches_per_step = 1 if chosen == "row" else 2
    # per-matrix schedule (built once per matrix, outside the timed region, like cuSPARSE's preprocess): the
    # library decides by itself whether this matrix and this width of B are worth one
    schedule, sched_info = None, None
    if ns.kernel == "auto" and not ns.no_schedule and my_rows > 0:
        def build_schedule():
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            sch = ops.Schedule(t["row_ptr"], t["col_idx"], Kd, Nd, threshold=ns.sched_threshold,
                               slab_rows=(ns.sched_slab_mib << 20) // (Nd * 4), piece_nnz=ns.sched_piece)
            torch.cuda.synchronize()
            return sch, (time.perf_counter() - t0) * 1e3
        # the first build of a process also loads the library's kernels; the second is what a schedule costs
        schedule, first_ms = build_schedule()
        schedule.close()
        schedule, wall_ms = build_schedule()
        sched_info = dict(schedule.info(), build_wall_ms=wall_ms, first_build_in_process_wall_ms=first_ms)
        if schedule.active:
            chosen, launches_per_step = "scheduled", 4
        else:
            schedule = None

    # ---- timed region -------------------------------------------------------------------------------
    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    barrier()
    with ClockSampler(physical_gpu_index(local)) as clocks:
        barrier()
        sec = time_spmm(torch, ops, t, C_out, None if schedule is not None else workspace, ns.kernel, ns.steps, ns.warmup,
                        flush_buf, schedule=schedule)
        barrier()
    sec_max = D.max_over_ranks(sec, dev)
    flops_total = 2.0 * nnz * Nd
    value = flops_total / sec_max / 1e9

    # parity on a row sample against the CPU oracle (outside every timed region): strict elementwise pass
    # rate at rtol 1e-5 / atol 1e-6 against the sequential fp32 oracle, and the worst error in units of the
    # accumulation-order bound 1e-5 * sum|a*b| + 1e-6 against the fp64 oracle (must be <= 1)
    check = None
    if rank == 0 and not ns.no_extras and not ns.only_e2e:
        import oracle
        check = tolerance_report(torch, oracle, shard.row_ptr, t["col_idx"], t["values"], B, C_out)

    # ---- end to end: pinned host buffers in, host C out ---------------------------------------------
    # N = 1: csrspmm_b200_spmm_host (one C-ABI call does the copies and the product).
    # N > 1: distributed.ShardedHostSpmm -- each rank uploads its block of A and 1/N of B, the
    #        slices of B are all-gathered over NVLink, C blocks go back to their hosts.
    e2e = None
    if not ns.no_extras:
        keep_rows = torch.arange(0, my_rows, max(my_rows // 4096, 1), device=dev)
        keep_vals = C_out[keep_rows].clone()  # the device-timed result on a row sample, to compare e2e against
        if world == 1 or Kd % world != 0:  # (an uneven split of B's rows: every rank uploads all of B itself)
            h = {k: torch.empty(v.shape, dtype=v.dtype, pin_memory=True) for k, v in t.items()}
            for k in h:
                h[k].copy_(t[k])
            C_host = torch.empty((my_rows, Nd), dtype=torch.float32, pin_memory=True)
            arena = torch.empty(ops.host_arena_bytes(my_rows, Kd, Nd, my_nnz), dtype=torch.uint8, device=dev)

            if ns.e2e_panels > 0:
                os.environ["CSRSPMM_HOST_PANELS"] = str(ns.e2e_panels)
            n_panels = len(D.column_panels(Kd, Nd, ns.e2e_panels or None))

            def e2e_step():  # the matrix stays on the device between products; B goes up and C comes back every step
                ops.spmm_host(t["row_ptr"], t["col_idx"], t["values"], h["B"], C_host, 1.0, 0.0, kernel=ns.kernel,
                              arena=arena, device=dev)

            def e2e_step_with_a():  # everything from the host, A included
                ops.spmm_host(h["row_ptr"], h["col_idx"], h["values"], h["B"], C_host, 1.0, 0.0, kernel=ns.kernel,
                              arena=arena, device=dev)

            h2d = Kd * Nd * 4
            h2d_with_a = my_nnz * 8 + (my_rows + 1) * 4 + Kd * Nd * 4
            d2h, xchg = my_rows * Nd * 4, 0
            api = (f"csrspmm_b200_spmm_host (per step: pinned host B in, host C out; A resident on the device, as over "
                   f"repeated products on one matrix; {n_panels} column panel(s): uploads, kernels and downloads of "
                   "different panels overlap)")
        else:
            sl = Kd // world
            hs = D.Shard(rank, world, shard.row_lo, shard.row_hi,
                         shard.row_ptr.cpu().pin_memory(), shard.col_idx.cpu().pin_memory(),
                         shard.values.cpu().pin_memory(), shard.max_row_nnz)
            hB = B[rank * sl:(rank + 1) * sl].cpu().pin_memory()
            del t, B, shard, C_out, workspace
            torch.cuda.empty_cache()
            runner = D.ShardedHostSpmm(hs, hB, Kd, dev, kernel=ns.kernel, panels=ns.e2e_panels or None, keep_matrix=True)
            e2e_step = runner.run
            e2e_step_with_a = None
            n_panels = len(runner.panels)
            h2d, d2h, xchg = runner.h2d_bytes, runner.d2h_bytes, runner.exchange_bytes
            h2d_with_a = h2d + hs.nnz * 8 + (hs.rows + 1) * 4
            api = ("distributed.ShardedHostSpmm (per rank and step: pinned host 1/N of B in, NCCL all-gather of B, host "
                   f"block of C out; the rank's block of A resident on the device; {n_panels} column panel(s), the stages "
                   "of different panels overlap)")
        torch.cuda.synchronize()
        e2e_step()  # warm-up
        # every call is synchronous (it returns when C is in host memory), so each is timed by itself, as
        # the max over ranks; the median call is reported (the host side of a shared box has hiccups)
        per_call = []
        for _ in range(ns.e2e_steps):
            barrier()
            t0 = time.perf_counter()
            e2e_step()
            torch.cuda.synchronize()
            per_call.append(D.max_over_ranks(time.perf_counter() - t0, dev))
        e2e_sec = float(np.median(per_call))
        C_e2e = C_host if (world == 1 or Kd % world != 0) else runner.C_host
        # same product as the device-timed run (row blocks may associate split rows differently)
        same = bool(torch.allclose(C_e2e[keep_rows.cpu()], keep_vals.cpu(), rtol=1e-3, atol=1e-3))
        same = D.sum_over_ranks(0.0 if same else 1.0, dev) == 0.0
        e2e = {"value": flops_total / e2e_sec / 1e9, "matches_device_run": same, "unit": "GFLOPS", "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(d2h), "nvlink_bytes_per_step": int(xchg), "ms_per_step": e2e_sec * 1e3,
               "ms_min": min(per_call) * 1e3, "ms_max": max(per_call) * 1e3,
               "steps": ns.e2e_steps, "bytes_are": "per rank", "column_panels": n_panels, "api": api}
        if e2e_step_with_a is not None:  # the same call with A uploaded every step as well
            e2e_step_with_a()
            with_a = []
            for _ in range(2):
                t0 = time.perf_counter()
                e2e_step_with_a()
                torch.cuda.synchronize()
                with_a.append(time.perf_counter() - t0)
            e2e["with_A_uploaded_every_step"] = {"ms_per_step": min(with_a) * 1e3, "h2d_bytes_per_step": int(h2d_with_a)}
        # what the host link gives with nothing but copies on it, all ranks at once: the floor of a step is the
        # larger of (bytes up / rate up) and (bytes down / rate down) when both directions run together
        if not ns.no_copy_ceiling:
            if world > 1:
                del runner
            else:
                del arena
            torch.cuda.empty_cache()
            cc = copy_ceiling(torch, dev, barrier, D)
            rate = cc["GBps_per_rank_each_way_together"] * 1e9
            cc["floor_ms_per_step"] = max(h2d, d2h) / rate * 1e3
            cc["e2e_over_floor"] = e2e_sec * 1e3 / cc["floor_ms_per_step"]
            cc["aggregate_GBps_each_way"] = cc["GBps_per_rank_each_way_together"] * world
            e2e["copy_ceiling"] = cc

    if world > 1:
        barrier()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    peak, peak_kind = measured_peak()
    traffic = ncu_traffic(prob.name, chosen, my_nnz)
    achieved = my_bytes / sec / 1e9
    gather_bytes = my_nnz * Nd * 4.0
    line = {
        "metric": "SpMM GFLOPS", "value": value, "unit": "GFLOPS", "n_gpus": world, "steps": ns.steps,
        "warmup": ns.warmup, "ms_per_step": sec_max * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": prob.name, "M": M, "Kd": Kd, "Nd": Nd, "nnz": nnz, "alpha": 1.0, "beta": 0.0,
                   "row_lengths": {k: cfg[k] for k in ("kind", "p", "zipf_a", "mean", "cap") if k in cfg},
                   "kernel": chosen, "partition": f"rows, equal nnz+rows over {world} GPU(s), imbalance {imbalance:.4f}",
                   "B": "replicated per GPU (NCCL broadcast outside the timed region)" if world > 1 else "resident",
                   "l2": "L2 flushed between steps (256 MiB write)" if flush else "inputs larger than L2, back to back",
                   "broadcast_s": round(t_bcast, 3)},
        "gpu_launches": ns.steps * launches_per_step,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": (traffic or {}).get("bytes"), "traffic_source": traffic, "peak_kind": f"of {peak_kind}",
                     "algorithmic_bytes": my_bytes, "b_rows_touched": touched,
                     "gather_bytes": gather_bytes, "gather_GBps": gather_bytes / sec / 1e9,
                     "gather_frac": gather_bytes / sec / 1e9 / peak,
                     "scope": "rank 0's row block, every kernel of a step"},
        "clocks": clocks.summary(),
    }
    if check is not None:
        line["oracle_check"] = check["within_bound"]
        line["parity"] = check
    if sched_info is not None:
        line["schedule"] = sched_info
    if e2e is not None:
        line["e2e"] = e2e

    if world == 1 and not ns.no_extras and not ns.only_e2e:
        import oracle
        rows = sample_rows_for(ns.workload, M)
        g, n_s, best = cpu_sample(torch, G, oracle, prob, rows, oracle.max_threads())
        line["cpu_baseline"] = {"value": g, "unit": "GFLOPS", "cores": oracle.max_threads(), "kind": "port",
                                "sample": f"rows [0, {rows}) of {M} ({n_s} of {nnz} nnz), B complete on the host, "
                                          f"best of 3 passes, {best:.2f} s per pass"}
        if schedule is not None:  # the same product without the schedule (the plain AUTO kernel), for comparison
            plain = ops.selected_kernel(my_rows, Kd, Nd, my_nnz, kernel=ns.kernel, max_row_nnz=0)
            sec_plain = time_spmm(torch, ops, t, C_out, workspace, ns.kernel, min(ns.steps, 5), 3, flush_buf)
            line["without_schedule"] = {"kernel": plain, "ms_per_step": sec_plain * 1e3, "gflops": flops_total / sec_plain / 1e9,
                                        "roofline_frac": my_bytes / sec_plain / 1e9 / peak,
                                        "traffic": (ncu_traffic(prob.name, plain, my_nnz) or {}).get("bytes")}
        line["cusparse"] = cusparse_summary(
            cusparse_direct(torch, t, my_rows, Kd, Nd, my_nnz, C_out, min(ns.steps, 5), 2, flush_buf), flops_total)
        if isinstance(line["cusparse"], dict) and "us" in line["cusparse"]:
            line["speedup_over_cusparse_best"] = line["cusparse"]["us"] / (sec * 1e6)
        del prob, t, B, C_out, workspace, shard
        torch.cuda.empty_cache()
        line["other_workloads"] = other_workloads(torch, ops, G, ns, dev, peak)

    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def other_workloads(torch, ops, G, ns, dev, peak):
    """Kernel-only numbers for the other BASELINE configs (1 GPU), each next to cuSPARSE, with the parity
    figures of every kernel on a row sample."""
    import oracle
    out = {}
    for name in ("cfg1_check", "cfg2_medium", "cfg3_powerlaw", "cfg4_fp4"):
        if name == ns.workload:
            continue
        try:
            p = G.make(name, device=dev)
            t = {"row_ptr": p.row_ptr, "col_idx": p.col_idx, "values": p.values, "B": p.B}
            C_out = torch.empty((p.M, p.Nd), dtype=torch.float32, device=dev)
            ws = torch.empty(max(ops.workspace_bytes(p.M, p.Kd, p.Nd, p.nnz), 256), dtype=torch.uint8, device=dev)
            footprint = p.nnz * 8 + p.M * 4 + (p.Kd + p.M) * p.Nd * 4
            fb = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev) if footprint < 2 * L2_BYTES else None
            mx = ops.row_stats(p.row_ptr)["max_row_nnz"]
            nbytes, _ = problem_bytes(G, t, p.M, p.Nd, p.nnz, p.Kd)
            flops = 2.0 * p.nnz * p.Nd
            gather = p.nnz * p.Nd * 4.0
            entry = {"nnz": p.nnz, "max_row_nnz": mx, "l2_flushed": fb is not None, "algorithmic_bytes": nbytes,
                     "gather_bytes": gather, "kernels": {}}
            for k in ("row", "merge", "tma"):
                sec = time_spmm(torch, ops, t, C_out, ws, k, 20, 3, fb, max_row_nnz=mx)
                entry["kernels"][k] = {"gflops": flops / sec / 1e9, "us": sec * 1e6,
                                       "roofline_frac": nbytes / sec / 1e9 / peak,
                                       "parity": tolerance_report(torch, oracle, p.row_ptr, p.col_idx, p.values, p.B, C_out)}
            auto = ops.selected_kernel(p.M, p.Kd, p.Nd, p.nnz, max_row_nnz=mx)
            entry["auto"] = auto
            sec_auto = entry["kernels"][auto]["us"] / 1e6
            tr = ncu_traffic(name, auto, p.nnz)
            entry["roofline"] = {"bound": "hbm" if name == "cfg3_powerlaw" else "l2", "kernel": auto,
                                 "achieved_GBps": nbytes / sec_auto / 1e9, "frac_of_measured_hbm_peak": nbytes / sec_auto / 1e9 / peak,
                                 "gather_TBps_l2_to_sm": gather / sec_auto / 1e12,
                                 "fp32_fma_TFLOPS": flops / sec_auto / 1e12,
                                 "frac_of_fp32_fma_peak": flops / sec_auto / 1e12 / FP32_FMA_PEAK_TFLOPS,
                                 "traffic": tr}
            # a schedule at the library's own choice (inactive for narrow rows of B), and for config 3 one with
            # a threshold given, to show what it costs there
            sch = ops.Schedule(p.row_ptr, p.col_idx, p.Kd, p.Nd)
            entry["schedule_auto"] = sch.info()
            if name == "cfg3_powerlaw":
                forced = ops.Schedule(p.row_ptr, p.col_idx, p.Kd, p.Nd, threshold=64, slab_rows=(32 << 20) // (p.Nd * 4))
                sec = time_spmm(torch, ops, t, C_out, None, "auto", 20, 3, fb, schedule=forced)
                entry["kernels"]["scheduled_threshold_64"] = {
                    "gflops": flops / sec / 1e9, "us": sec * 1e6, "roofline_frac": nbytes / sec / 1e9 / peak,
                    "schedule": forced.info(),
                    "parity": tolerance_report(torch, oracle, p.row_ptr, p.col_idx, p.values, p.B, C_out)}
                del forced
            del sch
            if fb is not None and p.nnz < 1_000_000:  # launch-bound sizes: how the call is issued matters
                modes = launch_bound_modes(torch, ops, t, C_out, ws, auto, mx, fb)
                for key in ("cold_us_median", "warm_us", "graph_us"):  # the same roofline, per way of launching
                    modes[key.replace("_us", "").replace("_median", "") + "_roofline_frac"] = nbytes / (modes[key] * 1e-6) / 1e9 / peak
                entry["launch_modes_auto_kernel"] = modes
            cs = cusparse_via_torch(torch, t, p.M, p.Kd, 20, 3, fb)
            entry["cusparse_torch"] = {"gflops": flops / cs / 1e9, "us": cs * 1e6} if isinstance(cs, float) else cs
            entry["cusparse"] = cusparse_summary(cusparse_direct(torch, t, p.M, p.Kd, p.Nd, p.nnz, C_out, 20, 3, fb), flops)
            if isinstance(entry["cusparse"], dict) and "us" in entry["cusparse"]:
                entry["speedup_over_cusparse_best"] = entry["cusparse"]["us"] / (sec_auto * 1e6)
            if name == "cfg4_fp4":
                packed, scale = ops.e2m1_quantize(p.values)
                e = (packed.to(dev), scale, p.nnz)
                decoded = ops.e2m1_dequantize(e[0], p.nnz, scale)
                nb4, _ = problem_bytes(G, t, p.M, p.Nd, p.nnz, p.Kd, 0.5)
                for k in ("row", "merge", "tma"):
                    sec = time_spmm(torch, ops, t, C_out, ws, k, 20, 3, fb, max_row_nnz=mx, e2m1=e)
                    entry["kernels"][k + "_e2m1"] = {"gflops": flops / sec / 1e9, "us": sec * 1e6,
                                                     "roofline_frac": nb4 / sec / 1e9 / peak,
                                                     "parity_on_decoded_values": tolerance_report(
                                                         torch, oracle, p.row_ptr, p.col_idx, decoded, p.B, C_out)}
            out[name] = entry
            del p, t, C_out, ws, fb
            torch.cuda.empty_cache()
        except Exception as e:  # secondary numbers must not take the headline down
            out[name] = f"failed: {type(e).__name__}: {e}"[:300]
    out["long_rows_wide_B"] = locality_pass_case(torch, ops, G, dev, skewed=False)
    out["long_skewed_rows_wide_B"] = locality_pass_case(torch, ops, G, dev, skewed=True)
    return out


def locality_pass_case(torch, ops, G, dev, skewed):
    """The opt-in tiled product (csrspmm_b200_spmm_tiled) next to the untiled kernels where it has its best
    chance: 65 536 rows of 328 non-zeros (ascending uniform columns) over Kd = 2^21, Nd = 256, so B is 2 GiB;
    `skewed` draws the row lengths from Zipf(2) with the same mean instead (longest row 16 384)."""
    try:
        M, Kd, Nd, per = 65536, 1 << 21, 256, 328
        gen = torch.Generator(device=dev)
        gen.manual_seed(0)
        lens = (G.zipf_lengths(np.random.default_rng(0), M, Kd, 2.0, float(per), 16384) if skewed
                else np.full(M, per, np.int64))
        rp = np.zeros(M + 1, np.int32)
        np.cumsum(lens, out=rp[1:])
        ci = G._columns_torch(gen, lens, Kd, dev)
        nnz = int(rp[-1])
        va = torch.empty(nnz, device=dev).uniform_(-1.0, 1.0, generator=gen)
        B = torch.randn((Kd, Nd), device=dev, generator=gen)
        rp = torch.from_numpy(rp).to(dev)
        C_out = torch.empty((M, Nd), device=dev)
        ws = torch.empty(ops.workspace_bytes(M, Kd, Nd, nnz) + 4 * M + 4096, dtype=torch.uint8, device=dev)
        mx = int(lens.max())
        t = {"row_ptr": rp, "col_idx": ci, "values": va, "B": B}
        res = {"M": M, "Kd": Kd, "Nd": Nd, "nnz": nnz, "max_row_nnz": mx, "B_bytes": Kd * Nd * 4, "us": {}}
        for k in ("row", "merge"):
            res["us"][k] = time_spmm(torch, ops, t, C_out, ws, k, 5, 2, None, max_row_nnz=mx) * 1e6
        ref = ops.spmm(rp, ci, va, B, kernel="row", max_row_nnz=mx, sync=True)
        for slab_mib in ((64,) if skewed else (32, 64, 96)):
            pr = (slab_mib << 20) // (Nd * 4)
            for _ in range(2):
                ops.spmm_tiled(rp, ci, va, B, C_out, panel_rows=pr, workspace=ws)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                ops.spmm_tiled(rp, ci, va, B, C_out, panel_rows=pr, workspace=ws)
            e1.record()
            torch.cuda.synchronize()
            res["us"][f"tiled_{slab_mib}MiB"] = e0.elapsed_time(e1) * 1e3 / 5
        res["tiled_bit_identical_to_row_kernel"] = bool(torch.equal(C_out, ref))
        return res
    except Exception as e:  # secondary numbers must not take the headline down
        return f"failed: {type(e).__name__}: {e}"[:300]


if __name__ == "__main__":
    sys.exit(main())
