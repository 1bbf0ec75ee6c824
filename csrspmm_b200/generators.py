"""Seeded synthetic CSR x dense problems.

The reference's only generator, ``dense_init_random`` (src/host/dense_utils.cpp:44-65), draws a
dense matrix and cannot reach the sizes this library is measured at, so the workloads are
described here: five named configurations (Bernoulli-sparse and Zipf row-length matrices with
uniform columns) plus free-form builders for tests.

Conventions: int32 ``row_ptr``/``col_idx``; columns ascending and distinct inside a row; one
``numpy.random.default_rng(seed)`` stream consumed in the order *row lengths -> columns ->
values -> B*.  Row lengths always come from numpy on the host, so ``row_ptr`` is identical
whichever device the rest is generated on.  With ``device="cpu"`` everything is numpy and the
result is reproducible anywhere; with a CUDA device the columns, values and B come from a seeded
``torch.Generator`` on that device (fast enough for 10^8 non-zeros), reproducible for a given
torch build and GPU model.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

CONFIGS = {
    # name: parameters of BASELINE configs 1..5
    "cfg1_check": dict(kind="bernoulli", M=1024, Kd=1024, p=0.01, vlo=-1.0, vhi=1.0, Nd=64, seed=0),
    "cfg2_medium": dict(kind="bernoulli", M=16384, Kd=16384, p=0.001, vlo=-1.0, vhi=1.0, Nd=128, seed=0),
    "cfg3_powerlaw": dict(kind="zipf", M=1 << 20, Kd=1 << 20, zipf_a=2.0, mean=16.0, cap=16384, vlo=0.0,
                          vhi=1.0, Nd=64, seed=0),
    "cfg4_fp4": dict(kind="bernoulli", M=65536, Kd=65536, p=0.005, vlo=-1.0, vhi=1.0, Nd=256, seed=0),
    "cfg5_xl": dict(kind="zipf", M=1 << 22, Kd=1 << 22, zipf_a=2.2, mean=32.0, cap=65536, vlo=-1.0,
                    vhi=1.0, Nd=512, seed=0),
}


@dataclass
class Problem:
    """A = (row_ptr, col_idx, values) is M x Kd; B is Kd x Nd.  Arrays are numpy or torch."""
    name: str
    M: int
    Kd: int
    Nd: int
    row_ptr: object
    col_idx: object
    values: object
    B: object
    seed: int = 0
    meta: dict = field(default_factory=dict)

    @property
    def nnz(self) -> int:
        return int(self.col_idx.shape[0])

    def row_lengths(self) -> np.ndarray:
        rp = self.row_ptr if isinstance(self.row_ptr, np.ndarray) else self.row_ptr.cpu().numpy()
        return np.diff(rp.astype(np.int64))

    def stats(self) -> dict:
        lens = self.row_lengths()
        ci = self.col_idx
        if isinstance(ci, np.ndarray):
            col_sum = int(ci.astype(np.int64).sum())
            col_xor = int(np.bitwise_xor.reduce(ci)) if ci.size else 0
        else:
            col_sum = int(ci.sum(dtype=ci.new_empty(0, dtype=__import__("torch").int64).dtype).item())
            col_xor = None
        return dict(M=self.M, Kd=self.Kd, Nd=self.Nd, nnz=self.nnz, mean_row=float(lens.mean()) if lens.size else 0.0,
                    median_row=float(np.median(lens)) if lens.size else 0.0,
                    max_row=int(lens.max()) if lens.size else 0, empty_rows=int((lens == 0).sum()),
                    col_sum=col_sum, col_xor=col_xor)


# ---- row lengths (always numpy, host) -----------------------------------------------------------

def bernoulli_lengths(rng: np.random.Generator, M: int, Kd: int, p: float) -> np.ndarray:
    """Row lengths of a matrix whose entries are non-zero independently with probability p."""
    return rng.binomial(Kd, p, size=M).astype(np.int64)


def zipf_lengths(rng: np.random.Generator, M: int, Kd: int, a: float, mean: float, cap: int) -> np.ndarray:
    """len = clip(rint(z * s), 1, cap) with z ~ Zipf(a) and the scalar s found by bisection so
    that the mean length is `mean` (a single rescale misses because of the clipping)."""
    cap = int(min(cap, Kd))
    z = rng.zipf(a, size=M).astype(np.float64)

    def lens_for(s):
        return np.clip(np.rint(z * s), 1, cap)

    lo, hi = 1e-6, 1.0
    while lens_for(hi).mean() < mean and hi < 1e12:
        hi *= 2.0
    for _ in range(80):
        mid = 0.5 * (lo + hi)
        if lens_for(mid).mean() < mean:
            lo = mid
        else:
            hi = mid
    return lens_for(hi).astype(np.int64)


# ---- columns --------------------------------------------------------------------------------

def _columns_numpy(rng: np.random.Generator, lens: np.ndarray, Kd: int) -> np.ndarray:
    """Distinct uniform columns per row, ascending, by sort + redraw of the (rare) repeats."""
    M = lens.shape[0]
    nnz = int(lens.sum())
    out = np.empty(nnz, np.int32)
    if nnz == 0:
        return out
    rp = np.concatenate([[0], np.cumsum(lens)])
    dense_rows = np.nonzero(lens * 2 > Kd)[0]  # redraw would crawl: draw these by permutation
    sparse_mask = np.ones(M, bool)
    sparse_mask[dense_rows] = False
    for r in dense_rows:
        out[rp[r]:rp[r + 1]] = np.sort(rng.choice(Kd, size=int(lens[r]), replace=False)).astype(np.int32)
    sl = np.where(sparse_mask, lens, 0)
    n = int(sl.sum())
    if n:
        rows = np.repeat(np.arange(M, dtype=np.int64), sl)
        key = rows * Kd + rng.integers(0, Kd, size=n, dtype=np.int64)
        key.sort()
        while True:
            dup = np.nonzero(key[1:] == key[:-1])[0] + 1
            if dup.size == 0:
                break
            key[dup] = (key[dup] // Kd) * Kd + rng.integers(0, Kd, size=dup.size, dtype=np.int64)
            key.sort()
        dst = np.repeat(rp[:-1], sl) + (np.arange(n, dtype=np.int64) - np.repeat(np.cumsum(sl) - sl, sl))
        out[dst] = (key % Kd).astype(np.int32)
    return out


def _columns_torch(gen, lens: np.ndarray, Kd: int, device):
    import torch
    M = lens.shape[0]
    nnz = int(lens.sum())
    if nnz == 0:
        return torch.empty(0, dtype=torch.int32, device=device)
    if (lens * 2 > Kd).any():
        raise ValueError("device generation expects rows shorter than Kd/2; use device='cpu'")
    lens_t = torch.from_numpy(lens).to(device)
    rows = torch.repeat_interleave(torch.arange(M, dtype=torch.int64, device=device), lens_t)
    key = rows * Kd + torch.randint(0, Kd, (nnz,), generator=gen, device=device, dtype=torch.int64)
    del rows
    key = torch.sort(key).values
    while True:
        dup = torch.nonzero(key[1:] == key[:-1]).flatten() + 1
        if dup.numel() == 0:
            break
        fresh = torch.randint(0, Kd, (dup.numel(),), generator=gen, device=device, dtype=torch.int64)
        key[dup] = torch.div(key[dup], Kd, rounding_mode="floor") * Kd + fresh
        key = torch.sort(key).values
    return (key % Kd).to(torch.int32)


# ---- builders -------------------------------------------------------------------------------

def from_lengths(name: str, lens: np.ndarray, Kd: int, Nd: int, rng: np.random.Generator, vlo: float,
                 vhi: float, seed: int, device="cpu") -> Problem:
    M = int(lens.shape[0])
    nnz = int(lens.sum())
    if nnz >= 2 ** 31:
        raise ValueError("nnz does not fit int32")
    row_ptr = np.zeros(M + 1, np.int32)
    np.cumsum(lens, out=row_ptr[1:])
    if str(device) == "cpu":
        col_idx = _columns_numpy(rng, lens, Kd)
        values = rng.uniform(vlo, vhi, size=nnz).astype(np.float32)
        B = rng.standard_normal(size=(Kd, Nd), dtype=np.float32)
        return Problem(name, M, Kd, Nd, row_ptr, col_idx, values, B, seed)
    import torch
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    col_idx = _columns_torch(gen, lens, Kd, device)
    values = torch.empty(nnz, dtype=torch.float32, device=device).uniform_(vlo, vhi, generator=gen)
    B = torch.randn((Kd, Nd), dtype=torch.float32, device=device, generator=gen)
    return Problem(name, M, Kd, Nd, torch.from_numpy(row_ptr).to(device), col_idx, values, B, seed)


def make(name: str, *, scale: int = 1, Nd: int | None = None, seed: int | None = None, device="cpu") -> Problem:
    """Build one of CONFIGS.  ``scale`` divides M, Kd (and the row-length cap) for quick tests;
    the per-row statistics (mean length, Zipf exponent) stay those of the full configuration."""
    cfg = dict(CONFIGS[name])
    M, Kd = max(cfg["M"] // scale, 1), max(cfg["Kd"] // scale, 1)
    nd = int(Nd if Nd is not None else cfg["Nd"])
    sd = int(cfg["seed"] if seed is None else seed)
    rng = np.random.default_rng(sd)
    if cfg["kind"] == "bernoulli":
        # keep the expected row length of the full configuration when Kd shrinks
        p = min(cfg["p"] * cfg["Kd"] / Kd, 0.45)
        lens = bernoulli_lengths(rng, M, Kd, p)
    else:
        lens = zipf_lengths(rng, M, Kd, cfg["zipf_a"], cfg["mean"], max(min(cfg["cap"] // scale, Kd // 2), 1))
    prob = from_lengths(name if scale == 1 else f"{name}/{scale}", lens, Kd, nd, rng, cfg["vlo"], cfg["vhi"], sd,
                        device)
    prob.meta.update(cfg, scale=scale)
    return prob


def random_csr(M: int, Kd: int, Nd: int, density: float, seed: int, *, vlo=-1.0, vhi=1.0,
               lengths: np.ndarray | None = None) -> Problem:
    """Free-form numpy problem for tests: Bernoulli(density) rows, or explicit row lengths."""
    rng = np.random.default_rng(seed)
    lens = bernoulli_lengths(rng, M, Kd, density) if lengths is None else np.asarray(lengths, np.int64)
    return from_lengths(f"random{M}x{Kd}x{Nd}", lens, Kd, Nd, rng, vlo, vhi, seed)


# ---- algorithmic traffic ----------------------------------------------------------------------

def min_bytes(M: int, Nd: int, nnz: int, touched_b_rows: int, beta: float = 0.0, value_bytes: float = 4.0) -> float:
    """Compulsory bytes of one SpMM: every stored (index, value) once, row_ptr once, each B row
    that is referenced once, C written once (and read once when beta != 0)."""
    b = nnz * (4.0 + value_bytes) + (M + 1) * 4.0 + touched_b_rows * Nd * 4.0 + M * Nd * 4.0
    if beta != 0.0:
        b += M * Nd * 4.0
    return b


def touched_rows(col_idx, Kd: int) -> int:
    """Distinct columns of A = rows of B that are read at least once."""
    if isinstance(col_idx, np.ndarray):
        return int(np.unique(col_idx).size)
    import torch
    seen = torch.zeros(Kd, dtype=torch.bool, device=col_idx.device)
    seen[col_idx.long()] = True
    return int(seen.sum().item())
