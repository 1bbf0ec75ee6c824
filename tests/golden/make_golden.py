"""Generates tests/golden/*.npz from the REFERENCE's own host code.

Run where a checkout of the reference is available (its location: the CSRSPMM_REFERENCE
environment variable or the REFERENCE variable of oracle/Makefile):

    make -C oracle ref && python tests/golden/make_golden.py

Every expected output in the fixtures is produced by the reference's ``dense2csr`` and
``dense_gemm_cpu`` (src/host/csr_utils.cpp:70-111, src/host/dense_utils.cpp:109-126), compiled
unmodified into oracle/_ref with contraction off, applied to the densified A.  Inputs come from
the seeded generators of this repository and are stored in full for the small cases; for the
1024x1024 case only the seed, the input checksums and the expected C are stored.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import oracle  # noqa: E402
from csrspmm_b200 import generators as G  # noqa: E402

OUT = Path(__file__).resolve().parent


def small_cases():
    """name -> (M, Kd, Nd, row lengths or density, seed, alpha, beta)"""
    yield "ragged_8x8x16", dict(M=8, Kd=8, Nd=16, lengths=[0, 1, 8, 0, 3, 5, 0, 2], seed=11, alpha=1.0, beta=1.0)
    yield "tail_13x29x7", dict(M=13, Kd=29, Nd=7, density=0.3, seed=12, alpha=1.5, beta=-0.5)
    yield "empty_5x6x4", dict(M=5, Kd=6, Nd=4, lengths=[0, 0, 0, 0, 0], seed=13, alpha=2.0, beta=0.25)
    yield "square_64x64x32", dict(M=64, Kd=64, Nd=32, density=0.3, seed=14, alpha=1.0, beta=0.0)
    yield "wide_33x128x260", dict(M=33, Kd=128, Nd=260, density=0.2, seed=15, alpha=-1.0, beta=0.5)
    yield "longrow_4x512x64", dict(M=4, Kd=512, Nd=64, lengths=[512, 0, 300, 1], seed=16, alpha=1.0, beta=0.5)


def main():
    ref = oracle.Reference()
    for name, c in small_cases():
        p = G.random_csr(c["M"], c["Kd"], c["Nd"], c.get("density", 0.0), c["seed"],
                         lengths=np.array(c["lengths"]) if "lengths" in c else None)
        rng = np.random.default_rng(c["seed"] + 1000)
        C0 = rng.standard_normal((p.M, p.Nd), dtype=np.float32)
        A = ref.csr2dense(p.M, p.Kd, p.row_ptr, p.col_idx, p.values) if p.nnz else np.zeros((p.M, p.Kd), np.float32)
        rp, ci, va, mx = ref.dense2csr(A)
        assert (rp == p.row_ptr).all() and (ci == p.col_idx).all() and (va == p.values).all()
        expect = ref.dense_gemm_cpu(A, p.B, C0, c["alpha"], c["beta"])
        np.savez_compressed(OUT / f"{name}.npz", row_ptr=p.row_ptr, col_idx=p.col_idx, values=p.values, B=p.B,
                            C0=C0, alpha=np.float32(c["alpha"]), beta=np.float32(c["beta"]), expect=expect,
                            max_row_nnz=np.int32(mx))
        print(name, "nnz", p.nnz, "max_row", mx)

    # BASELINE config 1 (1024 x 1024, p = 0.01, Nd = 64, seed 0): C = A*B, and the reference's
    # test setting alpha = 1, beta = 0.5 (tests/test_csrspmm.cu:19-20)
    p = G.make("cfg1_check")
    A = ref.csr2dense(p.M, p.Kd, p.row_ptr, p.col_idx, p.values)
    rp, ci, va, mx = ref.dense2csr(A)
    assert (rp == p.row_ptr).all() and (ci == p.col_idx).all() and (va == p.values).all()
    C0 = np.random.default_rng(1000).standard_normal((p.M, p.Nd), dtype=np.float32)
    np.savez_compressed(
        OUT / "cfg1_check.npz",
        nnz=np.int64(p.nnz), max_row_nnz=np.int32(mx),
        row_ptr_sum=np.int64(p.row_ptr.astype(np.int64).sum()), col_sum=np.int64(p.col_idx.astype(np.int64).sum()),
        values_sum=np.float64(p.values.astype(np.float64).sum()), B_sum=np.float64(p.B.astype(np.float64).sum()),
        expect_ab=ref.dense_gemm_cpu(A, p.B, np.zeros_like(C0), 1.0, 0.0),
        expect_half=ref.dense_gemm_cpu(A, p.B, C0, 1.0, 0.5))
    print("cfg1_check nnz", p.nnz, "max_row", mx)


if __name__ == "__main__":
    main()
