"""The CPU oracle against the reference: golden vectors made by the reference's own host code
(tests/golden/make_golden.py), the live reference build when oracle/_ref exists, and internal
consistency (fp32 vs fp64, fused vs unfused, coverage rule of the float4 kernels)."""
from pathlib import Path

import numpy as np
import pytest

import oracle
from csrspmm_b200 import generators as G

GOLDEN = Path(__file__).resolve().parent / "golden"
SMALL = sorted(p.stem for p in GOLDEN.glob("*.npz") if p.stem != "cfg1_check")


def test_golden_files_present():
    assert len(SMALL) >= 6 and (GOLDEN / "cfg1_check.npz").exists()


@pytest.mark.parametrize("name", SMALL)
def test_oracle_matches_reference_golden_bit_for_bit(name):
    g = np.load(GOLDEN / f"{name}.npz")
    got = oracle.spmm(g["row_ptr"], g["col_idx"], g["values"], g["B"], g["C0"], float(g["alpha"]),
                      float(g["beta"]), fused=False)
    # dense_gemm_cpu adds the products of the explicit zeros too; x + 0 = x, so the unfused
    # oracle must agree exactly (np == treats -0 and +0 as equal)
    assert np.array_equal(got, g["expect"])
    fused = oracle.spmm(g["row_ptr"], g["col_idx"], g["values"], g["B"], g["C0"], float(g["alpha"]),
                        float(g["beta"]), fused=True)
    np.testing.assert_allclose(fused, g["expect"], rtol=1e-5, atol=1e-5)


def test_oracle_matches_reference_golden_cfg1():
    g = np.load(GOLDEN / "cfg1_check.npz")
    p = G.make("cfg1_check")
    assert p.nnz == int(g["nnz"])
    assert int(p.row_ptr.astype(np.int64).sum()) == int(g["row_ptr_sum"])
    assert int(p.col_idx.astype(np.int64).sum()) == int(g["col_sum"])
    assert float(p.values.astype(np.float64).sum()) == float(g["values_sum"])
    assert float(p.B.astype(np.float64).sum()) == float(g["B_sum"])
    assert int(np.diff(p.row_ptr).max()) == int(g["max_row_nnz"])
    ab = oracle.spmm(p.row_ptr, p.col_idx, p.values, p.B, fused=False)
    assert np.array_equal(ab, g["expect_ab"])
    C0 = np.random.default_rng(1000).standard_normal((p.M, p.Nd), dtype=np.float32)
    half = oracle.spmm(p.row_ptr, p.col_idx, p.values, p.B, C0, 1.0, 0.5, fused=False)
    assert np.array_equal(half, g["expect_half"])
    # the order-faithful (fmaf) variant stays within the accumulation-order tolerance
    np.testing.assert_allclose(oracle.spmm(p.row_ptr, p.col_idx, p.values, p.B), g["expect_ab"], rtol=1e-5,
                               atol=1e-6)


@pytest.mark.skipif(not oracle.Reference.available(), reason="oracle/_ref not built (needs the reference checkout)")
def test_oracle_matches_live_reference():
    ref = oracle.Reference()
    p = G.random_csr(96, 80, 24, 0.15, seed=3)
    A = oracle.csr2dense(p.M, p.Kd, p.row_ptr, p.col_idx, p.values)
    assert np.array_equal(ref.csr2dense(p.M, p.Kd, p.row_ptr, p.col_idx, p.values), A)
    rp, ci, va, mx = ref.dense2csr(A)
    orp, oci, ova, omx = oracle.dense2csr(A)
    assert np.array_equal(rp, orp) and np.array_equal(ci, oci) and np.array_equal(va, ova) and mx == omx
    assert np.array_equal(rp, p.row_ptr) and np.array_equal(ci, p.col_idx)
    C0 = np.random.default_rng(4).standard_normal((p.M, p.Nd), dtype=np.float32)
    for alpha, beta in ((1.0, 0.0), (1.0, 0.5), (-2.0, 1.0)):
        expect = ref.dense_gemm_cpu(A, p.B, C0, alpha, beta)
        got = oracle.spmm(p.row_ptr, p.col_idx, p.values, p.B, C0, alpha, beta, fused=False)
        assert np.array_equal(got, expect)
        assert ref.dense_compare(got, expect, 0.0)
    # tolerance filter of dense2csr (fabs(v) > tol)
    rp2, ci2, va2, _ = ref.dense2csr(A, 0.5)
    orp2, oci2, ova2, _ = oracle.dense2csr(A, 0.5)
    assert np.array_equal(rp2, orp2) and np.array_equal(ci2, oci2) and np.array_equal(va2, ova2)
    assert ref.compression_ratio(p.M, p.Kd, p.nnz) == pytest.approx(p.M * p.Kd / (2 * p.nnz + p.M + 1))


def test_beta_zero_never_reads_c():
    p = G.random_csr(17, 23, 9, 0.3, seed=5)
    poison = np.full((p.M, p.Nd), np.nan, np.float32)
    out = oracle.spmm(p.row_ptr, p.col_idx, p.values, p.B, poison, 1.0, 0.0)
    assert np.isfinite(out).all()
    assert np.array_equal(out, oracle.spmm(p.row_ptr, p.col_idx, p.values, p.B))


def test_float4_coverage_rule():
    # the reference's float4 kernels write only the first 4*floor(Nd/4) columns
    p = G.random_csr(10, 12, 7, 0.4, seed=6)
    C0 = np.full((p.M, p.Nd), 7.0, np.float32)
    out = oracle.spmm(p.row_ptr, p.col_idx, p.values, p.B, C0, 1.0, 0.0, ncols=4)
    full = oracle.spmm(p.row_ptr, p.col_idx, p.values, p.B)
    assert np.array_equal(out[:, :4], full[:, :4]) and (out[:, 4:] == 7.0).all()


def test_fp64_variant_bounds_fp32():
    p = G.make("cfg3_powerlaw", scale=256)
    f32 = oracle.spmm(p.row_ptr, p.col_idx, p.values, p.B, threads=2)
    f64, mag = oracle.spmm_f64(p.row_ptr, p.col_idx, p.values, p.B, threads=2)
    assert (np.abs(f32 - f64) <= 1e-5 * mag + 1e-6).all()
    rows = np.array([0, 5, p.M - 1], np.int32)
    assert np.array_equal(oracle.spmm_rows(rows, p.row_ptr, p.col_idx, p.values, p.B), f32[rows])


def test_threads_do_not_change_bits():
    p = G.random_csr(300, 200, 33, 0.05, seed=7)
    a = oracle.spmm(p.row_ptr, p.col_idx, p.values, p.B, threads=1)
    b = oracle.spmm(p.row_ptr, p.col_idx, p.values, p.B, threads=4)
    assert np.array_equal(a, b)


# ---- e2m1 codec known answers (the format is defined by this library: parity unpinned) -----------

def test_e2m1_all_code_points_round_trip():
    mags = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for code in range(16):
        v = oracle.e2m1_decode_one(code)
        assert abs(v) == mags[code & 7]
        assert np.signbit(np.float32(v)) == bool(code & 8)
        assert oracle.e2m1_encode_one(v) == code


def test_e2m1_rounding_ties_saturation_sign():
    enc = oracle.e2m1_encode_one
    assert enc(0.25) == 0 and enc(0.75) == 2 and enc(1.25) == 2 and enc(1.75) == 4
    assert enc(2.5) == 4 and enc(3.5) == 6 and enc(5.0) == 6
    assert enc(0.26) == 1 and enc(5.01) == 7 and enc(100.0) == 7 and enc(-100.0) == 15
    assert enc(-0.0) == 8 and enc(-0.2) == 8 and enc(float("nan")) == 0
    assert enc(3.0, scale=0.5) == 7 and oracle.e2m1_decode_one(7, 0.5) == 3.0


def test_e2m1_packing_order_and_odd_tail():
    v = np.array([0.5, -6.0, 1.5], np.float32)
    packed = oracle.e2m1_encode(v, 1.0)
    assert packed.tolist() == [0x1 | (0xF << 4), 0x3]
    assert np.array_equal(oracle.e2m1_decode(packed, 3, 1.0), v)
    x = np.random.default_rng(8).uniform(-1, 1, 1001).astype(np.float32)
    s = oracle.e2m1_scale(x)
    assert s == np.float32(np.abs(x).max()) / np.float32(6.0)
    d = oracle.e2m1_decode(oracle.e2m1_encode(x, s), x.size, s)
    assert np.abs(d - x).max() <= s * 1.0 + 1e-7  # widest gap between code points is 2 (4 -> 6)
    assert np.array_equal(oracle.e2m1_decode(oracle.e2m1_encode(d, s), x.size, s), d)  # idempotent
