"""Seeded input generators: structure invariants, reproducibility, traffic accounting."""
import numpy as np
import pytest

from csrspmm_b200 import generators as G


def _check_structure(p):
    rp = p.row_ptr.astype(np.int64)
    assert p.row_ptr.dtype == np.int32 and p.col_idx.dtype == np.int32 and p.values.dtype == np.float32
    assert rp[0] == 0 and rp[-1] == p.nnz and (np.diff(rp) >= 0).all()
    assert p.nnz == 0 or (p.col_idx.min() >= 0 and p.col_idx.max() < p.Kd)
    d = np.diff(p.col_idx.astype(np.int64))
    inside = np.ones(max(p.nnz - 1, 0), bool)
    starts = rp[1:-1]
    inside[starts[(starts > 0) & (starts < p.nnz)] - 1] = False
    assert (d[inside] > 0).all(), "columns must be ascending and distinct inside a row"
    assert p.B.shape == (p.Kd, p.Nd) and p.B.dtype == np.float32


@pytest.mark.parametrize("name,scale", [("cfg1_check", 1), ("cfg2_medium", 1), ("cfg3_powerlaw", 64),
                                        ("cfg4_fp4", 32), ("cfg5_xl", 256)])
def test_configs(name, scale):
    p = G.make(name, scale=scale)
    _check_structure(p)
    cfg = G.CONFIGS[name]
    s = p.stats()
    if cfg["kind"] == "bernoulli":
        assert abs(s["mean_row"] - cfg["p"] * cfg["Kd"]) < 0.05 * cfg["p"] * cfg["Kd"] + 0.5
    else:
        assert abs(s["mean_row"] - cfg["mean"]) < 0.05 * cfg["mean"]
        assert s["max_row"] <= max(min(cfg["cap"] // scale, p.Kd // 2), 1) and s["median_row"] < s["mean_row"]
    lo, hi = cfg["vlo"], cfg["vhi"]
    assert p.values.min() >= lo and p.values.max() < hi
    q = G.make(name, scale=scale)
    assert np.array_equal(p.col_idx, q.col_idx) and np.array_equal(p.values, q.values) and np.array_equal(p.B, q.B)


def test_dense_rows_and_explicit_lengths():
    p = G.random_csr(6, 16, 4, 0.0, seed=1, lengths=np.array([16, 0, 15, 9, 1, 0]))
    _check_structure(p)
    assert np.diff(p.row_ptr).tolist() == [16, 0, 15, 9, 1, 0]
    assert p.col_idx[:16].tolist() == list(range(16))


def test_min_bytes_formula():
    # nnz*(idx+val) + rowptr + touched B rows + C (+ C read when beta != 0)
    assert G.min_bytes(10, 4, 7, 5) == 7 * 8 + 11 * 4 + 5 * 16 + 10 * 16
    assert G.min_bytes(10, 4, 7, 5, beta=0.5) == G.min_bytes(10, 4, 7, 5) + 10 * 16
    assert G.min_bytes(10, 4, 8, 5, value_bytes=0.5) == 8 * 4.5 + 11 * 4 + 5 * 16 + 10 * 16
    p = G.make("cfg1_check")
    assert G.touched_rows(p.col_idx, p.Kd) == np.unique(p.col_idx).size
