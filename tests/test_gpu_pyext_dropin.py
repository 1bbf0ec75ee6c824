"""The reference's own PyTorch extension, built UNCHANGED on top of this library, run through the
protocol of the reference's tests/test_pytorch.py.

oracle/build_pyext.py compiles the reference's torch_csrspmm/binding.cpp and its five
torch_csrspmm_*.cpp wrappers against this repository's include/csrspmm headers and links them with
libcsrspmm_b200.so (no reference kernel or launcher in it): the module the reference's
torch_csrspmm/__init__.py:3-7 imports as ``._C``.  Skipped when it was not built (it needs a
checkout of the reference at build time; the built module travels with the tree).
"""
import importlib.util
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from csrspmm_b200 import generators as G

ROOT = Path(__file__).resolve().parents[1]
EXT = ROOT / "oracle" / "_ref" / "torch_csrspmm_ref" / "_C.so"

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not EXT.exists(), reason="reference extension not built (make -C oracle pyext)")]

OPS = ["csrspmm_naive", "csrspmm_warp_per_row", "csrspmm_warp_per_row_smem", "csrspmm_warp_per_row_fp4",
       "csrspmm_warp_per_row_smem_fp4"]


@pytest.fixture(scope="module")
def ext():
    spec = importlib.util.spec_from_file_location("_C", EXT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_module_exports_what_the_reference_package_imports(ext):
    assert sorted(n for n in dir(ext) if n.startswith("csrspmm")) == sorted(OPS)  # torch_csrspmm/__init__.py:3-7


def _call(ext, name, rp, ci, va, mx, B, alpha, beta):
    fn = getattr(ext, name)
    return fn(rp, ci, va, mx, B, alpha, beta) if "smem" in name else fn(rp, ci, va, B, alpha, beta)


def test_reference_test_protocol_through_the_reference_wrappers(cuda_lib, ext):
    """Shapes, data and check of tests/test_pytorch.py:41-105 (A kept where rand > 0.7, values U(0,1), B randn,
    alpha = beta = 1, allclose 1e-4 against A_dense @ B), plus the CPU oracle on every result."""
    rng = np.random.default_rng(0)
    shapes = [(4, 4, 8), (8, 8, 16)] + [(2 ** int(a), 2 ** int(b), 2 ** int(c)) for a, b, c in rng.integers(2, 11, (5, 3))]
    for M, N, K in shapes:
        p = G.random_csr(M, N, K, 0.3, seed=M * 7 + N, vlo=0.0, vhi=1.0)
        rp, ci, va, B = (torch.from_numpy(x).cuda() for x in (p.row_ptr, p.col_idx, p.values, p.B))
        mx = int(np.diff(p.row_ptr).max()) if M else 0
        want = torch.from_numpy(oracle.csr2dense(M, N, p.row_ptr, p.col_idx, p.values)).cuda() @ B
        f64, mag = oracle.spmm_f64(p.row_ptr, p.col_idx, p.values, p.B, threads=4)
        for name in OPS:
            out = _call(ext, name, rp, ci, va, mx, B, 1, 1)
            torch.cuda.synchronize()
            assert out.shape == (M, K) and out.dtype == torch.float32 and out.is_cuda
            assert torch.allclose(out, want, atol=1e-4, rtol=1e-4), (name, M, N, K)
            assert (np.abs(out.cpu().numpy() - f64) <= 1e-5 * mag + 1e-6).all(), (name, M, N, K)


def test_reference_wrappers_on_an_even_and_a_skewed_matrix(cuda_lib, ext):
    """The wrappers that carry no max_row_nnz leave CSRMatrix::max_row_nnz unset
    (torch_csrspmm/torch_csrspmm_warp_per_row.cpp:34-40): the launchers measure the longest row themselves,
    so an even matrix still gets the whole-row kernel (bit-exact) and a skewed one the merge-path kernel."""
    even = G.make("cfg2_medium")
    t = [torch.from_numpy(x).cuda() for x in (even.row_ptr, even.col_idx, even.values, even.B)]
    want = oracle.spmm(even.row_ptr, even.col_idx, even.values, even.B, fused=True, threads=4)
    for name in ("csrspmm_naive", "csrspmm_warp_per_row", "csrspmm_warp_per_row_fp4"):
        out = _call(ext, name, *t[:3], 0, t[3], 1.0, 0.0)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), want), name  # sequential sums: the whole-row kernel ran
    skew = G.make("cfg3_powerlaw", scale=64)
    t = [torch.from_numpy(x).cuda() for x in (skew.row_ptr, skew.col_idx, skew.values, skew.B)]
    f64, mag = oracle.spmm_f64(skew.row_ptr, skew.col_idx, skew.values, skew.B, threads=4)
    for name in OPS:
        out = _call(ext, name, *t[:3], 3, t[3], 2.0, 0.0)  # a stale, far too small max_row_nnz on purpose
        torch.cuda.synchronize()
        assert (np.abs(out.cpu().numpy() - 2.0 * f64) <= 2e-5 * mag + 1e-6).all(), name
