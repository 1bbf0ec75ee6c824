"""The csrspmm:: C++ API on a GPU: this repository's own C++ test program, and -- when they were
built from a reference checkout -- the reference's unmodified test and benchmark programs linked
against this library."""
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _run(cmd, timeout=300):
    res = subprocess.run([str(c) for c in cmd], capture_output=True, text=True, timeout=timeout)
    return res.returncode, res.stdout + res.stderr


def test_cpp_api_program(cuda_lib):
    exe = ROOT / "tests" / "cpp" / "_bin" / "test_cpp_api"
    assert exe.exists(), "tests/cpp/_bin/test_cpp_api not built (python -m csrspmm_b200.build)"
    code, out = _run([exe])
    assert code == 0 and "ALL OK" in out, out[-3000:]


REF_TEST = ROOT / "oracle" / "_ref" / "ref_test_csrspmm"
REF_BENCH = ROOT / "oracle" / "_ref" / "ref_bench_csrspmm"


@pytest.mark.skipif(not REF_TEST.exists(), reason="reference programs not built (needs the reference checkout)")
@pytest.mark.parametrize("algo", ["Naive", "NaiveSmem", "WarpPerRow", "WarpPerRowFp4", "WarpPerRowSmem",
                                  "WarpPerRowSmemFp4"])
def test_reference_test_program_passes_unchanged(cuda_lib, algo):
    # the reference's tests/test_csrspmm.cu, compiled as it is, with this library underneath
    code, out = _run([REF_TEST, "-M", 512, "-N", 384, "-K", 128, "-s", 0.9, "-a", 1.0, "-b", 0.5, "-algo", algo])
    assert code == 0 and f"Pass: {algo}" in out, out[-2000:]


@pytest.mark.skipif(not REF_BENCH.exists(), reason="reference programs not built (needs the reference checkout)")
def test_reference_benchmark_program_runs_unchanged(cuda_lib):
    code, out = _run([REF_BENCH, "-M", 1024, "-N", 1024, "-K", 128, "-s", 0.95, "-algo", "WarpPerRowFp4"])
    assert code == 0 and "GFLOPS" in out, out[-2000:]
