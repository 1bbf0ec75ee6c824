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


def test_l2_partition_probe_gives_a_clean_picture(cuda_lib):
    """The probe behind the design notes on the two L2 partitions: on a two-die GPU the SMs fall into two groups
    (every line splits them the same way or the opposite way) and a far line, once read, is as near as a near
    one; on any other GPU the probe says so.  Either answer passes; a probe that cannot tell does not."""
    import json
    exe = ROOT / "tests" / "cpp" / "_bin" / "l2_partition_probe"
    assert exe.exists(), "tests/cpp/_bin/l2_partition_probe not built (python -m csrspmm_b200.build)"
    code, out = _run([exe])
    assert code == 0, out[-2000:]
    got = json.loads(out.strip().splitlines()[-1])
    assert got["reporting"] * 10 >= got["sms"] * 9, got
    if got["two_partitions"]:
        assert sum(got["group_sizes"]) == got["reporting"] and min(got["group_sizes"]) * 4 >= got["sms"], got
        assert got["atomic_cycles_far"] > 1.5 * got["atomic_cycles_near"], got
        assert got["load_cycles_far_home"] < 0.75 * got["atomic_cycles_far"], got  # the far lines were copied near
        assert 0 < got["lines_split_the_opposite_way"] < got["lines"], got
    else:
        assert got["group_sizes"] == [0, 0], got
