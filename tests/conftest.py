import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_sessionstart(session):
    """A fresh checkout has no built library (binaries are not committed): build it once, here,
    when a compiler is around.  Without nvcc the tests that need the library fail loudly."""
    import shutil
    from csrspmm_b200 import _lib
    if not _lib.LIB_PATH.exists() and (shutil.which("nvcc") or Path("/usr/local/cuda/bin/nvcc").exists()):
        from csrspmm_b200 import build
        build.build()
        build.build_cpp_tests()
        build.build_comparator()


@pytest.fixture(scope="session")
def cuda_lib():
    """The kernel library on a real GPU.  Fails (never skips) when either is missing: a GPU test
    that silently ran something else would prove nothing."""
    import torch
    from csrspmm_b200 import _lib
    assert torch.cuda.is_available(), "GPU test started without a CUDA device"
    return _lib.lib()
