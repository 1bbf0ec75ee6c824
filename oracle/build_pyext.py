"""Builds the reference's PyTorch extension UNCHANGED against this repository's library.

    python oracle/build_pyext.py <reference checkout> <output .so>

Compiles the reference's ``torch_csrspmm/binding.cpp`` and its five ``torch_csrspmm_*.cpp`` wrappers
where they lie (nothing is copied), with ``-I <repo>/include`` instead of the reference's own
headers and **without** any of the reference's ``src/device`` / ``src/host`` sources, and links the
result with ``libcsrspmm_b200.so``: the drop-in proof for the Python surface
(the reference's recipe is ``setup.py:76-84``, module name ``torch_csrspmm._C``).  Test
infrastructure: the module lands under the git-ignored ``oracle/_ref`` and only
``tests/test_gpu_pyext_dropin.py`` imports it.
"""
from __future__ import annotations

import subprocess
import sys
import sysconfig
from pathlib import Path

REPO = Path(__file__).resolve().parents[1]


def main(reference: str, out: str) -> int:
    import torch
    from torch.utils import cpp_extension as ce

    ref = Path(reference) / "torch_csrspmm"
    sources = [ref / "binding.cpp"] + sorted(ref.glob("torch_csrspmm_*.cpp"))
    out_path = Path(out)
    out_path.parent.mkdir(parents=True, exist_ok=True)
    lib_dir = REPO / "csrspmm_b200" / "lib"
    newest = max(p.stat().st_mtime for p in sources + [lib_dir / "libcsrspmm_b200.so"])
    if out_path.exists() and out_path.stat().st_mtime >= newest:
        return 0
    cuda_home = Path(ce.CUDA_HOME or "/usr/local/cuda")
    inc = [str(REPO / "include"), *ce.include_paths(), sysconfig.get_paths()["include"], str(cuda_home / "include")]
    torch_lib = str(Path(torch.__file__).parent / "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-w", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
           "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
           *[f"-I{i}" for i in inc], *map(str, sources), "-o", str(out_path),
           f"-L{lib_dir}", "-lcsrspmm_b200", f"-L{torch_lib}", "-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python",
           "-lc10_cuda", "-ltorch_cuda", f"-L{cuda_home / 'lib64'}", "-lcudart",
           f"-Wl,-rpath,{torch_lib}", "-Wl,-rpath,$ORIGIN/../../../csrspmm_b200/lib", f"-Wl,-rpath,{cuda_home / 'lib64'}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        return res.returncode
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1], sys.argv[2]))
