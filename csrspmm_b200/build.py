"""Builds libcsrspmm_b200.so (kernels + C ABI + the csrspmm C++ API) in-tree with nvcc.

    python -m csrspmm_b200.build [--force] [--verbose]

Everything is compiled for sm_100a only.  Objects go to ``csrspmm_b200/_obj`` and the library
to ``csrspmm_b200/lib/libcsrspmm_b200.so``; a source is recompiled when it, or any header of
the package, is newer than its object.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ = PKG / "_obj"
LIB_DIR = PKG / "lib"
LIB = LIB_DIR / "libcsrspmm_b200.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler",
              "-fPIC,-ffp-contract=off", "-Xptxas", "-v",
              "-DCSRSPMM_B200_BUILD"]


def nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or add it to PATH")
    return cand


CMP_SRC = CSRC / "cmp" / "cusparse_cmp.cu"
CMP_LIB = LIB_DIR / "libcsrspmm_b200_cusparse_cmp.so"


def sources() -> list[Path]:
    """Sources of the SpMM library itself (the cuSPARSE comparator under cmp/ is a separate object)."""
    return sorted(p for p in list(CSRC.rglob("*.cu")) + list(CSRC.rglob("*.cpp")) if p.parent.name != "cmp")


def build_comparator() -> Path:
    """libcsrspmm_b200_cusparse_cmp.so: cusparseSpMM timed on the bench's buffers (bench.py only)."""
    LIB_DIR.mkdir(exist_ok=True)
    if CMP_LIB.exists() and CMP_LIB.stat().st_mtime >= CMP_SRC.stat().st_mtime:
        return CMP_LIB
    cmd = [nvcc(), *ARCH_FLAGS, "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-ccbin",
           shutil.which("g++") or "g++", "-o", str(CMP_LIB), str(CMP_SRC), "-lcusparse"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {CMP_SRC}:\n{res.stdout}\n{res.stderr}")
    return CMP_LIB


def headers() -> list[Path]:
    return sorted(list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h")) + list((ROOT / "include").rglob("*.h"))
                  + list((ROOT / "include").rglob("*.cuh")))


def _compile(src: Path, obj: Path, verbose: bool) -> str:
    cmd = [nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(ROOT / "include"), "-I", str(CSRC), "-x", "cu",
           "-c", str(src), "-o", str(obj)]
    # host-only sources do not need the ccbin to use gcc from the environment's CC wrapper
    cmd += ["-ccbin", shutil.which("g++") or "g++"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    log = res.stdout + res.stderr
    (obj.with_suffix(".log")).write_text(log)
    if verbose:
        print(log)
    return log


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    newest_header = max((h.stat().st_mtime for h in headers()), default=0.0)
    jobs = []
    objs = []
    for src in sources():
        obj = OBJ / (src.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
        objs.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, newest_header)
        if stale:
            jobs.append((src, obj))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(lambda j: _compile(j[0], j[1], verbose), jobs))
    if jobs or not LIB.exists():
        cmd = [nvcc(), *ARCH_FLAGS, "-shared", "-o", str(LIB), *map(str, objs), "-ccbin",
               shutil.which("g++") or "g++", "-Xlinker", "--no-undefined"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


def build_cpp_tests(verbose: bool = False) -> list[Path]:
    """Compile tests/cpp/*.cu against include/ and the library into tests/cpp/_bin/."""
    lib = build(verbose=verbose)
    src_dir = ROOT / "tests" / "cpp"
    out_dir = src_dir / "_bin"
    out_dir.mkdir(exist_ok=True)
    outs = []
    for src in sorted(src_dir.glob("*.cu")):
        exe = out_dir / src.stem
        outs.append(exe)
        if exe.exists() and exe.stat().st_mtime >= max(src.stat().st_mtime, lib.stat().st_mtime):
            continue
        cmd = [nvcc(), *ARCH_FLAGS, "-O2", "-std=c++17", "-lineinfo", "-ccbin", shutil.which("g++") or "g++",
               "-I", str(ROOT / "include"), "-o", str(exe), str(src), "-L", str(LIB_DIR), "-lcsrspmm_b200",
               "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../../csrspmm_b200/lib"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    return outs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ns = ap.parse_args(argv)
    print(build(ns.force, ns.verbose))
    for exe in build_cpp_tests(ns.verbose):
        print(exe)
    print(build_comparator())
    return 0


if __name__ == "__main__":
    sys.exit(main())
