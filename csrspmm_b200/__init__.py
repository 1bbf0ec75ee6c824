"""csrspmm_b200 -- CSR x dense SpMM for NVIDIA B200 (sm_100a).

``C = alpha * A * B + beta * C`` with A in CSR (int32 indices, fp32 or packed e2m1 values) and
B, C dense row-major fp32.  All compute runs in hand-written CUDA kernels behind a C ABI
(``include/csrspmm_b200.h``, built into ``csrspmm_b200/lib/libcsrspmm_b200.so``); this package
is the Python face of that library for torch tensors, plus the seeded input generators and the
row partitioner used for multi-GPU runs.  The same shared object also carries the ``csrspmm::``
C++ API (``include/csrspmm``).
"""
from . import _lib
from ._lib import LibraryMissing, SpmmError

__all__ = ["_lib", "LibraryMissing", "SpmmError"]
