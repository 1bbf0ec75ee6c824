"""Drop-in for the reference's ``torch_csrspmm`` package (torch_csrspmm/__init__.py:10-23 there):
the same five functions with the same positional arguments, served by the sm_100a kernel library
through its C ABI instead of a pybind extension."""
from csrspmm_b200.ops import (csrspmm_naive, csrspmm_warp_per_row, csrspmm_warp_per_row_fp4,
                              csrspmm_warp_per_row_smem, csrspmm_warp_per_row_smem_fp4)

__all__ = ["csrspmm_naive", "csrspmm_warp_per_row", "csrspmm_warp_per_row_smem", "csrspmm_warp_per_row_fp4",
           "csrspmm_warp_per_row_smem_fp4"]
