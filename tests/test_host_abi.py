"""Host-side checks of the C ABI that need no GPU: the library loads, exports every declared
symbol, and its host-only logic (argument checks, kernel selection, workspace sizing, CSR
validation, row partition, e2m1 codec) behaves."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

import oracle
from csrspmm_b200 import _lib, distributed as D, generators as G, ops

ROOT = Path(__file__).resolve().parents[1]


def test_library_loads_and_exports_every_declared_symbol():
    L = _lib.lib()
    assert L.csrspmm_b200_abi_version() == _lib.ABI_VERSION == 2
    header = (ROOT / "include" / "csrspmm_b200.h").read_text()
    declared = set(re.findall(r"^(?:int|int32_t|size_t|float|const char\*)\s+(csrspmm_b200_[a-z0-9_]+)\(", header, re.M))
    assert declared == set(_lib.EXPORTED_SYMBOLS)
    for name in declared:
        assert hasattr(L, name), name


def test_cpp_api_symbols_exported():
    # the csrspmm:: C++ surface lives in the same shared object (mangled names)
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", str(_lib.LIB_PATH)], capture_output=True, text=True).stdout
    for needle in ("csrspmm4spmm", "csrspmm15parse_algorithm", "csrspmm12launch_naive", "csrspmm17launch_naive_smem",
                   "csrspmm19launch_warp_per_row", "csrspmm23launch_warp_per_row_fp4",
                   "csrspmm24launch_warp_per_row_smem", "csrspmm28launch_warp_per_row_smem_fp4", "csrspmm9dense2csr",
                   "csrspmm9csr2dense", "csrspmm15csr_host2device", "csrspmm15csr_device2host",
                   "csrspmm14csr_alloc_host", "csrspmm16csr_alloc_device", "csrspmm13csr_free_host",
                   "csrspmm15csr_free_device", "csrspmm9print_csr", "csrspmm17compression_ratio",
                   "csrspmm16dense_alloc_host", "csrspmm18dense_alloc_device", "csrspmm15dense_free_host",
                   "csrspmm17dense_free_device", "csrspmm17dense_host2device", "csrspmm17dense_device2host",
                   "csrspmm17dense_init_random", "csrspmm11print_dense", "csrspmm13dense_compare",
                   "csrspmm14dense_gemm_cpu"):
        assert needle in out, needle


def test_args_struct_layout_is_checked():
    L = _lib.lib()
    a = _lib.make_args(4, 4, 4, 4)
    assert C.sizeof(_lib.Args) == 144
    assert L.csrspmm_b200_select_kernel(C.byref(a)) > 0
    a.struct_size = 8
    assert L.csrspmm_b200_select_kernel(C.byref(a)) == -_lib.ERR_BAD_ARG
    assert b"struct_size" in L.csrspmm_b200_last_error()


@pytest.mark.parametrize("field,value", [("M", -1), ("nnz", 1 << 31), ("ldb", 3), ("value_format", 9),
                                         ("entry", 6), ("kernel", 7)])
def test_bad_arguments_are_rejected(field, value):
    a = _lib.make_args(8, 8, 4, 10)
    setattr(a, field, value)
    assert _lib.lib().csrspmm_b200_select_kernel(C.byref(a)) == -_lib.ERR_BAD_ARG
    assert _lib.lib().csrspmm_b200_spmm(C.byref(a), None) == _lib.ERR_BAD_ARG  # rejected before any CUDA call


def test_null_pointers_are_rejected_before_any_cuda_call():
    a = _lib.make_args(8, 8, 4, 10)
    assert _lib.lib().csrspmm_b200_spmm(C.byref(a), None) == _lib.ERR_BAD_ARG
    assert b"null" in _lib.lib().csrspmm_b200_last_error()


def test_kernel_selection():
    sel = ops.selected_kernel
    # short even rows with a trustworthy max_row_nnz -> row kernel
    assert sel(16384, 16384, 128, 268000, max_row_nnz=38) == "row"
    # few rows: still the row kernel (its deep-unroll variant for an underfilled chip)
    assert sel(1024, 2048, 128, 419_517, max_row_nnz=470) == "row"
    assert sel(512, 1024, 64, 52_205, max_row_nnz=140) == "row"
    assert sel(4096, 4096, 128, 3_356_995, max_row_nnz=900) == "row"
    # unknown or skewed row lengths -> merge-path
    assert sel(16384, 16384, 128, 268000) == "merge"
    assert sel(1 << 20, 1 << 20, 64, 16_000_000, max_row_nnz=16384) == "merge"
    # 2 KB rows of a B far larger than L2 -> bulk-copy (TMA) kernel, whatever the entry point
    assert sel(1 << 22, 1 << 22, 512, 134_000_000) == "tma"
    assert sel(1 << 22, 1 << 22, 512, 134_000_000, entry="warp_per_row_smem_fp4", max_row_nnz=65536) == "tma"
    assert sel(1 << 22, 1 << 22, 400, 134_000_000) == "tma"
    # ... but not for narrower rows, an L2-sized B, even rows, or a layout without 16-byte rows
    assert sel(1 << 22, 1 << 22, 256, 134_000_000) == "merge"
    assert sel(65536, 65536, 512, 21_000_000) == "merge"
    assert sel(1 << 22, 1 << 22, 512, 134_000_000, max_row_nnz=40) == "row"
    assert sel(1 << 22, 1 << 22, 510, 134_000_000) == "merge"
    assert sel(1 << 22, 1 << 22, 512, 134_000_000, aligned=False) == "merge"
    assert sel(65536, 65536, 256, 21_000_000, entry="warp_per_row_smem", max_row_nnz=400) == "row"
    # pinned kernels are honoured or refused, never silently replaced
    assert sel(100, 100, 64, 1000, kernel="row") == "row"
    assert sel(100, 100, 64, 1000, kernel="tma") == "tma"
    with pytest.raises(_lib.SpmmError) as e:
        sel(100, 100, 66, 1000, kernel="tma")
    assert e.value.status == _lib.ERR_UNSUPPORTED


def test_force_kernel_environment(monkeypatch):
    monkeypatch.setenv("CSRSPMM_FORCE_KERNEL", "merge")
    assert ops.selected_kernel(16384, 16384, 128, 268000, max_row_nnz=38) == "merge"
    monkeypatch.setenv("CSRSPMM_FORCE_KERNEL", "tma")
    assert ops.selected_kernel(100, 100, 66, 1000, max_row_nnz=12) == "row"  # cannot run -> AUTO
    assert ops.selected_kernel(100, 100, 64, 1000, kernel="row") == "row"    # explicit pin wins


def test_host_round_trip_scratch_covers_every_row_block():
    """spmm_host multiplies row blocks out of one scratch area.  A block can fall under the merge kernel's
    small-problem threshold (smaller tiles, more carry rows) although the whole matrix does not: the arena
    must be sized for that."""
    M, Kd, Nd, nnz = 40000, 40000, 512, 420000
    L = _lib.lib()
    whole = _lib.make_args(M, Kd, Nd, nnz)
    al = lambda v: -(-v // 256) * 256
    others = al((M + 1) * 4) + al(nnz * 4) + al(nnz * 4) + al(Kd * Nd * 4) + al(M * Nd * 4) + 256
    scratch = L.csrspmm_b200_host_arena_bytes(C.byref(whole)) - others
    # a block that holds a hub row of 200 000 entries and little else
    block = _lib.make_args(100, Kd, Nd, 200300, kernel=_lib.KERNEL_MERGE)
    assert L.csrspmm_b200_workspace_bytes(C.byref(block)) <= scratch
    assert L.csrspmm_b200_workspace_bytes(C.byref(whole)) <= scratch


def test_schedule_entry_points_reject_bad_arguments_before_any_cuda_call():
    L = _lib.lib()
    a = _lib.make_args(8, 8, 4, 10, row_ptr=256, col_idx=256)
    h = C.c_void_p(None)
    assert L.csrspmm_b200_schedule_create(C.byref(a), None, None, None) == _lib.ERR_BAD_ARG
    bad = _lib.ScheduleOptions(4, 0, 0, 0)
    assert L.csrspmm_b200_schedule_create(C.byref(a), C.byref(bad), C.byref(h), None) == _lib.ERR_BAD_ARG
    a.row_ptr_base = 2
    assert L.csrspmm_b200_schedule_create(C.byref(a), None, C.byref(h), None) == _lib.ERR_BAD_ARG
    a.row_ptr_base, a.row_ptr = 0, None
    assert L.csrspmm_b200_schedule_create(C.byref(a), None, C.byref(h), None) == _lib.ERR_BAD_ARG
    assert h.value is None
    assert L.csrspmm_b200_schedule_destroy(None) == _lib.OK
    info = _lib.ScheduleInfo()
    assert L.csrspmm_b200_schedule_info_get(None, C.byref(info)) == _lib.ERR_BAD_ARG


def test_workspace_depends_on_sizes_only():
    w = ops.workspace_bytes(1 << 20, 1 << 20, 64, 16_777_216)
    tiles = -(-((1 << 20) + 16_777_216) // 1024)
    assert w == -(-tiles * 4 // 256) * 256 + tiles * 64 * 4
    assert ops.workspace_bytes(0, 0, 64, 0) == 0
    assert ops.workspace_bytes(10, 10, 5, 7) >= 8 * 4 + 4


def _validate(rp, ci, Kd):
    flags = C.c_uint32(0)
    rp, ci = np.asarray(rp, np.int32), np.asarray(ci, np.int32)
    st = _lib.lib().csrspmm_b200_validate_csr_host(len(rp) - 1, Kd, len(ci), rp.ctypes.data, ci.ctypes.data,
                                                   C.byref(flags))
    return st, flags.value


def test_validate_csr_host():
    assert _validate([0, 2, 2, 3], [0, 4, 1], 5) == (_lib.OK, 0)
    assert _validate([0], [], 5) == (_lib.OK, 0)
    assert _validate([1, 2, 2, 3], [0, 4, 1], 5) == (_lib.ERR_INVALID_CSR, _lib.CSR_BAD_ROWPTR0)
    assert _validate([0, 2, 2, 2], [0, 4, 1], 5) == (_lib.ERR_INVALID_CSR, _lib.CSR_BAD_ROWPTR_END)
    st, fl = _validate([0, 2, 1, 3], [0, 4, 1], 5)
    assert st == _lib.ERR_INVALID_CSR and fl & _lib.CSR_NOT_MONOTONE
    assert _validate([0, 2, 2, 3], [0, 5, 1], 5) == (_lib.ERR_INVALID_CSR, _lib.CSR_COL_RANGE)
    assert _validate([0, 2, 2, 3], [0, -1, 1], 5)[0] == _lib.ERR_INVALID_CSR
    # unsorted / repeated columns are reported but allowed
    assert _validate([0, 2, 2, 3], [4, 0, 1], 5) == (_lib.OK, _lib.CSR_COL_UNSORTED)
    assert _validate([0, 2, 2, 3], [4, 4, 1], 5) == (_lib.OK, _lib.CSR_COL_UNSORTED)
    p = G.make("cfg1_check")
    assert _validate(p.row_ptr, p.col_idx, p.Kd) == (_lib.OK, 0)
    import torch
    assert ops.validate_csr(torch.from_numpy(p.row_ptr), torch.from_numpy(p.col_idx), p.Kd) == 0
    with pytest.raises(_lib.SpmmError):
        ops.validate_csr(torch.from_numpy(p.row_ptr), torch.from_numpy(p.col_idx), p.Kd - 900)


@pytest.mark.parametrize("parts", [1, 2, 3, 4, 8])
def test_partition_rows_balances_cost(parts):
    p = G.make("cfg3_powerlaw", scale=64)
    b = D.partition_rows(p.row_ptr, parts)
    assert b[0] == 0 and b[-1] == p.M and (np.diff(b) >= 0).all()
    cost = (p.row_ptr[b[1:]].astype(np.int64) - p.row_ptr[b[:-1]]) + np.diff(b)
    longest = int(np.diff(p.row_ptr).max()) + 1
    assert cost.max() - cost.min() <= 2 * longest  # no cut is further than one row from ideal
    assert D.partition_imbalance(p.row_ptr, b) < 1.05
    # nnz-only balance (row_weight 0)
    b0 = D.partition_rows(p.row_ptr, parts, 0.0)
    nnz = p.row_ptr[b0[1:]].astype(np.int64) - p.row_ptr[b0[:-1]]
    assert nnz.max() - nnz.min() <= 2 * longest


def test_partition_rows_edge_cases():
    assert D.partition_rows(np.array([0], np.int32), 4).tolist() == [0, 0, 0, 0, 0]
    assert D.partition_rows(np.array([0, 5], np.int32), 2).tolist() in ([0, 0, 1], [0, 1, 1])
    rp = np.array([0, 0, 0, 0, 100, 100, 100], np.int32)  # one heavy row among empty rows
    b = D.partition_rows(rp, 3)
    assert b[0] == 0 and b[-1] == 6 and (np.diff(b) >= 0).all()
    with pytest.raises(_lib.SpmmError):
        D.partition_rows(rp, 0)


def test_take_shard_rebases_offsets_and_keeps_indices():
    p = G.make("cfg3_powerlaw", scale=256)
    b = D.partition_rows(p.row_ptr, 4)
    got_cols, got_rows = [], 0
    for r in range(4):
        sh = D.take_shard(p.row_ptr, p.col_idx, p.values, b, r)
        assert sh.row_ptr[0] == 0 and sh.row_ptr[-1] == sh.nnz and sh.row_ptr.dtype == np.int32
        assert sh.max_row_nnz == (int(np.diff(sh.row_ptr).max()) if sh.rows else 0)
        got_cols.append(sh.col_idx)
        got_rows += sh.rows
    assert got_rows == p.M and np.array_equal(np.concatenate(got_cols), p.col_idx)  # bit-matching indices


def test_e2m1_host_codec_equals_oracle():
    x = np.random.default_rng(9).uniform(-1, 1, 4097).astype(np.float32)
    x[:8] = [0.0, -0.0, 1e-9, -1e-9, 1.0, -1.0, 0.5, np.nan]
    packed, scale = ops.e2m1_quantize(x)
    assert scale == oracle.e2m1_scale(x)
    assert np.array_equal(packed.numpy(), oracle.e2m1_encode(x, scale))
    dec = ops.e2m1_dequantize(packed, x.size, scale).numpy()
    assert np.array_equal(dec, oracle.e2m1_decode(oracle.e2m1_encode(x, scale), x.size, scale))
    allz, s = ops.e2m1_quantize(np.zeros(5, np.float32))
    assert s == 1.0 and not allz.numpy().any()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(_lib.LibraryMissing):
        _lib.lib()


def test_sweep_summary_matches_the_reference_summary_definition():
    # mean GFLOPS per algorithm and mean of per-point speed-ups over cuSPARSE
    # (the reference's benchmarks/csrspmm_vs_cusparse.py summary)
    from csrspmm_b200 import sweep
    rows = [["small", 1, 1, 1, 0.01, 0.99, "csrspmm_b200", "Naive", 100.0],
            ["small", 1, 1, 1, 0.01, 0.99, "cuSPARSE", "cuSPARSE", 50.0],
            ["XL", 1, 1, 1, 0.10, 0.90, "csrspmm_b200", "Naive", 300.0],
            ["XL", 1, 1, 1, 0.10, 0.90, "cuSPARSE", "cuSPARSE", 100.0]]
    s = {a: (g, sp) for a, g, sp in sweep.summarize(rows)}
    assert s["Naive"] == (200.0, 2.5) and s["cuSPARSE"] == (75.0, 1.0)
    assert len(sweep.SHAPES) == 4 and len(sweep.DENSITIES) == 5 and len(sweep.ENTRIES) == 5


@pytest.mark.parametrize("Kd,Nd,panels", [(1 << 22, 512, None), (1 << 22, 500, 4), (1000, 64, None), (1 << 20, 256, None),
                                         (1 << 22, 512, 40), (5, 33, 2), (7, 1, 3)])
def test_column_panels_cover_the_width(Kd, Nd, panels):
    """Host rule of the panelled round trip: panels tile [0, Nd) in order, widths are multiples of 32
    columns except the last, never more than 16 panels; small operands stay in one piece."""
    from csrspmm_b200.distributed import column_panels
    ps = column_panels(Kd, Nd, panels)
    assert 1 <= len(ps) <= 16
    assert ps[0][0] == 0 and sum(w for _, w in ps) == Nd
    for (c0, w), (c1, _) in zip(ps[:-1], ps[1:]):
        assert c0 + w == c1 and w % 32 == 0 and w > 0
    if panels is None and Kd * Nd * 4 < (256 << 20):
        assert len(ps) == 1
    if panels is None and Kd == 1 << 22 and Nd == 512:
        assert ps == [(0, 64), (64, 128), (192, 128), (320, 128), (448, 64)]  # short first and last panel


def test_copy_rows_rejects_bad_arguments_before_any_cuda_call():
    L = _lib.lib()
    buf = np.zeros(64, np.float32)
    assert L.csrspmm_b200_copy_rows(None, 16, buf.ctypes.data, 16, 16, 4, 0, None) == _lib.ERR_BAD_ARG
    assert L.csrspmm_b200_copy_rows(buf.ctypes.data, 8, buf.ctypes.data, 16, 16, 4, 0, None) == _lib.ERR_BAD_ARG
    assert L.csrspmm_b200_copy_rows(None, 0, None, 0, 0, 4, 0, None) == _lib.OK  # nothing to copy
