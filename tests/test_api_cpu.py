"""Host-side logic that needs no GPU: argument validation (exception types and order follow the reference),
the reference's launch-config helpers against golden outputs, the COO front-end, and the C ABI's symbol
table.  No kernel is launched here."""

import ctypes
import os
import re

import numpy as np
import pytest
import torch

import flagsparse_b200 as fs
from flagsparse_b200 import _lib, spmm_csr, spmv_csr
from helpers import golden_index

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _tiny(dtype=torch.float32):
    data = torch.tensor([1.0, 2.0, 3.0], dtype=dtype)
    indices = torch.tensor([0, 1, 1], dtype=torch.int32)
    indptr = torch.tensor([0, 2, 3], dtype=torch.int64)
    return data, indices, indptr


# ---- the shared library ------------------------------------------------------------------------------
def test_library_exports_every_declared_symbol(fsb_lib):
    header = open(os.path.join(ROOT, "include", "fsb.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(fsb_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found in include/fsb.h"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(raw, name), name
    # pure host queries may be called without a GPU
    assert fsb_lib.fsb_version() == 100
    assert fsb_lib.fsb_spmv_tile_nnz(_lib.FSB_F32, 0) == 2048
    assert fsb_lib.fsb_spmv_tile_nnz(_lib.FSB_F64, 1 << 8) == 1024
    assert fsb_lib.fsb_spmm_tile_nnz(_lib.FSB_F32) == 1024
    assert fsb_lib.fsb_csr_num_tiles(0, 2048) == 0
    assert fsb_lib.fsb_csr_num_tiles(2049, 2048) == 2
    assert fsb_lib.fsb_spmv_csr_scratch_bytes(_lib.FSB_F32, 4096, 0) >= 2 * 2 * 4
    assert fsb_lib.fsb_spmm_csr_scratch_bytes(_lib.FSB_F64, 1025, 7) >= 2 * 2 * 7 * 8


def test_checking_build_exports_the_same_symbols(fsb_lib):
    """libfsb_check.so (the sources with -DFSB_BOUNDS_CHECK) has the same ABI; the two builds tell themselves apart."""
    from flagsparse_b200 import build

    check = ctypes.CDLL(build.build(check=True))
    for name in _lib.SIGNATURES:
        assert hasattr(check, name), name
    assert check.fsb_bounds_check_enabled() == 1 and fsb_lib.fsb_bounds_check_enabled() == 0
    out = (ctypes.c_int64 * 5)(1, 2, 3, 4, 5)
    assert fsb_lib.fsb_bounds_check_report(ctypes.cast(out, ctypes.c_void_p)) == -1 and list(out) == [0] * 5
    check.fsb_bounds_check_report.argtypes = [ctypes.c_void_p]
    assert check.fsb_bounds_check_report(ctypes.cast(out, ctypes.c_void_p)) == 0 and list(out) == [0] * 5
    assert check.fsb_bounds_check_report(None) == -1
    with pytest.raises(RuntimeError, match="FSB_EINVAL"):
        _lib.check(-1, "x")


def test_layout_builder_refuses_bad_arguments_on_the_host(fsb_lib):
    """The entry points of the device-side layout builder check enums, sizes and pointers before any launch."""
    L, F32, I32 = fsb_lib, _lib.FSB_F32, _lib.FSB_I32
    assert L.fsb_panel_build_max_chunks() == 32768
    assert L.fsb_panel_build_window(0) == 128 and L.fsb_panel_build_window(1) == 640
    assert L.fsb_panel_build_count(7, I32, None, None, 4, 4, 1024, 4096, None, None) == -1          # bad index type
    assert L.fsb_panel_build_count(I32, I32, None, None, 4, 4, 0, 4096, None, None) == -1           # no rows per block
    assert L.fsb_panel_build_count(I32, I32, None, None, 0, 4, 1024, 4096, None, None) == 0         # nothing to count
    assert L.fsb_panel_build_count(I32, I32, None, None, 4, 4, 1024, 4096, None, None) == -1        # missing arrays
    assert L.fsb_panel_build_sort(F32, I32, I32, None, None, None, 4, 4, 1024, 4096, 0, None, None, None, None, None,
                                  None) == -1
    assert L.fsb_panel_build_sort(9, I32, I32, None, None, None, 4, 4, 1024, 4096, 0, None, None, None, None, None,
                                  None) == -1
    assert L.fsb_panel_build_runs(None, None, -1, 4096, None, None) == -1
    assert L.fsb_panel_build_cut(None, None, 0, 512, None, None, None, None, None) == -1            # no status word
    assert L.fsb_panel_build_cut(None, None, -1, 512, None, None, None, None, None) == -1
    assert L.fsb_panel_build_fill(F32, None, None, None, None, None, 1, None, None, 1, 1024, 4096, 2, 5, None, None,
                                  None) == -1                                                        # 5 rounds
    assert L.fsb_panel_build_fill(F32, None, None, None, None, None, 1, None, None, 0, 1024, 4096, 2, 8, None, None,
                                  None) == 0                                                         # no pieces
    assert L.fsb_panel_build_fill(F32, None, None, None, None, None, 1, None, None, 1, 1024, 40000, 2, 8, None, None,
                                  None) == -1                                                        # x slots > 65536
    assert L.fsb_panel_build_core_count(None, None, None, 3, 1024, 8, None, None, None) == -1
    assert L.fsb_panel_build_core_count(None, None, None, 0, 1024, 8, None, None, None) == 0
    assert L.fsb_panel_build_core_place(F32, None, None, None, None, None, None, 2, 1024, 4096, 2, 8, None, None, None,
                                        None, None, None, None, None, None) == -1


def test_argument_errors_are_reported_before_any_launch(fsb_lib):
    # bad enums / sizes are rejected on the host, so this needs no device
    assert fsb_lib.fsb_spmv_csr(7, 0, 0, None, None, None, None, None, 1, 1, 0, 0, 0, None, None, 0, None) == -1
    assert fsb_lib.fsb_spmv_csr(0, 0, 0, None, None, None, None, None, -1, 1, 0, 0, 0, None, None, 0, None) == -1
    assert fsb_lib.fsb_spmv_csr(0, 0, 0, None, None, 8, None, None, 2**31, 1, 0, 0, 0, None, None, 0, None) == -2
    assert fsb_lib.fsb_spmm_csr(0, 0, 9, None, None, None, None, 0, None, 0, 1, 1, 1, 0, 0, None, None, 0, None, None) == -1
    assert fsb_lib.fsb_csr_tile_plan(0, 8, 4, 10, 1000, 8, None) == -1  # tile size must be a power of two
    with pytest.raises(RuntimeError, match="FSB_EINVAL"):
        _lib.check(-1, "x")
    with pytest.raises(RuntimeError, match="CUDA error 700"):
        _lib.check(1700, "x")


# ---- validation: same exception types, raised in the same order as the reference -------------------------
def test_spmv_validation_on_cpu_tensors():
    data, indices, indptr = _tiny()
    x = torch.ones(2)
    with pytest.raises(ValueError, match="required"):
        fs.flagsparse_spmv_csr(data, indices, None, x, (2, 2))
    with pytest.raises(TypeError):
        fs.flagsparse_spmv_csr([1.0], indices, indptr, x, (2, 2))
    with pytest.raises(ValueError, match="one-dimensional"):
        fs.flagsparse_spmv_csr(data.reshape(1, 3), indices, indptr, x, (2, 2))
    with pytest.raises(ValueError, match="indptr has 2 entries"):
        fs.flagsparse_spmv_csr(data, indices, indptr[:-1], x, (2, 2))
    with pytest.raises(ValueError, match="2 values but 3 column indices"):
        fs.flagsparse_spmv_csr(data[:2], indices, indptr, x, (2, 2))
    # CPU tensors are refused exactly where the reference refuses them: no silent CPU path
    with pytest.raises(ValueError, match="CUDA"):
        fs.flagsparse_spmv_csr(data, indices, indptr, x, (2, 2))
    with pytest.raises(ValueError, match="CUDA"):
        fs.prepare_spmv_csr(data, indices, indptr, (2, 2))
    with pytest.raises(ValueError, match="CUDA"):
        fs.flagsparse_spmv_coo_tocsr(data, indices, indices, x, (2, 2))
    with pytest.raises(TypeError):
        fs.flagsparse_spmv_coo_tocsr(data, indices, indices, None, (2, 2))


def test_spmm_validation_on_cpu_tensors():
    data, indices, indptr = _tiny()
    B = torch.ones(2, 4)
    with pytest.raises(ValueError, match="block_n"):
        fs.flagsparse_spmm_csr(data, indices, indptr, B, (2, 2), block_n=0)
    with pytest.raises(ValueError, match="block_nnz"):
        fs.flagsparse_spmm_csr(data, indices, indptr, B, (2, 2), block_nnz=0)
    with pytest.raises(ValueError, match="max_segments"):
        fs.flagsparse_spmm_csr(data, indices, indptr, B, (2, 2), max_segments=0)
    with pytest.raises(ValueError, match="2D"):
        fs.flagsparse_spmm_csr(data, indices, indptr, B[0], (2, 2))
    with pytest.raises(ValueError, match="2-tuple"):
        fs.flagsparse_spmm_csr(data, indices, indptr, B, (2,))
    with pytest.raises(ValueError, match="non-negative"):
        fs.flagsparse_spmm_csr(data, indices, indptr, B, (-1, 2))
    with pytest.raises(ValueError, match="indptr length"):
        fs.flagsparse_spmm_csr(data, indices, indptr[:-1], B, (2, 2))
    with pytest.raises(ValueError, match="CUDA"):
        fs.flagsparse_spmm_csr(data, indices, indptr, B, (2, 2))
    with pytest.raises(TypeError, match="PreparedCsrSpmmOpt"):
        fs.flagsparse_spmm_csr_opt(B=B, prepared=object())
    with pytest.raises(ValueError, match="required"):
        fs.flagsparse_spmm_csr_opt(data, indices, indptr, B, None)
    with pytest.raises(ValueError, match="CUDA"):
        fs.flagsparse_spmm_csr_opt(data, indices, indptr, B, (2, 2))


def test_value_dtype_messages():
    from flagsparse_b200._common import _check_value_dtype

    for ok in (torch.float16, torch.bfloat16, torch.float32, torch.float64, torch.complex64, torch.complex128):
        _check_value_dtype(ok)
    assert fs.SUPPORTED_VALUE_DTYPES == (torch.float16, torch.bfloat16, torch.float32, torch.float64,
                                         torch.complex64, torch.complex128)       # the reference's whitelist
    for bad in (torch.int32, torch.int64, torch.bool, torch.uint8):
        with pytest.raises(TypeError, match="must be one of"):
            _check_value_dtype(bad)
    assert fs._tolerance_for_dtype(torch.float32) == (1e-6, 1e-5)
    assert fs._tolerance_for_dtype(torch.float64) == (1e-10, 1e-8)


# ---- host helpers against outputs of the reference's own functions -------------------------------------
def test_alg1_launch_config_matches_reference():
    for case in golden_index()["host"]["alg1"]:
        want = case["result"]
        try:
            got = spmm_csr._check_launch_overrides(case["n"], case["max_row_nnz"], **case["kw"])
        except Exception as exc:
            got = {"raises": type(exc).__name__}
        assert got == want, case


def test_opt_block_n_matches_reference():
    for n, want in golden_index()["host"]["opt_block_n"].items():
        assert spmm_csr._select_spmm_opt_block_n(int(n)) == want


def test_block_nnz_bookkeeping():
    # reference: spmv_csr.py:465-475
    assert spmv_csr._resolve_block_nnz(0, 256, None) == (256, 1)
    assert spmv_csr._resolve_block_nnz(257, 256, None) == (256, 2)
    assert spmv_csr._resolve_block_nnz(2048 * 256 + 1, 256, None) == (512, 1025)
    assert spmv_csr._resolve_block_nnz(10**9, 256, None)[0] == 65536
    assert spmv_csr._resolve_block_nnz(10**6, 256, 7) == (256, 7)


def test_coo_to_csr_matches_reference():
    g = golden_index()["host"]["coo"]
    d, i, p = fs.coo_to_csr_for_spmv(torch.tensor(g["val"], dtype=torch.float32), torch.tensor(g["row"]),
                                     torch.tensor(g["col"]), (9, 7))
    assert d.tolist() == g["data"] and i.tolist() == g["indices"] and p.tolist() == g["indptr"]
    assert str(i.dtype) == g["indices_dtype"] and str(p.dtype) == g["indptr_dtype"]
    # already sorted input is passed through; empty input gives an all-zero indptr
    d2, i2, p2 = fs.coo_to_csr_for_spmv(d, torch.repeat_interleave(torch.arange(9), p[1:] - p[:-1]), i, (9, 7))
    assert torch.equal(d2, d) and torch.equal(i2, i) and torch.equal(p2, p)
    e = fs.coo_to_csr_for_spmv(torch.zeros(0), torch.zeros(0, dtype=torch.int64), torch.zeros(0, dtype=torch.int64), (3, 3))
    assert e[2].tolist() == [0, 0, 0, 0]


def test_algo_selector():
    sel = spmv_csr._select_spmv_algo
    assert sel(4096, 65536, 16) == _lib.FSB_SPMV_VECTOR
    assert sel(1 << 22, 1 << 27, 70) == _lib.FSB_SPMV_VECTOR      # Poisson(32): uniform rows
    assert sel(1 << 24, 248_000_000, 1 << 17) == _lib.FSB_SPMV_STREAM  # power-law rows
    assert sel(1 << 22, 1 << 24, 2000) == _lib.FSB_SPMV_STREAM    # mean 4, a few rows of 2000
    assert sel(10, 50000, 40000) == _lib.FSB_SPMV_STREAM  # long rows go to the tiled kernel even when small
    os.environ["FSB_SPMV_ALGO"] = "stream"
    try:
        assert sel(1 << 22, 1 << 27, 70) == _lib.FSB_SPMV_STREAM
    finally:
        del os.environ["FSB_SPMV_ALGO"]
