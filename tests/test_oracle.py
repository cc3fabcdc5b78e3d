"""The CPU oracle against the golden fixtures (outputs of the reference's own Triton kernels), and the
C restatement against the scipy one.  CPU only."""

import numpy as np
import pytest

from helpers import golden_files, handmade_csr, load_golden
from oracle import csr_oracle as O
from oracle import csr_ref as C


@pytest.mark.parametrize("path", golden_files("spmv"), ids=lambda p: p.split("/")[-1])
def test_spmv_oracle_matches_reference_outputs(path):
    g = load_golden(path)
    args = (g["data"], g["indices"], g["indptr"], g["shape"], g["x"])
    ref, mag = O.spmv_f64(*args)
    base = O.spmv_base(*args)
    if g["data"].dtype == np.float32:
        # the reference's base path accumulates in float64 and rounds once: the oracle reproduces its bits
        assert np.array_equal(base, g["y_base"])
    # both reference paths sit well inside the acceptance bound the CUDA kernels are held to
    assert O.within_bound(g["y_base"], ref, mag, g["data"].dtype)
    assert O.within_bound(g["y_opt"], ref, mag, g["data"].dtype)
    # empty rows are exact zeros in the reference and in the oracle
    empty = np.diff(g["indptr"].astype(np.int64)) == 0
    assert np.all(g["y_opt"][empty] == 0) and np.all(base[empty] == 0)


@pytest.mark.parametrize("path", golden_files("spmm"), ids=lambda p: p.split("/")[-1])
def test_spmm_oracle_matches_reference_outputs(path):
    g = load_golden(path)
    args = (g["data"], g["indices"], g["indptr"], g["shape"], g["B"])
    ref, mag = O.spmm_f64(*args)
    base = O.spmm_base(*args)
    if g["data"].dtype == np.float32:
        assert np.array_equal(base, g["C_base"])
    assert O.within_bound(g["C_base"], ref, mag, g["data"].dtype)
    assert O.within_bound(g["C_opt"], ref, mag, g["data"].dtype)


@pytest.mark.parametrize("path", golden_files("spmv"), ids=lambda p: p.split("/")[-1])
def test_c_restatement_spmv(path):
    g = load_golden(path)
    args = (g["data"], g["indices"], g["indptr"], g["shape"], g["x"])
    ref, mag = O.spmv_f64(*args)
    y1 = C.spmv(*args, threads=1)
    y4 = C.spmv(*args, threads=4)
    assert np.array_equal(y1, y4)  # threads split rows only
    if g["data"].dtype == np.float32:
        assert np.array_equal(y1, g["y_base"])
    assert O.within_bound(y1, ref, mag, g["data"].dtype)
    assert O.within_bound(C.spmv(*args, native=True, threads=3), ref, mag, g["data"].dtype)


@pytest.mark.parametrize("path", golden_files("spmm"), ids=lambda p: p.split("/")[-1])
def test_c_restatement_spmm(path):
    g = load_golden(path)
    args = (g["data"], g["indices"], g["indptr"], g["shape"], g["B"])
    ref, mag = O.spmm_f64(*args)
    c1 = C.spmm(*args, threads=1)
    assert np.array_equal(c1, C.spmm(*args, threads=5))
    if g["data"].dtype == np.float32:
        assert np.array_equal(c1, g["C_base"])
    assert O.within_bound(c1, ref, mag, g["data"].dtype)
    assert O.within_bound(C.spmm(*args, native=True, threads=2), ref, mag, g["data"].dtype)


def test_oracle_does_not_touch_its_inputs():
    # duplicate, unsorted columns: scipy would canonicalise a shared array in place
    data, idx, ptr = handmade_csr(3, [5, 0, 7, 2], 6, sort=False, replace=True)
    keep = (data.copy(), idx.copy(), ptr.copy())
    x = np.linspace(-1, 1, 6).astype(np.float32)
    y, mag = O.spmv_f64(data, idx, ptr, (4, 6), x)
    assert all(np.array_equal(a, b) for a, b in zip(keep, (data, idx, ptr)))
    loop = O.spmv_rowloop(data, idx, ptr, (4, 6), x, acc_dtype=np.float64)
    assert np.allclose(loop, y, rtol=0, atol=1e-6)
    assert y[1] == 0 and mag[1] == 0


def test_bound_helper():
    ref = np.array([1.0, 0.0, -2.0])
    mag = np.array([2.0, 0.0, 4.0])
    assert O.max_bound_ratio(ref, ref, mag) == 0
    assert O.max_bound_ratio(ref + np.array([2e-5, 0, 0]), ref, mag) == pytest.approx(1e-5)
    assert O.max_bound_ratio(ref + np.array([0, 1e-30, 0]), ref, mag) == np.inf  # an empty row must be exactly 0
    assert not O.within_bound(ref + np.array([3e-5, 0, 0]), ref, mag, np.float32)
