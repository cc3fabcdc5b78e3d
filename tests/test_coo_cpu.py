"""COO entry points, the parts that need no GPU: the oracle against the outputs of the reference's COO kernels
(tests/golden/coo_*.npz), the ordering helpers against the reference's sorted arrays and row-run bounds, the
launch bookkeeping, and the argument checks that fire before any CUDA call."""

import numpy as np
import pytest
import scipy.sparse as sp
import torch

from flagsparse_b200 import coo
from helpers import golden_files, golden_index, load_golden
from oracle import csr_oracle as O

COO_GOLDENS = golden_files("coo")


def _as_csr(g):
    """scipy sums duplicates and orders the columns: the matrix the COO triple denotes."""
    m = sp.coo_matrix((g["data"].astype(np.float64), (g["row"].astype(np.int64), g["col"].astype(np.int64))),
                      shape=g["shape"]).tocsr()
    return m.data.astype(g["data"].dtype), m.indices, m.indptr


def test_goldens_present():
    assert len(COO_GOLDENS) == 3
    assert set(golden_index()["coo"]) == {"dups_f32", "dups_f64", "sparse_rows_f32"}


@pytest.mark.parametrize("path", COO_GOLDENS, ids=lambda p: p.split("coo_")[-1][:-4])
def test_oracle_matches_reference_coo_kernels(path):
    g = load_golden(path)
    dtype = g["data"].dtype
    # the un-merged entries as a row-pointer matrix (duplicates kept): what the kernels here are given
    order = np.lexsort((g["col"], g["row"]))
    indptr = np.zeros(g["shape"][0] + 1, dtype=np.int64)
    indptr[1:] = np.cumsum(np.bincount(g["row"][order], minlength=g["shape"][0]))
    ref, mag = O.spmv_f64(g["data"][order], g["col"][order], indptr, g["shape"], g["x"])
    for key in ("y_seg", "y_atomic"):
        assert g[key].dtype == dtype and g[key].shape == (g["shape"][0],)
        assert O.max_bound_ratio(g[key], ref, mag) <= O.TOL[np.dtype(dtype)], key
    cref, cmag = O.spmm_f64(g["data"][order], g["col"][order], indptr, g["shape"], g["B"])
    assert g["C"].dtype == dtype and g["C"].shape == (g["shape"][0], g["B"].shape[1])
    assert O.max_bound_ratio(g["C"], cref, cmag) <= O.TOL[np.dtype(dtype)]
    # merged duplicates give the same matrix
    d2, i2, p2 = _as_csr(g)
    ref2, _ = O.spmv_f64(d2, i2, p2, g["shape"], g["x"])
    assert np.allclose(ref, ref2, rtol=0, atol=1e-5 if dtype == np.float32 else 1e-13)
    # rows without entries are exact zeros in the reference's outputs
    empty = np.diff(indptr) == 0
    assert empty.any()
    assert not g["y_seg"][empty].any() and not g["y_atomic"][empty].any() and not g["C"][empty].any()


@pytest.mark.parametrize("path", COO_GOLDENS, ids=lambda p: p.split("coo_")[-1][:-4])
def test_ordering_helpers_match_reference(path):
    g = load_golden(path)
    n_rows, n_cols = g["shape"]
    data, row, col = (torch.from_numpy(g[k]) for k in ("data", "row", "col"))
    d, r, c = coo._sort_coo_lex(data, row.to(torch.int64), col.to(torch.int64), n_cols)
    assert np.array_equal(r.numpy(), g["sorted_row"]) and np.array_equal(c.numpy(), g["sorted_col"])
    # duplicates of one (row, col) may come out in either order: compare the values per pair as multisets
    key = g["sorted_row"] * n_cols + g["sorted_col"]
    for k in np.unique(key):
        assert np.array_equal(np.sort(d.numpy()[key == k]), np.sort(g["sorted_data"][key == k]))
    seg = coo._seg_starts_from_sorted_rows(r, d.numel(), d.device)
    assert seg.dtype == torch.int32 and np.array_equal(seg.numpy(), g["seg_starts"])
    p = coo.PreparedCoo(d, r.to(torch.int32), c.to(torch.int32), g["shape"], seg_starts=seg)
    meta = golden_index()["coo"][path.split("coo_")[-1][:-4]]
    assert p.n_segs == meta["n_segs"] and p.use_seg_kernel and p.nnz == meta["nnz"]
    indptr = coo._row_pointer(r, n_rows)
    assert indptr.dtype == torch.int64 and int(indptr[-1]) == d.numel()
    assert np.array_equal(np.diff(indptr.numpy()), np.bincount(g["row"], minlength=n_rows))
    # the row runs and the row pointer describe the same partition of the entries
    starts = indptr.numpy()[:-1][np.diff(indptr.numpy()) > 0]
    assert np.array_equal(starts, g["seg_starts"][:-1])


def test_launch_bookkeeping_matches_reference():
    for name, meta in golden_index()["coo"].items():
        g = load_golden([p for p in COO_GOLDENS if p.endswith(f"coo_{name}.npz")][0])
        merged = len(set(zip(g["row"].tolist(), g["col"].tolist())))
        assert coo._resolve_spmm_coo_launch_config(g["B"].shape[1], merged) == meta["launch"]
    with pytest.raises(ValueError):
        coo._resolve_spmm_coo_launch_config(8, 10, block_n=0)
    with pytest.raises(ValueError):
        coo._resolve_spmm_coo_launch_config(8, 10, block_nnz=-1)


def test_prepared_coo_without_runs():
    z = torch.zeros(0)
    p = coo.PreparedCoo(z, z.to(torch.int32), z.to(torch.int32), (3, 4), seg_starts=None)
    assert (p.n_rows, p.n_cols, p.nnz, p.n_segs, p.use_seg_kernel) == (3, 4, 0, 0, False)


def test_argument_checks_before_any_cuda_call():
    d = torch.ones(3)
    r = torch.tensor([0, 1, 1])
    c = torch.tensor([0, 1, 0])
    x = torch.ones(2)
    with pytest.raises(ValueError):  # prepared is None and something is missing
        coo.flagsparse_spmv_coo(d, r, c, None, (2, 2))
    with pytest.raises(TypeError):
        coo.prepare_spmv_coo(d.numpy(), r, c, (2, 2))
    with pytest.raises(ValueError):
        coo.prepare_spmv_coo(d.reshape(3, 1), r, c, (2, 2))
    with pytest.raises(ValueError):  # CPU tensors: there is no CPU path
        coo.prepare_spmv_coo(d, r, c, (2, 2))
    with pytest.raises(ValueError):
        coo.flagsparse_spmv_coo(d, r, c, x, (2, 2))
    B = torch.ones(2, 3)
    with pytest.raises(ValueError):
        coo.flagsparse_spmm_coo(d, r, c, B, (2,))
    with pytest.raises(ValueError):
        coo.flagsparse_spmm_coo(d, r, c, B[0], (2, 2))
    with pytest.raises(ValueError):
        coo.flagsparse_spmm_coo(d, r, c, B, (2, -1))
    with pytest.raises(ValueError):
        coo.flagsparse_spmm_coo(d, r[:2], c, B, (2, 2))
    with pytest.raises(ValueError):
        coo.flagsparse_spmm_coo(d, r, c, torch.ones(3, 3), (2, 2))
    with pytest.raises(ValueError):
        coo.flagsparse_spmm_coo(d, r, c, B, (2, 2), block_n=0)
    with pytest.raises(ValueError):  # CPU tensors
        coo.flagsparse_spmm_coo(d, r, c, B, (2, 2))
    with pytest.raises(TypeError):
        coo.flagsparse_spmv_coo(x=x, prepared=object())
