"""COO entry points on the GPU: against the outputs of the reference's own COO kernels (tests/golden/coo_*.npz),
against the float64 oracle on larger seeded cases, and the reference's argument contract
(spmv_coo.py:183-249 and :292-347, spmm_coo.py:312-371 of the reference)."""

import numpy as np
import pytest
import torch

import flagsparse_b200 as fs
from helpers import assert_spmm_ok, assert_spmv_ok, golden_files, load_golden
from oracle import csr_oracle as O

pytestmark = pytest.mark.gpu

COO_GOLDENS = golden_files("coo")


def _rowptr_form(val, row, col, n_rows):
    order = np.lexsort((col, row))
    indptr = np.zeros(n_rows + 1, dtype=np.int64)
    indptr[1:] = np.cumsum(np.bincount(row[order], minlength=n_rows))
    return val[order], col[order], indptr


def _random_coo(seed, n_rows, n_cols, nnz, vt=np.float32, rt=np.int32, ct=np.int32, skew=False):
    rng = np.random.default_rng(seed)
    row = rng.integers(0, n_rows, nnz)
    if skew:  # a few rows take a large share of the entries
        row[rng.random(nnz) < 0.3] = rng.integers(0, 4, 1)[0]
    col = rng.integers(0, n_cols, nnz)
    val = rng.uniform(-1, 1, nnz).astype(vt)
    return val, row.astype(rt), col.astype(ct)


@pytest.mark.parametrize("path", COO_GOLDENS, ids=lambda p: p.split("coo_")[-1][:-4])
@pytest.mark.parametrize("sort_by_row", [True, False])
def test_spmv_coo_against_reference_outputs(path, sort_by_row, cuda, fsb_lib):
    g = load_golden(path)
    data, row, col, x = (torch.from_numpy(g[k]).to(cuda) for k in ("data", "row", "col", "x"))
    y = fs.flagsparse_spmv_coo(data, row, col, x, g["shape"], sort_by_row=sort_by_row)
    d, i, p = _rowptr_form(g["data"], g["row"], g["col"], g["shape"][0])
    assert_spmv_ok(y.cpu().numpy(), d, i, p, g["shape"], g["x"], what=path)
    # and next to the reference's own result, with the bound that holds for two correctly rounded sums
    _, mag = O.spmv_f64(d, i, p, g["shape"], g["x"])
    ref_y = g["y_seg" if sort_by_row else "y_atomic"]
    assert O.max_bound_ratio(y.cpu().numpy(), ref_y.astype(np.float64), mag) <= 2 * O.TOL[np.dtype(g["data"].dtype)]
    empty = np.diff(p) == 0
    assert not y.cpu().numpy()[empty].any()


@pytest.mark.parametrize("path", COO_GOLDENS, ids=lambda p: p.split("coo_")[-1][:-4])
def test_prepared_coo_keeps_reference_attributes(path, cuda, fsb_lib):
    g = load_golden(path)
    data, row, col, x = (torch.from_numpy(g[k]).to(cuda) for k in ("data", "row", "col", "x"))
    p = fs.prepare_spmv_coo(data, row, col, g["shape"])
    assert isinstance(p, fs.PreparedCoo) and p.shape == g["shape"] and p.nnz == g["data"].size
    assert p.row.dtype == torch.int32 and p.col.dtype == torch.int32 and p.seg_starts.dtype == torch.int32
    assert np.array_equal(p.row.cpu().numpy(), g["sorted_row"]) and np.array_equal(p.col.cpu().numpy(), g["sorted_col"])
    assert np.array_equal(p.seg_starts.cpu().numpy(), g["seg_starts"]) and p.use_seg_kernel
    y1 = fs.flagsparse_spmv_coo(x=x, prepared=p)
    y2, ms = fs.flagsparse_spmv_coo(x=x, prepared=p, shape=g["shape"], return_time=True)
    assert torch.equal(y1, y2) and ms >= 0
    out = torch.full_like(y1, 7.0)
    assert fs.flagsparse_spmv_coo(x=x, prepared=p, out=out) is out and torch.equal(out, y1)
    # unsorted form: entries stay as given, no row runs
    q = fs.prepare_spmv_coo(data, row, col, g["shape"], sort_by_row=False)
    assert q.seg_starts is None and not q.use_seg_kernel and q.n_segs == 0
    assert np.array_equal(q.row.cpu().numpy(), g["row"]) and torch.equal(q.data, data)
    y3 = fs.flagsparse_spmv_coo(x=x, prepared=q)
    assert torch.equal(y3, fs.flagsparse_spmv_coo(x=x, prepared=q))  # same bits on every call
    tol = 1e-5 if g["data"].dtype == np.float32 else 1e-12
    assert torch.allclose(y3, y1, rtol=0, atol=tol * 64)


@pytest.mark.parametrize("path", COO_GOLDENS, ids=lambda p: p.split("coo_")[-1][:-4])
def test_spmm_coo_against_reference_outputs(path, cuda, fsb_lib):
    g = load_golden(path)
    data, row, col, B = (torch.from_numpy(g[k]).to(cuda) for k in ("data", "row", "col", "B"))
    C = fs.flagsparse_spmm_coo(data, row, col, B, g["shape"])
    d, i, p = _rowptr_form(g["data"], g["row"], g["col"], g["shape"][0])
    assert_spmm_ok(C.cpu().numpy(), d, i, p, g["shape"], g["B"], what=path)
    _, mag = O.spmm_f64(d, i, p, g["shape"], g["B"])
    assert O.max_bound_ratio(C.cpu().numpy(), g["C"].astype(np.float64), mag) <= 2 * O.TOL[np.dtype(g["data"].dtype)]
    assert C.is_contiguous() and not C.cpu().numpy()[np.diff(p) == 0].any()
    out = torch.empty_like(C)
    C2, ms = fs.flagsparse_spmm_coo(data, row, col, B, g["shape"], out=out, return_time=True)
    assert C2 is out and torch.equal(C2, C) and ms >= 0
    # strided B is accepted
    Bt = B.t().contiguous().t()
    assert not Bt.is_contiguous() or B.shape[1] == 1
    assert torch.equal(fs.flagsparse_spmm_coo(data, row, col, Bt, g["shape"]), C)


@pytest.mark.parametrize("vt,rt,ct,skew", [
    (np.float32, np.int32, np.int32, False),
    (np.float32, np.int64, np.int64, True),
    (np.float64, np.int32, np.int64, True),
])
def test_coo_larger_cases_against_oracle(vt, rt, ct, skew, cuda, fsb_lib):
    n_rows, n_cols, nnz = 50_000, 30_000, 1_500_000  # enough entries for the tiled kernels
    val, row, col = _random_coo(7, n_rows, n_cols, nnz, vt, rt, ct, skew)
    x = np.random.default_rng(8).uniform(-1, 1, n_cols).astype(vt)
    B = np.random.default_rng(9).uniform(-1, 1, (n_cols, 16)).astype(vt)
    tv, tr, tc, tx, tB = (torch.from_numpy(a).to(cuda) for a in (val, row, col, x, B))
    d, i, p = _rowptr_form(val, row.astype(np.int64), col.astype(np.int64), n_rows)
    for sort_by_row in (True, False):
        y = fs.flagsparse_spmv_coo(tv, tr, tc, tx, (n_rows, n_cols), sort_by_row=sort_by_row)
        assert_spmv_ok(y.cpu().numpy(), d, i, p, (n_rows, n_cols), x, what=f"sort_by_row={sort_by_row}")
    prepared = fs.prepare_spmv_coo(tv, tr, tc, (n_rows, n_cols))
    y = fs.flagsparse_spmv_coo(x=tx, prepared=prepared)
    assert_spmv_ok(y.cpu().numpy(), d, i, p, (n_rows, n_cols), x, what="prepared")
    C = fs.flagsparse_spmm_coo(tv, tr, tc, tB, (n_rows, n_cols))
    assert_spmm_ok(C.cpu().numpy(), d, i, p, (n_rows, n_cols), B, what="spmm")


def test_coo_empty_and_degenerate(cuda, fsb_lib):
    z = torch.zeros(0, dtype=torch.float32, device=cuda)
    zi = torch.zeros(0, dtype=torch.int32, device=cuda)
    x = torch.ones(5, dtype=torch.float32, device=cuda)
    y = fs.flagsparse_spmv_coo(z, zi, zi, x, (4, 5))
    assert y.shape == (4,) and not y.any()
    p = fs.prepare_spmv_coo(z, zi, zi, (4, 5))
    assert p.seg_starts is None and p.n_segs == 0
    assert not fs.flagsparse_spmv_coo(x=x, prepared=p).any()
    C = fs.flagsparse_spmm_coo(z, zi, zi, torch.ones(5, 3, device=cuda), (4, 5))
    assert C.shape == (4, 3) and not C.any()
    assert fs.flagsparse_spmv_coo(z, zi, zi, torch.ones(0, device=cuda), (0, 0)).shape == (0,)
    assert fs.flagsparse_spmm_coo(z, zi, zi, torch.ones(5, 0, device=cuda), (4, 5)).shape == (4, 0)
    # one entry, many duplicates of it
    d = torch.full((1000,), 0.5, dtype=torch.float32, device=cuda)
    r = torch.full((1000,), 2, dtype=torch.int64, device=cuda)
    c = torch.full((1000,), 4, dtype=torch.int64, device=cuda)
    y = fs.flagsparse_spmv_coo(d, r, c, x, (4, 5))
    assert y.tolist() == [0.0, 0.0, 500.0, 0.0]


def test_coo_argument_contract(cuda, fsb_lib):
    f = lambda v, dt=torch.float32: torch.tensor(v, dtype=dt, device=cuda)  # noqa: E731
    d, r, c, x = f([1.0, 2.0, 3.0]), f([0, 1, 1], torch.int32), f([0, 1, 0], torch.int32), f([1.0, 1.0])
    B = torch.ones(2, 3, device=cuda)
    p = fs.prepare_spmv_coo(d, r, c, (2, 2))
    cases = [
        (lambda: fs.flagsparse_spmv_coo(d, f([0, 2, 1], torch.int32), c, x, (2, 2)), IndexError),
        (lambda: fs.flagsparse_spmv_coo(d, r, f([0, -1, 0], torch.int32), x, (2, 2)), IndexError),
        (lambda: fs.flagsparse_spmv_coo(d, r[:2], c, x, (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmv_coo(d.half(), r, c, x.half(), (2, 2)), TypeError),
        (lambda: fs.flagsparse_spmv_coo(d, r, c, x.double(), (2, 2)), TypeError),
        (lambda: fs.flagsparse_spmv_coo(d, r, c, f([1.0, 1.0, 1.0]), (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmv_coo(d, r, c, x.cpu(), (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmv_coo(d, r, c, x.reshape(2, 1), (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmv_coo(prepared=p), TypeError),
        (lambda: fs.flagsparse_spmv_coo(x=x, prepared=p, shape=(3, 2)), ValueError),
        (lambda: fs.flagsparse_spmv_coo(x=x, prepared=p, num_warps=3), ValueError),
        (lambda: fs.flagsparse_spmv_coo(x=x, prepared=p, block_inner=48), ValueError),
        (lambda: fs.flagsparse_spmv_coo(x=x, prepared=p, out=f([0.0, 0.0, 0.0])), ValueError),
        (lambda: fs.flagsparse_spmv_coo(x=x, prepared=p, out=f([0.0, 0.0], torch.float64)), ValueError),
        (lambda: fs.flagsparse_spmm_coo(d, f([0, 2, 1], torch.int32), c, B, (2, 2)), IndexError),
        (lambda: fs.flagsparse_spmm_coo(d, r, f([0, 5, 0], torch.int32), B, (2, 2)), IndexError),
        (lambda: fs.flagsparse_spmm_coo(d, r, c, B.double(), (2, 2)), TypeError),
        (lambda: fs.flagsparse_spmm_coo(d.half(), r, c, B, (2, 2)), TypeError),
        (lambda: fs.flagsparse_spmm_coo(d.to(torch.int32), r, c, B.to(torch.int32), (2, 2)), TypeError),
        (lambda: fs.flagsparse_spmm_coo(d, r.to(torch.int16), c, B, (2, 2)), TypeError),
        (lambda: fs.flagsparse_spmm_coo(d, r, c.to(torch.int16), B, (2, 2)), TypeError),
        (lambda: fs.flagsparse_spmm_coo(d, r, c, B.cpu(), (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmm_coo(d, r, c, B, (2, 2), out=torch.empty(2, 4, device=cuda)), ValueError),
        (lambda: fs.flagsparse_spmm_coo(d, r, c, B, (2, 2), out=torch.empty(2, 3)), ValueError),
        (lambda: fs.flagsparse_spmm_coo(d, r, c, B, (2, 2), block_nnz=0), ValueError),
    ]
    for k, (call, exc) in enumerate(cases):
        with pytest.raises(exc):
            call()
            pytest.fail(f"case {k} did not raise")
    y = fs.flagsparse_spmv_coo(d, r, c, x, (2, 2))
    assert y.tolist() == [1.0, 5.0]
    assert fs.flagsparse_spmm_coo(d, r, c, B, (2, 2)).tolist() == [[1.0] * 3, [5.0] * 3]
