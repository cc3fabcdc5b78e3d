"""The reference's API contract on the GPU: its SpMM validation list (tests/test_spmm.py:685-807 of the
reference: 15 calls that must raise a given exception type, 5 that must succeed) and the same contract for
SpMV, whose checks live in spmv_csr.py:379-452 of the reference."""

import numpy as np
import pytest
import torch

import flagsparse_b200 as fs
from helpers import assert_spmm_ok, assert_spmv_ok, handmade_csr

pytestmark = pytest.mark.gpu


@pytest.fixture()
def tiny(cuda):
    data = torch.tensor([1.0, 2.0, 3.0], dtype=torch.float32, device=cuda)
    indices = torch.tensor([0, 1, 1], dtype=torch.int32, device=cuda)
    indptr = torch.tensor([0, 2, 3], dtype=torch.int64, device=cuda)
    B = torch.randn((2, 4), dtype=torch.float32, device=cuda)
    return data, indices, indptr, B


def _long_row_case(cuda):
    # a 1536-nnz row followed by a 4-nnz row, 48 dense columns (the reference's constructed long-row case)
    cols = np.concatenate([np.arange(1536), [7, 129, 511, 1024]])
    data = np.random.default_rng(0).uniform(-1, 1, cols.size).astype(np.float32)
    indptr = np.array([0, 1536, 1540], dtype=np.int64)
    B = np.random.default_rng(1).uniform(-1, 1, (2048, 48)).astype(np.float32)
    return data, cols.astype(np.int32), indptr, B, (2, 2048)


def test_spmm_negative_cases(tiny, cuda, fsb_lib):
    data, indices, indptr, B = tiny
    t = lambda v, dt=torch.int64: torch.tensor(v, dtype=dt, device=cuda)  # noqa: E731
    ld, li, lp, lB, lshape = _long_row_case(cuda)
    ld, li, lp, lB = (torch.from_numpy(a).to(cuda) for a in (ld, li, lp, lB))
    cases = [
        (lambda: fs.flagsparse_spmm_csr(data, indices, indptr, B, (2,)), ValueError),
        (lambda: fs.flagsparse_spmm_csr(data, indices, indptr, B[0], (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmm_csr(data, indices, indptr, B.to(torch.float64), (2, 2)), TypeError),
        (lambda: fs.flagsparse_spmm_csr(data, indices, indptr, torch.randn((3, 4), device=cuda), (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmm_csr(data, indices, indptr[:-1], B, (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmm_csr(data, indices, t([1, 2, 3]), B, (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmm_csr(data, indices, t([0, 2, 2]), B, (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmm_csr(data, indices, t([0, 3, 2]), B, (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmm_csr(data, t([0, 3, 1], torch.int32), indptr, B, (2, 2)), IndexError),
        (lambda: fs.flagsparse_spmm_csr(data, indices, indptr, B, (2, 2), block_n=0), ValueError),
        (lambda: fs.flagsparse_spmm_csr(data, indices, indptr, B, (2, 2), block_nnz=0), ValueError),
        (lambda: fs.flagsparse_spmm_csr(data, indices, indptr, B, (2, 2), max_segments=0), ValueError),
        (lambda: fs.flagsparse_spmm_csr(data, indices, indptr, B, (2, 2), out=torch.empty((3, 4), device=cuda)), ValueError),
        (lambda: fs.flagsparse_spmm_csr(data, indices, indptr, B, (2, 2), out=torch.empty((2, 4))), ValueError),
        (lambda: fs.flagsparse_spmm_csr(ld, li, lp, lB, lshape, block_nnz=128, max_segments=4), ValueError),
        # a few more from the checks in the reference's source
        (lambda: fs.flagsparse_spmm_csr(data, t([-1, 1, 1], torch.int32), indptr, B, (2, 2)), IndexError),
        (lambda: fs.flagsparse_spmm_csr(data.to(torch.int32), indices, indptr, B.to(torch.int32), (2, 2)), TypeError),
        (lambda: fs.flagsparse_spmm_csr(data.to(torch.float16), indices, indptr, B, (2, 2)), TypeError),
        (lambda: fs.flagsparse_spmm_csr_opt(data.to(torch.float16), indices, indptr, B.to(torch.float16), (2, 2)), TypeError),
        (lambda: fs.flagsparse_spmm_csr(data, indices.to(torch.int16), indptr, B, (2, 2)), TypeError),
        (lambda: fs.flagsparse_spmm_csr(data, indices, indptr.to(torch.int16), B, (2, 2)), TypeError),
        (lambda: fs.flagsparse_spmm_csr_opt(data, indices, indptr, None, (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmm_csr_opt(B=B, prepared=fs.prepare_spmm_csr_opt(data, indices, indptr, (2, 2)), shape=(3, 2)), ValueError),
        (lambda: fs.flagsparse_spmm_csr_opt(data, indices, indptr, B.cpu(), (2, 2)), ValueError),
    ]
    for k, (fn, exc) in enumerate(cases):
        with pytest.raises(exc):
            fn()
            pytest.fail(f"case {k} did not raise")


def test_spmm_positive_cases(tiny, cuda, fsb_lib):
    data, indices, indptr, B = tiny
    host = (data.cpu().numpy(), indices.cpu().numpy(), indptr.cpu().numpy(), (2, 2))
    out = torch.empty((2, 4), dtype=torch.float32, device=cuda)
    res = fs.flagsparse_spmm_csr(data, indices, indptr, B, (2, 2), out=out)
    assert res.data_ptr() == out.data_ptr()
    assert_spmm_ok(res.cpu().numpy(), *host, B.cpu().numpy())
    # empty matrix
    e = fs.flagsparse_spmm_csr(data[:0], indices[:0], torch.zeros(3, dtype=torch.int64, device=cuda), B, (2, 2))
    assert e.shape == (2, 4) and torch.count_nonzero(e) == 0
    # no dense columns
    z = fs.flagsparse_spmm_csr(data, indices, indptr, torch.empty((2, 0), device=cuda), (2, 2))
    assert z.shape == (2, 0)
    # no rows
    r0 = fs.flagsparse_spmm_csr(data[:0], indices[:0], torch.zeros(1, dtype=torch.int64, device=cuda), B, (0, 2))
    assert r0.shape == (0, 4)
    # non-contiguous B
    dense = torch.randn((4, 2), device=cuda).transpose(0, 1)
    assert not dense.is_contiguous()
    assert_spmm_ok(fs.flagsparse_spmm_csr(data, indices, indptr, dense, (2, 2)).cpu().numpy(), *host, dense.cpu().numpy())
    # the long row, default launch parameters and generous overrides
    ld, li, lp, lB, lshape = _long_row_case(cuda)
    dev = lambda a: torch.from_numpy(a).to(cuda)  # noqa: E731
    for kw in ({}, {"block_nnz": 128, "max_segments": 12}):
        c = fs.flagsparse_spmm_csr(dev(ld), dev(li), dev(lp), dev(lB), lshape, **kw)
        assert_spmm_ok(c.cpu().numpy(), ld, li, lp, lshape, lB)


def test_spmv_contract(tiny, cuda, fsb_lib):
    data, indices, indptr, _ = tiny
    x = torch.tensor([0.5, -2.0], dtype=torch.float32, device=cuda)
    t = lambda v, dt=torch.int64: torch.tensor(v, dtype=dt, device=cuda)  # noqa: E731
    y = fs.flagsparse_spmv_csr(data, indices, indptr, x, (2, 2))
    assert y.tolist() == [1.0 * 0.5 + 2.0 * -2.0, 3.0 * -2.0]
    assert y.dtype == torch.float32 and y.is_contiguous() and y.device == data.device
    cases = [
        (lambda: fs.flagsparse_spmv_csr(data, indices, t([1, 2, 3]), x, (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmv_csr(data, indices, t([0, 2, 2]), x, (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmv_csr(data, indices, t([0, 3, 2]), x, (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmv_csr(data, t([0, 2, 1], torch.int32), indptr, x, (2, 2)), IndexError),
        (lambda: fs.flagsparse_spmv_csr(data, t([0, -1, 1], torch.int32), indptr, x, (2, 2)), IndexError),
        (lambda: fs.flagsparse_spmv_csr(data, indices.to(torch.int16), indptr, x, (2, 2)), TypeError),
        (lambda: fs.flagsparse_spmv_csr(data.to(torch.int64), indices, indptr, x.to(torch.int64), (2, 2)), TypeError),
        (lambda: fs.flagsparse_spmv_csr(data.to(torch.bfloat16), indices, indptr, x, (2, 2)), TypeError),
        (lambda: fs.flagsparse_spmv_csr(data, indices, indptr, x.to(torch.float64), (2, 2)), TypeError),
        (lambda: fs.flagsparse_spmv_csr(data, indices, indptr, torch.ones(3, device=cuda), (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmv_csr(data, indices, indptr, x.reshape(1, 2), (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmv_csr(data, indices, indptr, x.cpu(), (2, 2)), ValueError),
        (lambda: fs.flagsparse_spmv_csr(data, indices, indptr, None, (2, 2)), TypeError),
    ]
    for k, (fn, exc) in enumerate(cases):
        with pytest.raises(exc):
            fn()
            pytest.fail(f"case {k} did not raise")
    # empty matrix, no rows, strided x
    assert fs.flagsparse_spmv_csr(data[:0], indices[:0], t([0, 0, 0]), x, (2, 2)).tolist() == [0.0, 0.0]
    assert fs.flagsparse_spmv_csr(data[:0], indices[:0], t([0]), x, (0, 2)).shape == (0,)
    x2 = torch.stack([x, x], dim=1)[:, 0]
    assert not x2.is_contiguous() and torch.equal(fs.flagsparse_spmv_csr(data, indices, indptr, x2, (2, 2)), y)


def test_coo_front_end(cuda, fsb_lib):
    lens = [3, 0, 40, 7, 0, 900]
    data, idx, ptr = handmade_csr(41, lens, 1000)
    rows = np.repeat(np.arange(len(lens)), lens)
    perm = np.random.default_rng(42).permutation(data.size)
    x = np.random.default_rng(43).uniform(-1, 1, 1000).astype(np.float32)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)  # noqa: E731
    shape = (len(lens), 1000)
    y = fs.flagsparse_spmv_coo_tocsr(dev(data[perm]), dev(rows[perm]), dev(idx[perm]), dev(x), shape)
    assert_spmv_ok(y.cpu().numpy(), data, idx, ptr, shape, x, what="coo unsorted")
    prep = fs.prepare_spmv_coo_tocsr(dev(data), dev(rows), dev(idx), shape, assume_sorted=True)
    y2 = fs.flagsparse_spmv_coo_tocsr(x=dev(x), prepared=prep)
    assert_spmv_ok(y2.cpu().numpy(), data, idx, ptr, shape, x, what="coo prepared")
    with pytest.raises(ValueError):
        fs.flagsparse_spmv_coo_tocsr(x=dev(x), prepared=prep, shape=(7, 1000))
