"""float16 / bfloat16 / complex64 / complex128 values on the GPU entry points that take them in the reference
(flagsparse_spmv_csr, flagsparse_spmm_csr, flagsparse_spmm_coo): results against a float64 / complex128 product of
the same stored values, the prepared objects' attributes, and the entry points that refuse these types."""

import numpy as np
import pytest
import scipy.sparse as sp
import torch

import flagsparse_b200 as fs
from flagsparse_b200 import widetypes as W
from helpers import handmade_csr

pytestmark = pytest.mark.gpu

# |y - y_ref| <= tol * (|A| |x|): rounding of the result to the caller's type plus the real kernels' own bound
TOL = {torch.float16: 1e-3, torch.bfloat16: 8e-3, torch.complex64: 4e-5, torch.complex128: 4e-13}


def _values(n, dtype, seed):
    rng = np.random.default_rng(seed)
    v = rng.uniform(-1, 1, n)
    if dtype in W.COMPLEX_DTYPES:
        v = v + 1j * rng.uniform(-1, 1, n)
    return torch.from_numpy(v).to(dtype)


def _case(dtype, lens, n_cols, seed):
    _, i, p = handmade_csr(seed, lens, n_cols)
    return _values(int(p[-1]), dtype, seed + 1), i, p, (len(lens), n_cols)


def _check(y, vals, i, p, shape, operand, dtype, what):
    wide = torch.complex128 if dtype in W.COMPLEX_DTYPES else torch.float64
    a = sp.csr_matrix((vals.to(wide).numpy(), i, p), shape=shape)
    o = operand.cpu().to(wide).numpy()
    ref, mag = np.asarray(a @ o), np.asarray(abs(a) @ np.abs(o))
    got = y.cpu().to(wide).numpy()
    assert y.dtype == dtype and got.shape == ref.shape, what
    # float16 results below 2^-14 are subnormal: their rounding error is absolute (half a step of 2^-24), not relative
    floor = 2.0 ** -25 if dtype == torch.float16 else 0.0
    ratio = float((np.maximum(np.abs(got - ref) - floor, 0) / np.maximum(mag, 1e-300)).max()) if ref.size else 0.0
    assert ratio <= TOL[dtype], f"{what}: {ratio:.3e}"
    assert not got[np.diff(p) == 0].any(), what


def _lens(kind):
    rng = np.random.default_rng(5)
    if kind == "uniform":
        return rng.integers(20, 44, 9000).tolist()                      # vector kernel
    lens = rng.integers(0, 9, 9000)
    lens[rng.choice(9000, 40, replace=False)] = rng.integers(3000, 9000, 40)   # stream kernel
    return lens.tolist()


@pytest.mark.parametrize("dtype", W.WIDE_DTYPES, ids=str)
@pytest.mark.parametrize("ptr_dtype", [torch.int32, torch.int64], ids=str)
def test_direct_c_abi_call(cuda, fsb_lib, dtype, ptr_dtype):
    """fsb_spmv_csr_wide itself: 2-byte values with float32 x / y, complex values interleaved."""
    from flagsparse_b200 import _lib

    lens = [0, 1, 0, 33, 2, 700, 0, 0, 5, 64, 31, 17] * 50
    vals, i, p, shape = _case(dtype, lens, 900, seed=11)
    x = _values(shape[1], dtype, 12)
    half = dtype in W.HALF_DTYPES
    dense = torch.float32 if half else dtype
    d, ti, tp = vals.to(cuda), torch.from_numpy(i).to(cuda), torch.from_numpy(p).to(cuda).to(ptr_dtype)
    tx = x.to(dense).to(cuda)
    y = torch.full((shape[0],), 7, dtype=dense, device=cuda)
    vt = {torch.float16: _lib.FSB_F16, torch.bfloat16: _lib.FSB_BF16, torch.complex64: _lib.FSB_C64,
          torch.complex128: _lib.FSB_C128}[dtype]
    st = torch.cuda.current_stream().cuda_stream
    call = lambda out: fsb_lib.fsb_spmv_csr_wide(vt, 0 if ptr_dtype == torch.int32 else 1, d.data_ptr(), ti.data_ptr(),  # noqa: E731
                                                 tp.data_ptr(), tx.data_ptr(), out.data_ptr(), shape[0], shape[1],
                                                 d.numel(), st)
    assert call(y) == 0
    _check(y.to(dtype), vals, i, p, shape, x, dtype, "C ABI")
    y2 = torch.empty_like(y)
    assert call(y2) == 0 and torch.equal(y, y2)                       # fixed summation order
    assert fsb_lib.fsb_spmv_csr_wide(0, 0, d.data_ptr(), ti.data_ptr(), tp.data_ptr(), tx.data_ptr(), y.data_ptr(),
                                     shape[0], shape[1], d.numel(), st) == -1     # float32 is not this entry's
    assert fsb_lib.fsb_spmv_csr_wide(vt, 0, None, None, tp.data_ptr(), None, None, 0, 5, 0, st) == 0   # no rows


@pytest.mark.parametrize("dtype", W.WIDE_DTYPES, ids=str)
@pytest.mark.parametrize("rows", ["uniform", "skewed"])
def test_spmv(cuda, fsb_lib, dtype, rows):
    vals, i, p, shape = _case(dtype, _lens(rows), 12000, seed=3)
    x = _values(shape[1], dtype, 9)
    d, ti, tp, tx = vals.to(cuda), torch.from_numpy(i).to(cuda), torch.from_numpy(p).to(cuda), x.to(cuda)
    y = fs.flagsparse_spmv_csr(d, ti, tp, tx, shape)
    _check(y, vals, i, p, shape, x, dtype, "one-shot")
    assert torch.equal(fs.flagsparse_spmv_csr(d, ti, tp, tx, shape, use_opt=True), y)   # same kernels either way
    prep = fs.prepare_spmv_csr(d, ti, tp, shape)
    assert prep.data.dtype == dtype and not prep.supports_opt and prep.shape == shape
    assert prep.wide == ("native", [])          # read as stored by fsb_spmv_csr_wide: no widened or split copy
    y2, ms = fs.flagsparse_spmv_csr(x=tx, prepared=prep, return_time=True)
    _check(y2, vals, i, p, shape, x, dtype, "prepared")
    assert ms >= 0 and torch.equal(y2, fs.flagsparse_spmv_csr(x=tx, prepared=prep))
    out = torch.zeros_like(y2)
    assert fs.flagsparse_spmv_csr(x=tx, prepared=prep, out=out) is out and torch.equal(out, y2)
    with pytest.raises(ValueError):
        fs.flagsparse_spmv_csr(x=tx, prepared=prep, out=torch.zeros(shape[0], dtype=torch.float32, device=cuda))
    with pytest.raises(TypeError):
        fs.flagsparse_spmv_csr(x=tx.to(torch.float32) if dtype in W.HALF_DTYPES else tx.real.contiguous(),
                               prepared=prep)


@pytest.mark.parametrize("dtype", W.WIDE_DTYPES, ids=str)
def test_spmm(cuda, fsb_lib, dtype):
    lens = np.random.default_rng(6).integers(0, 30, 3000)
    lens[[7, 1500]] = [2500, 1200]
    vals, i, p, shape = _case(dtype, lens.tolist(), 4000, seed=13)
    B = _values(shape[1] * 8, dtype, 17).reshape(shape[1], 8)
    d, ti, tp, tB = vals.to(cuda), torch.from_numpy(i).to(cuda), torch.from_numpy(p).to(cuda), B.to(cuda)
    C = fs.flagsparse_spmm_csr(d, ti, tp, tB, shape)
    _check(C, vals, i, p, shape, B, dtype, "spmm")
    assert C.is_contiguous()
    out = torch.empty_like(C)
    C2, ms = fs.flagsparse_spmm_csr(d, ti, tp, tB, shape, out=out, return_time=True)
    assert C2 is out and torch.equal(C2, C) and ms >= 0
    # column-major B (copied by the entry point) and B with a row stride (handed to the kernel as it is)
    Bt = tB.t().contiguous().t()
    assert torch.equal(fs.flagsparse_spmm_csr(d, ti, tp, Bt, shape), C)
    wide = torch.zeros((shape[1], 11), dtype=dtype, device=cuda)
    wide[:, 2:10] = tB
    assert torch.equal(fs.flagsparse_spmm_csr(d, ti, tp, wide[:, 2:10], shape), C)
    # wider than one column tile of the kernel
    B40 = _values(shape[1] * 40, dtype, 23).reshape(shape[1], 40)
    _check(fs.flagsparse_spmm_csr(d, ti, tp, B40.to(cuda), shape), vals, i, p, shape, B40, dtype, "spmm N=40")
    # the prepared ("opt") entry point is float32 / float64 only, as in the reference
    prep = fs.prepare_spmm_csr_opt(d, ti, tp, shape)
    assert not prep.supports_opt and prep.data.dtype == dtype and prep.wide == ("native", [])
    with pytest.raises(TypeError):
        fs.flagsparse_spmm_csr_opt(B=tB, prepared=prep)
    # COO entry point: same matrix given as unsorted triples
    row = np.repeat(np.arange(shape[0]), np.diff(p))
    perm = np.random.default_rng(19).permutation(row.size)
    Cc = fs.flagsparse_spmm_coo(d[torch.from_numpy(perm).to(cuda)], torch.from_numpy(row[perm]).to(cuda),
                                torch.from_numpy(i[perm].astype(np.int64)).to(cuda), tB, shape)
    _check(Cc, vals, i, p, shape, B, dtype, "spmm_coo")


def test_tiny_and_empty(cuda, fsb_lib):
    for dtype in W.WIDE_DTYPES:
        d = _values(3, dtype, 1).to(cuda)
        i = torch.tensor([0, 1, 1], dtype=torch.int32, device=cuda)
        p = torch.tensor([0, 2, 2, 3], dtype=torch.int64, device=cuda)
        x = _values(2, dtype, 2).to(cuda)
        y = fs.flagsparse_spmv_csr(d, i, p, x, (3, 2))
        _check(y, d.cpu(), i.cpu().numpy(), p.cpu().numpy(), (3, 2), x.cpu(), dtype, "tiny")
        z = torch.zeros(0, dtype=dtype, device=cuda)
        zi = torch.zeros(0, dtype=torch.int32, device=cuda)
        y0 = fs.flagsparse_spmv_csr(z, zi, torch.zeros(4, dtype=torch.int64, device=cuda), x, (3, 2))
        assert y0.dtype == dtype and y0.shape == (3,) and not y0.cpu().to(torch.complex128).abs().any()
        C0 = fs.flagsparse_spmm_csr(z, zi, torch.zeros(4, dtype=torch.int64, device=cuda), x.reshape(2, 1), (3, 2))
        assert C0.dtype == dtype and C0.shape == (3, 1) and not C0.cpu().to(torch.complex128).abs().any()
    # the COO SpMV entry point stays float32 / float64, as in the reference
    with pytest.raises(TypeError):
        fs.flagsparse_spmv_coo(d, i, i, x, (3, 2))


@pytest.mark.parametrize("tag", ["bf16", "c128", "c64", "f16"])
def test_against_reference_outputs(cuda, fsb_lib, tag):
    """The public entry points on the inputs of tests/golden/wide_*.npz against the outputs of the reference's own
    base SpMV / SpMM helpers for these value types."""
    from test_widetypes_cpu import GOLDEN_TOL, load_wide_golden

    g, dt = load_wide_golden(tag)
    wide = torch.complex128 if dt in W.COMPLEX_DTYPES else torch.float64
    a = sp.csr_matrix((g["data"].to(wide).numpy(), g["indices"], g["indptr"]), shape=g["shape"])
    d, i, p = g["data"].to(cuda), torch.from_numpy(g["indices"]).to(cuda), torch.from_numpy(g["indptr"]).to(cuda)
    y = fs.flagsparse_spmv_csr(d, i, p, g["x"].to(cuda), g["shape"])
    C = fs.flagsparse_spmm_csr(d, i, p.to(torch.int64), g["B"].to(cuda), g["shape"])
    for got, ref_out, operand in ((y, g["y"], g["x"]), (C, g["C"], g["B"])):
        mag = np.asarray(abs(a) @ np.abs(operand.to(wide).numpy()))
        err = np.abs(got.cpu().to(wide).numpy() - ref_out.to(wide).numpy())
        assert got.dtype == ref_out.dtype and tuple(got.shape) == tuple(ref_out.shape)
        assert np.all(err <= GOLDEN_TOL[tag] * mag + 1e-300), float((err / np.maximum(mag, 1e-300)).max())
