"""SDDMM without a GPU: the float64 oracle against outputs of the reference's own kernel (tests/golden/sddmm_*.npz),
and the host code of flagsparse_sddmm_csr (checks, their order and exception types as in the reference's
src/flagsparse/sparse_operations/sddmm_csr.py:46-80, 206-242, 350-422) with the launch replaced by a numpy
stand-in.  No kernel is launched here."""

from unittest import mock

import numpy as np
import pytest
import torch

import flagsparse_b200 as fs
from flagsparse_b200 import sddmm_csr
from helpers import golden_files, golden_index, load_golden
from oracle import csr_oracle as O


@pytest.mark.parametrize("path", golden_files("sddmm"), ids=lambda p: p.split("/")[-1])
def test_oracle_matches_reference_outputs(path):
    g = load_golden(path)
    data = g["data"] if bool(g["has_in"]) else None
    ref, mag = O.sddmm_f64(data, g["indices"], g["indptr"], g["x"], g["y"], float(g["alpha"]), float(g["beta"]))
    assert ref.shape == g["out"].shape
    assert O.within_bound(g["out"], ref, mag, g["x"].dtype)
    # the row of every entry, as the reference's prepare builds it
    rows = np.repeat(np.arange(g["indptr"].shape[0] - 1), np.diff(g["indptr"].astype(np.int64)))
    assert np.array_equal(rows, g["row_ids"])


def test_oracle_definition_by_loops():
    g = load_golden(golden_files("sddmm")[0])
    ref, _ = O.sddmm_f64(g["data"], g["indices"], g["indptr"], g["x"], g["y"], 0.5, -2.0)
    p = 0
    for r in range(g["indptr"].shape[0] - 1):
        for q in range(int(g["indptr"][r]), int(g["indptr"][r + 1])):
            want = 0.5 * float(np.dot(g["x"][r].astype(np.float64), g["y"][g["indices"][q]].astype(np.float64)))
            want += -2.0 * float(g["data"][q])
            assert abs(ref[q] - want) <= 1e-12 * max(1.0, abs(want))
            p += 1
    assert p == ref.shape[0]


def _stand_in(prepared, x, y, data, alpha, beta, out):
    """What fsb_sddmm_csr computes, in numpy (value-type result of the float64 definition)."""
    assert x.stride(1) == 1 or x.shape[1] <= 1
    assert y.stride(1) == 1 or y.shape[1] <= 1
    assert out.is_contiguous() and (data is None or data.is_contiguous())
    ref, _ = O.sddmm_f64(None if data is None else data.numpy(), prepared.indices.numpy(), prepared.indptr.numpy(),
                         x.numpy(), y.numpy(), alpha, beta)
    out.copy_(torch.from_numpy(ref.astype(x.numpy().dtype)))


@pytest.fixture()
def host():
    patches = [
        mock.patch.object(torch.Tensor, "is_cuda", new_callable=mock.PropertyMock, return_value=True),
        mock.patch.object(sddmm_csr, "_sddmm_launch", _stand_in),
        mock.patch.object(torch.cuda, "synchronize", lambda *a, **k: None),
    ]
    for p in patches:
        p.start()
    yield
    for p in reversed(patches):
        p.stop()


def _pattern():
    indices = torch.tensor([0, 2, 1, 1, 3], dtype=torch.int32)
    indptr = torch.tensor([0, 2, 2, 5], dtype=torch.int64)
    return indices, indptr, (3, 4)


def test_goldens_through_the_entry_point(host):
    for path in golden_files("sddmm"):
        g = load_golden(path)
        t = {k: torch.from_numpy(g[k]) for k in ("data", "indices", "indptr", "x", "y")}
        data = t["data"] if bool(g["has_in"]) else None
        out, meta = fs.flagsparse_sddmm_csr(data, t["indices"], t["indptr"], t["x"], t["y"], g["shape"],
                                            alpha=float(g["alpha"]), beta=float(g["beta"]), return_meta=True)
        ref, mag = O.sddmm_f64(None if data is None else g["data"], g["indices"], g["indptr"], g["x"], g["y"],
                               float(g["alpha"]), float(g["beta"]))
        assert O.within_bound(out.numpy(), ref, mag, g["x"].dtype)
        name = path.split("sddmm_")[-1][:-4]
        want = golden_index()["sddmm"][name]
        assert (meta["block_k"], meta["num_warps"]) == (want["block_k"], want["num_warps"])
        assert meta["fallback_used"] is False


def test_prepared_pattern_and_bookkeeping(host):
    indices, indptr, shape = _pattern()
    p = fs.prepare_sddmm_csr(indices, indptr.to(torch.int32), shape, k_hint=200)
    assert isinstance(p, fs.SDDMMPrepared)
    assert (p.n_rows, p.n_cols, p.nnz, p.block_k, p.num_warps) == (3, 4, 5, 128, 8)
    assert p.indptr.dtype == torch.int64 and p.row_ids.dtype == torch.int32
    assert p.row_ids.tolist() == [0, 0, 2, 2, 2]
    for k, want in ((1, (32, 2)), (32, (32, 2)), (33, (64, 4)), (128, (64, 4)), (129, (128, 8))):
        assert sddmm_csr._launch_bookkeeping(k) == want
    empty = fs.prepare_sddmm_csr(indices[:0], torch.zeros(1, dtype=torch.int64), (0, 4))
    assert empty.nnz == 0 and empty.row_ids.numel() == 0


def test_checks_and_exception_types(host):
    indices, indptr, shape = _pattern()
    x = torch.randn(3, 6)
    y = torch.randn(4, 6)
    data = torch.randn(5)
    f = fs.flagsparse_sddmm_csr
    cases = [
        (lambda: f(None, None, indptr, x, y, shape), ValueError),
        (lambda: f(None, indices, indptr, x, y, (3, 4, 1)), ValueError),
        (lambda: f(None, indices.reshape(1, -1), indptr, x, y, shape), ValueError),
        (lambda: f(None, indices, indptr, x, y, (-1, 4)), ValueError),
        (lambda: f(None, indices, indptr[:-1], x, y, shape), ValueError),
        (lambda: f(None, indices.to(torch.int64), indptr, x, y, shape), TypeError),
        (lambda: f(None, indices, indptr.to(torch.float32), x, y, shape), TypeError),
        (lambda: f(None, indices, torch.tensor([1, 2, 2, 5]), x, y, shape), ValueError),
        (lambda: f(None, indices, torch.tensor([0, 2, 2, 4]), x, y, shape), ValueError),
        (lambda: f(None, indices, torch.tensor([0, 3, 2, 5]), x, y, shape), ValueError),
        (lambda: f(None, torch.tensor([0, 2, 1, 1, 4], dtype=torch.int32), indptr, x, y, shape), IndexError),
        (lambda: f(None, torch.tensor([0, -1, 1, 1, 3], dtype=torch.int32), indptr, x, y, shape), IndexError),
        (lambda: f(None, indices, indptr, None, y, shape), ValueError),
        (lambda: f(None, indices, indptr, x, y, shape, beta=1.0), ValueError),
        (lambda: f(None, indices, indptr, x[0], y, shape), ValueError),
        (lambda: f(None, indices, indptr, x.to(torch.float16), y.to(torch.float16), shape), TypeError),
        (lambda: f(None, indices, indptr, x, y.to(torch.float64), shape), TypeError),
        (lambda: f(data.to(torch.float64), indices, indptr, x, y, shape, beta=1.0), TypeError),
        (lambda: f(None, indices, indptr, x[:2], y, shape), ValueError),
        (lambda: f(None, indices, indptr, x, y[:3], shape), ValueError),
        (lambda: f(None, indices, indptr, x, y[:, :5], shape), ValueError),
        (lambda: f(data[:4], indices, indptr, x, y, shape, beta=1.0), ValueError),
        (lambda: f(None, indices, indptr, x, y, shape, out=torch.empty(4)), ValueError),
        (lambda: f(None, indices, indptr, x, y, shape, out=torch.empty(5, dtype=torch.float64)), TypeError),
        (lambda: f(None, indices, indptr, x, y, shape, prepared=object()), TypeError),
    ]
    for i, (call, exc) in enumerate(cases):
        with pytest.raises(exc):
            call()
            pytest.fail(f"case {i} did not raise")


def test_return_forms_out_and_k_zero(host):
    indices, indptr, shape = _pattern()
    x = torch.randn(3, 6, dtype=torch.float64)
    y = torch.randn(4, 6, dtype=torch.float64)
    data = torch.randn(5, dtype=torch.float64)
    p = fs.prepare_sddmm_csr(indices, indptr, shape)
    ref, _ = O.sddmm_f64(data.numpy(), indices.numpy(), indptr.numpy(), x.numpy(), y.numpy(), 2.0, 0.5)
    out = torch.empty(5, dtype=torch.float64)
    got = fs.flagsparse_sddmm_csr(data, x=x, y=y, alpha=2.0, beta=0.5, prepared=p, out=out)
    assert got is out and np.allclose(out.numpy(), ref, rtol=1e-14, atol=0)
    r = fs.flagsparse_sddmm_csr(data, x=x, y=y, prepared=p, return_time=True)
    assert len(r) == 2 and r[1] >= 0.0
    r = fs.flagsparse_sddmm_csr(data, x=x, y=y, prepared=p, return_time=True, return_meta=True)
    assert len(r) == 3 and r[2]["prepare_ms"] == 0.0 and r[2]["out_dtype"] == "float64"
    # a strided `out` still receives the result; strided x / y are passed with their row stride
    wide = torch.zeros(10, dtype=torch.float64)
    fs.flagsparse_sddmm_csr(data, x=x, y=y, alpha=2.0, beta=0.5, prepared=p, out=wide[::2])
    assert np.allclose(wide[::2].numpy(), ref, rtol=1e-14, atol=0) and float(wide[1::2].abs().sum()) == 0.0
    xs = torch.randn(3, 9, dtype=torch.float64)[:, :6]
    got = fs.flagsparse_sddmm_csr(None, x=xs, y=y.t().contiguous().t(), prepared=p)
    ref2, _ = O.sddmm_f64(None, indices.numpy(), indptr.numpy(), xs.numpy(), y.numpy())
    assert np.allclose(got.numpy(), ref2, rtol=1e-14, atol=0)
    # K = 0: out = beta * data, or zeros without data (the reference's :385-397)
    x0, y0 = x[:, :0], y[:, :0]
    assert torch.equal(fs.flagsparse_sddmm_csr(data, x=x0, y=y0, beta=3.0, prepared=p), data * 3.0)
    z = fs.flagsparse_sddmm_csr(None, x=x0, y=y0, prepared=p, out=torch.ones(5, dtype=torch.float64))
    assert float(z.abs().sum()) == 0.0
    out0, ms = fs.flagsparse_sddmm_csr(data, x=x0, y=y0, prepared=p, return_time=True)
    assert ms == 0.0 and float(out0.abs().sum()) == 0.0
