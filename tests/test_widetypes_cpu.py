"""float16 / bfloat16 / complex values through real products (flagsparse_b200/widetypes.py), with a host stand-in
for the CUDA launch: the arithmetic of the split and of the recombination, for a vector and for a dense block."""

import numpy as np
import pytest
import scipy.sparse as sp
import torch

from flagsparse_b200 import widetypes as W
from helpers import handmade_csr


def _launch(part, operand, result):
    """Stand-in for the CUDA launch: part is a scipy matrix in the compute type."""
    assert operand.is_contiguous() and operand.dtype == result.dtype
    result.copy_(torch.from_numpy(np.asarray(part @ operand.numpy())))


def _matrix(dtype, seed=1):
    lens = [0, 3, 17, 1, 0, 40, 5, 9]
    d, i, p = handmade_csr(seed, lens, 64, value_dtype=np.float64)
    rng = np.random.default_rng(seed + 1)
    if dtype in W.COMPLEX_DTYPES:
        vals = torch.from_numpy(d + 1j * rng.uniform(-1, 1, d.size)).to(dtype)
    else:
        vals = torch.from_numpy(d).to(dtype)
    return vals, i, p, (len(lens), 64)


@pytest.mark.parametrize("dtype", W.WIDE_DTYPES, ids=str)
@pytest.mark.parametrize("n_dense", [None, 5])
def test_product_through_real_parts(dtype, n_dense):
    vals, i, p, shape = _matrix(dtype)
    kind, reals = W.split_values(vals)
    comp = W.compute_dtype(dtype)
    assert kind == ("cast" if dtype in W.HALF_DTYPES else "complex") and all(r.dtype == comp for r in reals)
    assert len(reals) == (1 if kind == "cast" else 2) and all(r.is_contiguous() for r in reals)
    parts = [sp.csr_matrix((r.numpy(), i, p), shape=shape) for r in reals]
    rng = np.random.default_rng(7)
    oshape = (shape[1],) if n_dense is None else (shape[1], n_dense)
    if dtype in W.COMPLEX_DTYPES:
        operand = torch.from_numpy(rng.uniform(-1, 1, oshape) + 1j * rng.uniform(-1, 1, oshape)).to(dtype)
    else:
        operand = torch.from_numpy(rng.uniform(-1, 1, oshape)).to(dtype)
    out_shape = (shape[0],) if n_dense is None else (shape[0], n_dense)
    y = W.product(kind, parts, operand, _launch, out_shape, dtype)
    assert y.dtype == dtype and tuple(y.shape) == out_shape
    # reference: the same matrix and operand (as stored, i.e. after their own rounding) in the widest type
    wide = torch.complex128 if dtype in W.COMPLEX_DTYPES else torch.float64
    a = sp.csr_matrix((vals.to(wide).numpy(), i, p), shape=shape)
    ref = np.asarray(a @ operand.to(wide).numpy())
    mag = np.asarray(abs(a) @ np.abs(operand.to(wide).numpy()))
    eps = {torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -8, torch.complex64: 1e-6, torch.complex128: 1e-14}[dtype]
    err = np.abs(y.to(wide).numpy() - ref)
    assert np.all(err <= 2 * eps * mag + 1e-300), float((err / np.maximum(mag, 1e-300)).max())
    assert not y.to(wide).numpy()[np.diff(p) == 0].any()          # empty rows stay exact zeros


def test_half_precision_result_is_the_rounded_float32_result():
    vals, i, p, shape = _matrix(torch.float16)
    kind, reals = W.split_values(vals)
    part = sp.csr_matrix((reals[0].numpy(), i, p), shape=shape)
    x = torch.from_numpy(np.random.default_rng(3).uniform(-1, 1, shape[1])).to(torch.float16)
    y = W.product(kind, [part], x, _launch, (shape[0],), torch.float16)
    y32 = torch.from_numpy(np.asarray(part @ x.to(torch.float32).numpy()))
    assert torch.equal(y, y32.to(torch.float16))


def test_native_types_are_not_split():
    for dt in (torch.float32, torch.float64):
        assert W.compute_dtype(dt) == dt
        with pytest.raises(TypeError):
            W.split_values(torch.ones(3, dtype=dt))
    assert W.compute_dtype(torch.complex128) == torch.float64 and W.compute_dtype(torch.bfloat16) == torch.float32
    with pytest.raises(ValueError):
        W.product("other", [], torch.ones(2), _launch, (2,), torch.float32)


# ---- against outputs of the reference's own base paths (tests/golden/wide_*.npz) ----------------------------------
GOLDEN_DTYPES = {"f16": torch.float16, "bf16": torch.bfloat16, "c64": torch.complex64, "c128": torch.complex128}
# the reference rounds a float32 (or float64) sum to the caller's type as this package does; the sums themselves may
# differ in their last bits (another order of additions), which can move the rounded result by one unit
GOLDEN_TOL = {"f16": 2.0 ** -10, "bf16": 2.0 ** -7, "c64": 4e-6, "c128": 4e-15}


def load_wide_golden(tag):
    import os

    from helpers import GOLDEN, load_golden

    g = load_golden(os.path.join(GOLDEN, f"wide_{tag}.npz"))
    dt = GOLDEN_DTYPES[tag]
    for k in ("data", "x", "B", "y", "C"):
        g[k] = torch.from_numpy(g[k]).to(dt)      # float16 / bfloat16 were stored widened to float32 (exact)
    return g, dt


@pytest.mark.parametrize("tag", sorted(GOLDEN_DTYPES))
def test_arithmetic_against_reference_outputs(tag):
    g, dt = load_wide_golden(tag)
    kind, reals = W.split_values(g["data"])
    parts = [sp.csr_matrix((r.numpy(), g["indices"], g["indptr"]), shape=g["shape"]) for r in reals]
    wide = torch.complex128 if dt in W.COMPLEX_DTYPES else torch.float64
    a = sp.csr_matrix((g["data"].to(wide).numpy(), g["indices"], g["indptr"]), shape=g["shape"])
    for operand, ref_out in ((g["x"], g["y"]), (g["B"], g["C"])):
        out_shape = (g["shape"][0],) + tuple(operand.shape[1:])
        got = W.product(kind, parts, operand, _launch, out_shape, dt)
        mag = np.asarray(abs(a) @ np.abs(operand.to(wide).numpy()))
        err = np.abs(got.to(wide).numpy() - ref_out.to(wide).numpy())
        assert got.dtype == ref_out.dtype and got.shape == ref_out.shape
        assert np.all(err <= GOLDEN_TOL[tag] * mag + 1e-300), float((err / np.maximum(mag, 1e-300)).max())
        # the reference's own output against the exact product of the stored values: same bound as ours gets
        exact = np.asarray(a @ operand.to(wide).numpy())
        assert np.all(np.abs(ref_out.to(wide).numpy() - exact) <= GOLDEN_TOL[tag] * mag + 1e-300)
