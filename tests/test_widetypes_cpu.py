"""float16 / bfloat16 / complex values on CPU: the host side of the entry points (flagsparse_b200/widetypes.py:
widening of the dense operand, one launch, one rounding) with host stand-ins for fsb_spmv_csr_wide /
fsb_spmm_csr_wide, against exact products of the stored values and against outputs of the reference's own base
paths (tests/golden/wide_*.npz)."""

import numpy as np
import pytest
import scipy.sparse as sp
import torch

import flagsparse_b200 as fs
from fake_device import fake_cuda
from flagsparse_b200 import widetypes as W
from helpers import handmade_csr


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
def test_product_of_the_stored_values(dtype, n_dense, fsb_lib):
    vals, i, p, shape = _matrix(dtype)
    rng = np.random.default_rng(7)
    oshape = (shape[1],) if n_dense is None else (shape[1], n_dense)
    if dtype in W.COMPLEX_DTYPES:
        operand = torch.from_numpy(rng.uniform(-1, 1, oshape) + 1j * rng.uniform(-1, 1, oshape)).to(dtype)
    else:
        operand = torch.from_numpy(rng.uniform(-1, 1, oshape)).to(dtype)
    ti, tp = torch.from_numpy(i), torch.from_numpy(p)
    with fake_cuda() as launches:
        if n_dense is None:
            y = fs.flagsparse_spmv_csr(vals, ti, tp, operand, shape)
            assert launches.spmv == ["wide"]
        else:
            y = fs.flagsparse_spmm_csr(vals, ti, tp, operand, shape)
            assert launches.spmm == [("wide", n_dense)]
    assert y.dtype == dtype and tuple(y.shape) == ((shape[0],) if n_dense is None else (shape[0], n_dense))
    # reference: the same matrix and operand (as stored, i.e. after their own rounding) in the widest type
    wide = torch.complex128 if dtype in W.COMPLEX_DTYPES else torch.float64
    a = sp.csr_matrix((vals.to(wide).numpy(), i, p), shape=shape)
    ref = np.asarray(a @ operand.to(wide).numpy())
    mag = np.asarray(abs(a) @ np.abs(operand.to(wide).numpy()))
    eps = {torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -8, torch.complex64: 1e-6, torch.complex128: 1e-14}[dtype]
    err = np.abs(y.to(wide).numpy() - ref)
    assert np.all(err <= 2 * eps * mag + 1e-300), float((err / np.maximum(mag, 1e-300)).max())
    assert not y.to(wide).numpy()[np.diff(p) == 0].any()          # empty rows stay exact zeros


def test_half_precision_result_is_the_rounded_float32_result(fsb_lib):
    vals, i, p, shape = _matrix(torch.float16)
    x = torch.from_numpy(np.random.default_rng(3).uniform(-1, 1, shape[1])).to(torch.float16)
    with fake_cuda():
        y = fs.flagsparse_spmv_csr(vals, torch.from_numpy(i), torch.from_numpy(p), x, shape)
    part = sp.csr_matrix((vals.to(torch.float32).numpy(), i, p), shape=shape)
    y32 = torch.from_numpy(np.asarray(part @ x.to(torch.float32).numpy()))
    assert torch.equal(y, y32.to(torch.float16))


def test_dense_types_and_strided_operands():
    assert W.dense_dtype(torch.float16) == W.dense_dtype(torch.bfloat16) == torch.float32
    assert W.dense_dtype(torch.complex64) == torch.complex64 and W.dense_dtype(torch.complex128) == torch.complex128
    for dt in (torch.float32, torch.float64):
        with pytest.raises(TypeError):
            W.dense_dtype(dt)

    class P:
        data = torch.ones(2, dtype=torch.complex64)

    seen = []

    def launch(prepared, o, r):
        seen.append((o.dtype, o.is_contiguous(), o.stride(-1)))
        r.zero_()

    wide = torch.zeros(6, 8, dtype=torch.complex64)
    W.run(P, wide[:, :5], launch, (2, 5))                 # a row stride: handed on as it is
    W.run(P, wide.t()[:5], launch, (2, 6))                # column-major: copied
    W.run(P, wide[0, ::2], launch, (2,))                  # strided vector: copied
    assert seen == [(torch.complex64, False, 1), (torch.complex64, True, 1), (torch.complex64, True, 1)]


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
def test_arithmetic_against_reference_outputs(tag, fsb_lib):
    g, dt = load_wide_golden(tag)
    wide = torch.complex128 if dt in W.COMPLEX_DTYPES else torch.float64
    a = sp.csr_matrix((g["data"].to(wide).numpy(), g["indices"], g["indptr"]), shape=g["shape"])
    ti, tp = torch.from_numpy(g["indices"]), torch.from_numpy(g["indptr"])
    with fake_cuda():
        got_y = fs.flagsparse_spmv_csr(g["data"], ti, tp, g["x"], g["shape"])
        got_c = fs.flagsparse_spmm_csr(g["data"], ti, tp.to(torch.int64), g["B"], g["shape"])
    for operand, ref_out, got in ((g["x"], g["y"], got_y), (g["B"], g["C"], got_c)):
        mag = np.asarray(abs(a) @ np.abs(operand.to(wide).numpy()))
        err = np.abs(got.to(wide).numpy() - ref_out.to(wide).numpy())
        assert got.dtype == ref_out.dtype and got.shape == ref_out.shape
        assert np.all(err <= GOLDEN_TOL[tag] * mag + 1e-300), float((err / np.maximum(mag, 1e-300)).max())
        # the reference's own output against the exact product of the stored values: same bound as ours gets
        exact = np.asarray(a @ operand.to(wide).numpy())
        assert np.all(np.abs(ref_out.to(wide).numpy() - exact) <= GOLDEN_TOL[tag] * mag + 1e-300)
