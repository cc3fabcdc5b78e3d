"""SDDMM on the GPU, through the C ABI (fsb_sddmm_csr) and through flagsparse_sddmm_csr: the reference kernel's own
outputs (tests/golden/sddmm_*.npz), edge shapes, every vector width and group size the launcher can pick, strided
operands, and size-independent properties on a pattern with 2^24 entries."""

import numpy as np
import pytest
import torch

import flagsparse_b200 as fs
from flagsparse_b200 import _lib
from flagsparse_b200 import synthetic as S
from gpu_util import dev
from helpers import golden_files, handmade_csr, load_golden
from oracle import csr_oracle as O

pytestmark = pytest.mark.gpu

TOL = {np.dtype(np.float32): 1e-5, np.dtype(np.float64): 1e-13}


def _check(out, data, indices, indptr, x, y, alpha=1.0, beta=0.0, what=""):
    ref, mag = O.sddmm_f64(data, indices, indptr, x, y, alpha, beta)
    got = out.cpu().numpy()
    assert got.dtype == x.dtype and got.shape == ref.shape, what
    ratio = O.max_bound_ratio(got, ref, mag)
    assert ratio <= TOL[np.dtype(x.dtype)], f"{what}: max |out-ref| / bound = {ratio:.3e}"
    return ratio


@pytest.mark.parametrize("path", golden_files("sddmm"), ids=lambda p: p.split("/")[-1])
def test_golden_fixtures(path, cuda, fsb_lib):
    g = load_golden(path)
    has_in = bool(g["has_in"])
    alpha, beta = float(g["alpha"]), float(g["beta"])
    data = dev(g["data"]) if has_in else None
    out = fs.flagsparse_sddmm_csr(data, dev(g["indices"]), dev(g["indptr"]), dev(g["x"]), dev(g["y"]), g["shape"],
                                  alpha=alpha, beta=beta)
    _check(out, g["data"] if has_in else None, g["indices"], g["indptr"], g["x"], g["y"], alpha, beta, path)
    # next to the reference kernel's own output: both within the bound of the float64 definition, so within twice
    # the bound of each other
    ref, mag = O.sddmm_f64(g["data"] if has_in else None, g["indices"], g["indptr"], g["x"], g["y"], alpha, beta)
    assert O.max_bound_ratio(out.cpu().numpy(), g["out"], mag) <= 2 * TOL[np.dtype(g["x"].dtype)]


def test_direct_c_abi_call(cuda, fsb_lib):
    g = load_golden(golden_files("sddmm")[0])
    idx, x, y, d = dev(g["indices"]), dev(g["x"]), dev(g["y"]), dev(g["data"])
    rows = dev(np.repeat(np.arange(g["shape"][0], dtype=np.int32), np.diff(g["indptr"].astype(np.int64))))
    out = torch.empty_like(d)
    vt = _lib.FSB_F32 if g["x"].dtype == np.float32 else _lib.FSB_F64
    st = torch.cuda.current_stream().cuda_stream
    call = lambda o, dd, a, b: fsb_lib.fsb_sddmm_csr(  # noqa: E731
        vt, idx.data_ptr(), rows.data_ptr(), x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0),
        None if dd is None else dd.data_ptr(), o.data_ptr(), g["shape"][0], g["shape"][1], idx.numel(), x.shape[1], a, b, st)
    assert call(out, d, 0.5, -2.0) == 0
    _check(out, g["data"], g["indices"], g["indptr"], g["x"], g["y"], 0.5, -2.0, "C ABI")
    # out may alias data
    alias = d.clone()
    assert call(alias, alias, 0.5, -2.0) == 0
    assert torch.equal(alias, out)
    # argument errors come back as codes, before any launch
    assert fsb_lib.fsb_sddmm_csr(9, idx.data_ptr(), rows.data_ptr(), x.data_ptr(), x.stride(0), y.data_ptr(),
                                 y.stride(0), None, out.data_ptr(), 1, 1, 1, 1, 1.0, 0.0, st) == -1
    assert fsb_lib.fsb_sddmm_csr(vt, idx.data_ptr(), rows.data_ptr(), x.data_ptr(), 2, y.data_ptr(), y.stride(0),
                                 None, out.data_ptr(), g["shape"][0], g["shape"][1], idx.numel(), x.shape[1], 1.0, 0.0,
                                 st) == -1  # ldx < K
    assert fsb_lib.fsb_sddmm_csr(vt, None, None, None, 0, None, 0, None, None, 3, 3, 0, 4, 1.0, 0.0, st) == 0  # nnz = 0


@pytest.mark.parametrize("vdtype", [np.float32, np.float64])
@pytest.mark.parametrize("k", [1, 2, 3, 4, 5, 8, 12, 16, 31, 32, 33, 64, 100, 128, 129, 256, 300, 515])
def test_every_width(vdtype, k, cuda, fsb_lib):
    lens = [0, 1, 0, 9, 33, 2, 0, 0, 64, 7, 130, 1, 1, 0, 5]
    data, indices, indptr = handmade_csr(100 + k, lens, 90, vdtype, np.int32, np.int64)
    rng = np.random.default_rng(k)
    x = rng.uniform(-1, 1, (len(lens), k)).astype(vdtype)
    y = rng.uniform(-1, 1, (90, k)).astype(vdtype)
    p = fs.prepare_sddmm_csr(dev(indices), dev(indptr), (len(lens), 90), k_hint=k)
    out = fs.flagsparse_sddmm_csr(dev(data), x=dev(x), y=dev(y), alpha=-0.75, beta=1.5, prepared=p)
    _check(out, data, indices, indptr, x, y, -0.75, 1.5, f"K={k}")
    again = fs.flagsparse_sddmm_csr(dev(data), x=dev(x), y=dev(y), alpha=-0.75, beta=1.5, prepared=p)
    assert torch.equal(out, again)
    no_in = fs.flagsparse_sddmm_csr(None, x=dev(x), y=dev(y), prepared=p)
    _check(no_in, None, indices, indptr, x, y, 1.0, 0.0, f"K={k} no data")


def test_edge_shapes_and_strides(cuda, fsb_lib):
    # no entries at all; one entry; a single long row; rows of X / Y with a stride; operands that start off 16 bytes
    z = fs.flagsparse_sddmm_csr(None, torch.empty(0, dtype=torch.int32, device=cuda),
                                torch.zeros(4, dtype=torch.int64, device=cuda), torch.randn(3, 8, device=cuda),
                                torch.randn(5, 8, device=cuda), (3, 5))
    assert z.numel() == 0
    for lens, n_cols in (([1], 1), ([0, 0, 1], 7), ([700], 700), ([3] * 1000, 50)):
        data, indices, indptr = handmade_csr(len(lens), lens, n_cols)
        rng = np.random.default_rng(7)
        xw = rng.uniform(-1, 1, (len(lens), 40)).astype(np.float32)
        yw = rng.uniform(-1, 1, (n_cols, 44)).astype(np.float32)
        for lo, k in ((0, 40), (0, 36), (1, 33), (4, 32), (3, 1)):
            xd, yd = dev(xw)[:, lo:lo + k], dev(yw)[:, lo:lo + k]
            out = fs.flagsparse_sddmm_csr(dev(data), dev(indices), dev(indptr), xd, yd, (len(lens), n_cols), beta=1.0)
            _check(out, data, indices, indptr, xw[:, lo:lo + k], yw[:, lo:lo + k], 1.0, 1.0, f"{lens[:3]} {lo}:{k}")
    # column-major operands are copied by the entry point, as the reference's .contiguous() does
    data, indices, indptr = handmade_csr(5, [4, 0, 6], 9)
    x = np.random.default_rng(1).uniform(-1, 1, (3, 10)).astype(np.float32)
    y = np.random.default_rng(2).uniform(-1, 1, (9, 10)).astype(np.float32)
    out = fs.flagsparse_sddmm_csr(None, dev(indices), dev(indptr), dev(x.T.copy()).t(), dev(y.T.copy()).t(), (3, 9))
    _check(out, None, indices, indptr, x, y, what="column-major operands")
    # a strided `out`
    wide = torch.zeros(20, device=cuda)
    fs.flagsparse_sddmm_csr(None, dev(indices), dev(indptr), dev(x), dev(y), (3, 9), out=wide[::2])
    assert torch.equal(wide[::2], out) and float(wide[1::2].abs().sum()) == 0.0


@pytest.mark.parametrize("k", [32, 64, 128])
def test_large_pattern_properties(k, cuda, fsb_lib):
    """2^20 rows x 16 entries (the SpMM configuration's pattern): sampled rows against the oracle, run-to-run bit
    equality, exact scaling in alpha, and beta * data added exactly once."""
    spec = S.config_spec("c4")
    data, indices, indptr = S.generate_csr(spec, cuda)
    n_rows, n_cols = spec.n_rows, spec.n_cols
    g = torch.Generator(device=cuda).manual_seed(k)
    x = torch.rand((n_rows, k), device=cuda, generator=g) * 2 - 1
    y = torch.rand((n_cols, k), device=cuda, generator=g) * 2 - 1
    p = fs.prepare_sddmm_csr(indices.to(torch.int32), indptr, (n_rows, n_cols), k_hint=k)
    out = fs.flagsparse_sddmm_csr(None, x=x, y=y, prepared=p)
    assert torch.equal(out, fs.flagsparse_sddmm_csr(None, x=x, y=y, prepared=p))
    assert torch.equal(fs.flagsparse_sddmm_csr(None, x=x, y=y, alpha=4.0, prepared=p), out * 4.0)
    with_in = fs.flagsparse_sddmm_csr(data, x=x, y=y, alpha=0.0, beta=2.0, prepared=p)
    assert torch.equal(with_in, data * 2.0)
    ptr = indptr.cpu().numpy().astype(np.int64)
    yh = y.cpu().numpy()
    for r0 in (0, 524288 - 5, n_rows - 2048):
        r1 = r0 + 2048
        lo, hi = int(ptr[r0]), int(ptr[r1])
        _check(out[lo:hi], None, indices[lo:hi].cpu().numpy(), ptr[r0:r1 + 1] - lo, x[r0:r1].cpu().numpy(), yh,
               what=f"rows {r0}:{r1}")
