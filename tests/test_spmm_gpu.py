"""CSR SpMM on the GPU against the oracle: golden fixtures, dense widths that exercise every vector width
and column tiling, long rows, both staging modes, and the benchmark configuration."""

import numpy as np
import pytest
import torch

import flagsparse_b200 as fs
from flagsparse_b200 import synthetic as S
from gpu_util import check_spmm_blocks, dev, env, sample_blocks, spmm
from helpers import assert_spmm_ok, golden_files, handmade_csr, load_golden

pytestmark = pytest.mark.gpu

STAGING = ["plain", "bulk"]


@pytest.mark.parametrize("staging", STAGING)
@pytest.mark.parametrize("path", golden_files("spmm"), ids=lambda p: p.split("/")[-1])
def test_golden_fixtures(cuda, fsb_lib, path, staging):
    g = load_golden(path)
    args = (g["data"], g["indices"], g["indptr"], g["shape"], g["B"])
    for opt in (False, True):
        c = spmm(*args, algo=staging, opt=opt)
        assert_spmm_ok(c, *args, what=path)
        atol, rtol = fs._tolerance_for_dtype(torch.float32 if c.dtype == np.float32 else torch.float64)
        for key in ("C_base", "C_opt"):
            assert np.allclose(c, g[key], atol=atol * 10, rtol=rtol * 10), key


# widths: 1..3 (scalar), 2/6 (64-bit), multiples of 4 (128-bit), above 128 (several column tiles);
# the first group mirrors the reference's tile-branch list N in {4,5,12,24,48,96} (tests/test_spmm.py:47-54)
@pytest.mark.parametrize("n_dense", [1, 2, 3, 4, 5, 6, 8, 12, 24, 32, 48, 64, 96, 128, 129, 200, 256])
def test_dense_widths(cuda, fsb_lib, n_dense):
    T = 1024
    lens = [0, 16, 16, 1, 0, T - 33, 40, 3 * T + 7, 0, 0, 5, 64, 2500, 1]
    for vdt, idt, pdt in ((np.float32, np.int32, np.int64), (np.float64, np.int64, np.int32)):
        data, idx, ptr = handmade_csr(31, lens, 5000, vdt, idt, pdt)
        b = np.random.default_rng(32).uniform(-1, 1, (5000, n_dense)).astype(vdt)
        got = {}
        for staging in STAGING:
            c = spmm(data, idx, ptr, (len(lens), 5000), b, algo=staging)
            assert_spmm_ok(c, data, idx, ptr, (len(lens), 5000), b, what=f"N={n_dense}/{staging}")
            assert np.all(c[np.asarray(lens) == 0] == 0)
            got[staging] = c
        assert np.array_equal(got["plain"], got["bulk"])  # staging changes how the tile arrives, not the sums


def test_many_short_rows_and_tile_edges(cuda, fsb_lib):
    T = 1024
    for lens in ([1] * 3000, [T] * 3 + [T // 2, T // 2, 7], [0] * 2000 + [2] * 1500, [5 * T + 1]):
        data, idx, ptr = handmade_csr(33, lens, 4096)
        b = np.random.default_rng(34).uniform(-1, 1, (4096, 20)).astype(np.float32)
        for staging in STAGING:
            c = spmm(data, idx, ptr, (len(lens), 4096), b, algo=staging, opt=True)
            assert_spmm_ok(c, data, idx, ptr, (len(lens), 4096), b, what=f"{len(lens)} rows/{staging}")


def test_noncontiguous_b_out_and_determinism(cuda, fsb_lib):
    spec = S.config_spec("c4").scaled(1 << 12)
    data, idx, ptr = S.generate_csr(spec, None)
    bt = np.random.default_rng(35).uniform(-1, 1, (24, spec.n_cols)).astype(np.float32)
    d, i, p = dev(data), dev(idx), dev(ptr)
    b_nc = dev(bt).transpose(0, 1)
    assert not b_nc.is_contiguous()
    shape = (spec.n_rows, spec.n_cols)
    c = fs.flagsparse_spmm_csr(d, i, p, b_nc, shape)
    assert c.is_contiguous()
    assert_spmm_ok(c.cpu().numpy(), data, idx, ptr, shape, bt.T)
    out = torch.empty((spec.n_rows, 24), dtype=torch.float32, device="cuda:0")
    c2 = fs.flagsparse_spmm_csr(d, i, p, b_nc, shape, out=out)
    assert c2.data_ptr() == out.data_ptr() and torch.equal(out, c)
    prep = fs.prepare_spmm_csr_opt(d, i, p, shape)
    c3 = fs.flagsparse_spmm_csr_opt(B=b_nc, prepared=prep)
    c4, ms = fs.flagsparse_spmm_csr_opt(B=b_nc, prepared=prep, return_time=True)
    assert torch.equal(c3, c) and torch.equal(c4, c) and ms > 0
    assert int(prep.status_word().item()) == 0  # no bounded wait ran out
    assert prep.row_lengths.tolist() == [16] * spec.n_rows and prep.max_row_nnz == 16
    assert not prep.long_row_fallback_only and prep.supports_opt
    # a strided output is filled through a copy
    wide = torch.zeros((spec.n_rows, 48), dtype=torch.float32, device="cuda:0")
    c5 = fs.flagsparse_spmm_csr_opt(B=b_nc, prepared=prep, out=wide[:, ::2])
    assert torch.equal(wide[:, ::2], c) and c5.data_ptr() == wide.data_ptr()


@pytest.mark.parametrize("vdt", ["float32", "float64"])
@pytest.mark.parametrize("n_panels", [2, 3])
def test_column_panels_and_tiles(cuda, fsb_lib, vdt, n_panels):
    """The split product (column panels of A, column tiles of B and C, later passes adding to C) on a matrix with
    long rows that cross tile boundaries, empty rows, a width that is not a multiple of the tile, a row-strided B
    and a row-strided C."""
    lens = ([0, 3, 40, 0, 1, 2500, 7, 0] * 60) + [9000, 0, 0, 5]
    data, idx, ptr = handmade_csr(21, lens, 3000, value_dtype=np.dtype(vdt).type, sort=False, replace=True)
    n_rows, n_dense = len(lens), 72
    rng = np.random.default_rng(5)
    b_wide = rng.uniform(-1, 1, (3000, 100)).astype(vdt)
    bd = dev(b_wide)[:, 10:10 + n_dense]                       # rows 100 elements apart
    assert not bd.is_contiguous()
    with env(FSB_SPMM_PANELS=n_panels):
        prep = fs.prepare_spmm_csr_opt(dev(data), dev(idx), dev(ptr), (n_rows, 3000))
        passes = prep.passes_for(n_dense)
        tile = 128 // np.dtype(vdt).itemsize
        assert len(passes) == n_panels * -(-n_dense // tile) and prep.launches_per_product(n_dense) >= len(passes)
        c = fs.flagsparse_spmm_csr_opt(B=bd, prepared=prep)
        assert_spmm_ok(c.cpu().numpy(), data, idx, ptr, (n_rows, 3000), b_wide[:, 10:10 + n_dense])
        assert np.all(c.cpu().numpy()[np.asarray(lens) == 0] == 0)
        assert torch.equal(fs.flagsparse_spmm_csr_opt(B=bd, prepared=prep), c)     # bit-reproducible
        out_wide = torch.full((n_rows, 96), 7.0, dtype=bd.dtype, device="cuda:0")
        view = out_wide[:, 8:8 + n_dense]
        c2 = fs.flagsparse_spmm_csr_opt(B=bd, prepared=prep, out=view)
        assert torch.equal(view, c) and c2.data_ptr() == view.data_ptr()
        assert torch.all(out_wide[:, :8] == 7.0) and torch.all(out_wide[:, 8 + n_dense:] == 7.0)
        with env(FSB_SPMM_ALGO="plain"):
            assert torch.equal(fs.flagsparse_spmm_csr_opt(B=bd, prepared=prep), c)
        prep.check_status()
    # one-shot entry point and goldens through the split path
    with env(FSB_SPMM_PANELS=n_panels):
        for path in golden_files("spmm"):
            g = load_golden(path)
            if g["data"].dtype != np.dtype(vdt):
                continue
            cg = spmm(g["data"], g["indices"], g["indptr"], g["shape"], g["B"])
            assert_spmm_ok(cg, g["data"], g["indices"], g["indptr"], g["shape"], g["B"], what=path)


@pytest.mark.parametrize("n_dense", [32, 64, 128])
def test_config_c4_full_size(cuda, fsb_lib, n_dense):
    spec = S.config_spec("c4")
    d, i, p = S.generate_csr(spec, "cuda:0")
    b = S.dense_vector(spec, spec.n_cols, "cuda:0", n_dense=n_dense)
    prep = fs.prepare_spmm_csr_opt(d, i, p, (spec.n_rows, spec.n_cols))
    c = fs.flagsparse_spmm_csr_opt(B=b, prepared=prep)
    assert prep.n_panels_for(n_dense) == 1          # one pass by default
    with env(FSB_SPMM_PANEL_MB=64):                 # B gathered panel by panel (64 MiB per pass and column tile)
        assert prep.n_panels_for(n_dense) == 2
        split = fs.flagsparse_spmm_csr_opt(B=b, prepared=prep)
    check_spmm_blocks(spec, split, b.cpu().numpy(), sample_blocks(spec.n_rows, 4, 1024, seed=3))
    worst = check_spmm_blocks(spec, c, b.cpu().numpy(), sample_blocks(spec.n_rows, 12, 1024))
    assert torch.equal(fs.flagsparse_spmm_csr_opt(B=b * 2, prepared=prep), c * 2)  # exact under power-of-two scaling
    with env(FSB_SPMM_ALGO="plain"):
        assert torch.equal(fs.flagsparse_spmm_csr_opt(B=b, prepared=prep), c)
    assert int(prep.status_word().item()) == 0
    print(f"c4 N={n_dense}: worst bound ratio {worst:.2e}")
