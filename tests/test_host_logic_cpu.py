"""The host code above the C ABI, run on CPU tensors with the CUDA launches replaced by host stand-ins
(tests/fake_device.py): which kernel a matrix is sent to, the regrouped layouts being built (or not), one-shot
against prepared calls, `out=` / `return_time`, the COO and wide-dtype paths, the Matrix Market batch harness."""

import numpy as np
import pytest
import torch

import flagsparse_b200 as fs
from fake_device import fake_cuda
from flagsparse_b200 import longrows, panel
from flagsparse_b200 import synthetic as S
from helpers import assert_spmm_ok, assert_spmv_ok, handmade_csr

T = torch.from_numpy


def test_analysis_stand_in_matches_the_tile_model(fsb_lib):
    """The stand-ins are held to the same definitions the CUDA kernels are tested against on the GPU."""
    from fake_device import fake_analyze, fake_tile_plan
    from helpers import tile_plan_model

    d, i, p = handmade_csr(2, [0, 5, 0, 300, 1, 0, 64, 7, 0], 512)
    s = fake_analyze(T(i), T(p), 9)
    assert (s.ptr_first, s.ptr_last, s.n_decreasing, s.max_row_nnz, s.n_empty_rows) == (0, 377, 0, 300, 4)
    assert (s.min_index, s.max_index) == (int(i.min()), int(i.max()))
    for tile in (32, 64, 256):
        assert np.array_equal(fake_tile_plan(T(p), 9, 377, tile).numpy(), tile_plan_model(p, tile))


def test_kernel_selection_and_layouts(fsb_lib, monkeypatch):
    with fake_cuda() as launches:
        # small uniform matrix: vector kernel, nothing regrouped
        c1 = S.config_spec("c1")
        d, i, p = S.generate_csr(c1, None)
        x = S.dense_vector(c1, c1.n_cols)
        prep = fs.prepare_spmv_csr(T(d), T(i), T(p), (c1.n_rows, c1.n_cols))
        assert prep.opt_buckets[0]["kind"] == "vector" and prep.panel is None and prep.long_rows is None
        y = fs.flagsparse_spmv_csr(x=T(x), prepared=prep)
        assert_spmv_ok(y.numpy(), d, i, p, (c1.n_rows, c1.n_cols), x)
        # banded matrix above the size limit: panel layout for a prepared matrix, not for a one-shot call
        c2 = S.config_spec("c2").scaled(1 << 18)
        d, i, p = S.generate_csr(c2, None)
        x = S.dense_vector(c2, c2.n_cols)
        shape = (c2.n_rows, c2.n_cols)
        prep = fs.prepare_spmv_csr(T(d), T(i), T(p), shape)
        assert prep.opt_buckets[0]["kind"] == "panel" and prep.panel.x_overhead <= panel.MAX_X_OVERHEAD
        assert prep.panel.n_buffers == 2 and prep.panel.slot_overhead <= panel.MAX_SLOT_OVERHEAD
        launches.spmv.clear()
        y = fs.flagsparse_spmv_csr(x=T(x), prepared=prep)
        assert launches.spmv == ["panel"]
        assert_spmv_ok(y.numpy(), d, i, p, shape, x)
        launches.spmv.clear()
        y1 = fs.flagsparse_spmv_csr(T(d), T(i), T(p), T(x), shape)
        assert launches.spmv == ["vector"] and torch.equal(y1, y)
        monkeypatch.setenv("FSB_SPMV_ALGO", "stream")
        assert fs.prepare_spmv_csr(T(d), T(i), T(p), shape).opt_buckets[0]["kind"] == "stream"
        monkeypatch.delenv("FSB_SPMV_ALGO")
        # columns all over the matrix: the regrouping is refused, the vector kernel stays
        c4 = S.config_spec("c4").scaled(1 << 19)
        d, i, p = S.generate_csr(c4, None)
        prep = fs.prepare_spmv_csr(T(d), T(i), T(p), (c4.n_rows, c4.n_cols))
        assert d.size >= panel.MIN_NNZ and prep.opt_buckets[0]["kind"] == "vector" and prep.panel is None


def test_long_rows_are_split_off_for_prepared_skewed_matrices(fsb_lib, monkeypatch):
    monkeypatch.setattr(longrows, "MIN_LONG_NNZ", 1 << 12)
    monkeypatch.setattr(longrows, "MIN_UNIT_ENTRIES", 256)
    c3 = S.config_spec("c3").scaled(1 << 18)
    d, i, p = S.generate_csr(c3, None)
    x = S.dense_vector(c3, c3.n_cols)
    shape = (c3.n_rows, c3.n_cols)
    with fake_cuda() as launches:
        prep = fs.prepare_spmv_csr(T(d), T(i), T(p), shape)
        assert prep.long_rows is not None and "long-row panel" in prep.opt_buckets[0]["kind"]
        short, lay = prep.long_rows
        assert short.data.numel() + lay.nnz == d.size and short.long_rows is None
        lens = np.diff(p)
        taken = np.zeros(c3.n_rows, dtype=bool)
        taken[lay.long_rows.numpy()] = True
        assert lens[taken].min() >= lens[~taken].max()           # the longest rows, and all of them down to a cut
        assert int(short.max_row_nnz) == int(lens[~taken].max())
        y = fs.flagsparse_spmv_csr(x=T(x), prepared=prep)
        assert launches.spmv == ["long rows"]
        assert_spmv_ok(y.numpy(), d, i, p, shape, x)
        # one-shot calls and FSB_SPMV_LONG_ROWS=0 keep the single stream kernel
        launches.spmv.clear()
        fs.flagsparse_spmv_csr(T(d), T(i), T(p), T(x), shape)
        assert launches.spmv == ["stream"]
        monkeypatch.setenv("FSB_SPMV_LONG_ROWS", "0")
        assert fs.prepare_spmv_csr(T(d), T(i), T(p), shape).long_rows is None


def test_out_and_return_time_semantics(fsb_lib):
    d, i, p = handmade_csr(4, [3, 0, 9, 1], 16)
    x = np.random.default_rng(5).uniform(-1, 1, 16).astype(np.float32)
    B = np.random.default_rng(6).uniform(-1, 1, (16, 3)).astype(np.float32)
    with fake_cuda():
        y = fs.flagsparse_spmv_csr(T(d), T(i), T(p), T(x), (4, 16))
        out = torch.full((4,), 9.0)
        got, ms = fs.flagsparse_spmv_csr(T(d), T(i), T(p), T(x), (4, 16), out=out, return_time=True)
        assert got is out and torch.equal(out, y) and ms >= 0 and y[1] == 0
        strided = torch.zeros(8)[::2]
        assert fs.flagsparse_spmv_csr(T(d), T(i), T(p), T(x), (4, 16), out=strided) is strided
        assert torch.equal(strided, y)
        with pytest.raises(ValueError):
            fs.flagsparse_spmv_csr(T(d), T(i), T(p), T(x), (4, 16), out=torch.zeros(5))
        C = fs.flagsparse_spmm_csr(T(d), T(i), T(p), T(B), (4, 16))
        assert_spmm_ok(C.numpy(), d, i, p, (4, 16), B)
        outC = torch.empty(4, 3)
        gotC, ms = fs.flagsparse_spmm_csr(T(d), T(i), T(p), T(B), (4, 16), out=outC, return_time=True)
        assert gotC is outC and torch.equal(outC, C)
        prep = fs.prepare_spmm_csr_opt(T(d), T(i), T(p), (4, 16))
        assert torch.equal(fs.flagsparse_spmm_csr_opt(B=T(B), prepared=prep), C)
        with pytest.raises(ValueError):
            fs.flagsparse_spmm_csr_opt(B=T(B), prepared=prep, shape=(5, 16))
        with pytest.raises(TypeError):
            fs.flagsparse_spmm_csr_opt(B=T(B), prepared=object())


def test_coo_and_wide_dtype_paths(fsb_lib):
    rng = np.random.default_rng(8)
    row, col = rng.integers(0, 30, 400), rng.integers(0, 20, 400)
    val = rng.uniform(-1, 1, 400).astype(np.float32)
    x = rng.uniform(-1, 1, 20).astype(np.float32)
    order = np.lexsort((col, row))
    indptr = np.zeros(31, dtype=np.int64)
    indptr[1:] = np.cumsum(np.bincount(row, minlength=30))
    with fake_cuda() as launches:
        for sort_by_row in (True, False):
            y = fs.flagsparse_spmv_coo(T(val), T(row), T(col), T(x), (30, 20), sort_by_row=sort_by_row)
            assert_spmv_ok(y.numpy(), val[order], col[order], indptr, (30, 20), x)
        p = fs.prepare_spmv_coo(T(val), T(row), T(col), (30, 20))
        assert p.use_seg_kernel and p.n_segs == np.unique(row).size
        assert torch.allclose(fs.flagsparse_spmv_coo(x=T(x), prepared=p), y, rtol=0, atol=1e-5)
        # complex values: one launch of the kernel that reads them as stored
        launches.spmv.clear()
        cval = torch.from_numpy(val[order] + 1j * rng.uniform(-1, 1, 400)).to(torch.complex64)
        cx = torch.from_numpy(x + 1j * rng.uniform(-1, 1, 20)).to(torch.complex64)
        cy = fs.flagsparse_spmv_csr(cval, T(col[order]), T(indptr), cx, (30, 20))
        assert launches.spmv == ["wide"] and cy.dtype == torch.complex64
        import scipy.sparse as sp

        ref = sp.csr_matrix((cval.numpy(), col[order], indptr), shape=(30, 20)) @ cx.numpy()
        assert np.allclose(cy.numpy(), ref, rtol=0, atol=1e-4)
        # half precision: one launch on the 2-byte values, x widened and y rounded once
        launches.spmv.clear()
        hy = fs.flagsparse_spmv_csr(T(val[order]).half(), T(col[order]), T(indptr), T(x).half(), (30, 20))
        assert launches.spmv == ["wide"] and hy.dtype == torch.float16


def test_mtx_batch_through_the_real_prepare(fsb_lib):
    import glob
    import os

    from flagsparse_b200 import mtx_bench as MB
    from helpers import GOLDEN

    files = sorted(glob.glob(os.path.join(GOLDEN, "mtx", "*.mtx")))
    with fake_cuda():
        for vdt, idt in ((torch.float32, torch.int32), (torch.float64, torch.int64)):
            results = MB.run_mtx_batch(files, value_dtype=vdt, index_dtype=idt, warmup=1, iters=2, device="cpu")
            assert [r["status"] for r in results] == ["PASS"] * len(files), results
            assert all(r["kernel"] == "vector" for r in results)
