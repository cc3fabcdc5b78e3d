"""SpMV of skewed matrices with the long rows split off to the row-group panel kernel, on the GPU: against the
float64 oracle, against the stream kernel on the same matrix, for both value types, wide indices, rows that need
several accumulators, several groups, unsorted and duplicate columns, and bit-equality of repeated calls."""

import numpy as np
import pytest
import torch

import flagsparse_b200 as fs
from flagsparse_b200 import longrows
from flagsparse_b200 import synthetic as S
from gpu_util import dev, env
from helpers import assert_spmv_ok, handmade_csr

pytestmark = pytest.mark.gpu


@pytest.fixture()
def small_limits(monkeypatch):
    """Let matrices of test size through the checks that keep the split away from small inputs."""
    monkeypatch.setattr(longrows, "MIN_LONG_NNZ", 1 << 12)
    monkeypatch.setattr(longrows, "MIN_UNIT_ENTRIES", 256)


def _prepared(d, i, p, shape, **envkw):
    with env(**envkw):
        return fs.prepare_spmv_csr(dev(d), dev(i), dev(p), shape)


@pytest.mark.parametrize("vdt,idt,pdt", [("float32", "int32", "int32"), ("float64", "int64", "int64")])
def test_power_law_matrix(cuda, fsb_lib, small_limits, vdt, idt, pdt):
    spec = S.config_spec("c3").scaled(1 << 20)
    d, i, p = S.generate_csr(spec, None, value_dtype=vdt, index_dtype=idt, indptr_dtype=pdt)
    x = S.dense_vector(spec, spec.n_cols, value_dtype=vdt)
    shape = (spec.n_rows, spec.n_cols)
    pr = _prepared(d, i, p, shape)
    assert pr.long_rows is not None, "the long rows of a power-law matrix are expected to be split off"
    short, lay = pr.long_rows
    assert short.long_rows is None and short.data.numel() + lay.nnz == d.size
    assert "long-row panel" in pr.opt_buckets[0]["kind"]
    tx = dev(x)
    y = fs.flagsparse_spmv_csr(x=tx, prepared=pr)
    assert int(lay.status.item()) == 0
    assert_spmv_ok(y.cpu().numpy(), d, i, p, shape, x, what="split")
    assert torch.equal(y, fs.flagsparse_spmv_csr(x=tx, prepared=pr))          # same bits on every call
    out = torch.full_like(y, 3.0)
    assert fs.flagsparse_spmv_csr(x=tx, prepared=pr, out=out) is out and torch.equal(out, y)
    # the same matrix without the split
    ref = _prepared(d, i, p, shape, FSB_SPMV_LONG_ROWS=0)
    assert ref.long_rows is None
    y_ref = fs.flagsparse_spmv_csr(x=tx, prepared=ref)
    assert_spmv_ok(y_ref.cpu().numpy(), d, i, p, shape, x, what="stream")
    # rows that stayed in the CSR part come out of the same kernel: identical bits unless the tile cuts moved
    is_short = torch.ones(spec.n_rows, dtype=torch.bool, device=cuda)
    is_short[lay.long_rows.long()] = False
    tol = 1e-4 if vdt == "float32" else 1e-12
    assert torch.allclose(y[is_short], y_ref[is_short], rtol=0, atol=tol)
    # a one-shot call does not pay for the regrouping
    y1 = fs.flagsparse_spmv_csr(dev(d), dev(i), dev(p), tx, shape)
    assert torch.equal(y1, y_ref)


@pytest.mark.parametrize("vdt", ["float32", "float64"])
def test_rows_with_many_entries_per_chunk_and_several_groups(cuda, fsb_lib, small_limits, monkeypatch, vdt):
    cap = 1024 if vdt == "float32" else 512
    monkeypatch.setattr(longrows, "ACC_CAP", cap)
    rng = np.random.default_rng(17)
    n_rows, n_cols = 3000, 70000
    lens = rng.integers(0, 10, n_rows)
    lens[rng.choice(n_rows, 300, replace=False)] = rng.integers(64, 2000, 300)
    lens[[5, 1700, 2999]] = [60000, 25000, 41000]        # thousands of entries per chunk of 8192 columns
    d, i, p = handmade_csr(18, lens.tolist(), n_cols, value_dtype=np.dtype(vdt), indptr_dtype=np.int64)
    x = rng.uniform(-1, 1, n_cols).astype(vdt)
    shape = (n_rows, n_cols)
    pr = _prepared(d, i, p, shape, FSB_SPMV_LONG_ROW=64)
    assert pr.long_rows is not None
    short, lay = pr.long_rows
    assert lay.n_long == int((lens >= 64).sum()) and lay.n_groups > 1 and lay.max_group_acc <= cap
    assert int((lay.vbase[1:] - lay.vbase[:-1]).max()) > 100
    assert int(short.max_row_nnz) < 64
    y = fs.flagsparse_spmv_csr(x=dev(x), prepared=pr)
    assert int(lay.status.item()) == 0
    assert_spmv_ok(y.cpu().numpy(), d, i, p, shape, x, what="groups")
    assert torch.equal(y, fs.flagsparse_spmv_csr(x=dev(x), prepared=pr))
    # automatic choice: only the groups that are dense enough are kept, the result does not change beyond rounding
    pa = _prepared(d, i, p, shape)
    assert pa.long_rows is not None and pa.long_rows[1].n_long <= lay.n_long
    ya = fs.flagsparse_spmv_csr(x=dev(x), prepared=pa)
    assert_spmv_ok(ya.cpu().numpy(), d, i, p, shape, x, what="automatic")


def test_unsorted_and_duplicate_columns_in_long_rows(cuda, fsb_lib, small_limits):
    lens = [3, 0, 5000, 1, 0, 0, 900, 64, 63, 2, 12000, 0]
    d, i, p = handmade_csr(23, lens, 20000, sort=False, replace=True)
    x = np.random.default_rng(24).uniform(-1, 1, 20000).astype(np.float32)
    shape = (len(lens), 20000)
    pr = _prepared(d, i, p, shape, FSB_SPMV_LONG_ROW=64)
    assert pr.long_rows is not None and pr.long_rows[1].n_long == 4
    y = fs.flagsparse_spmv_csr(x=dev(x), prepared=pr)
    assert_spmv_ok(y.cpu().numpy(), d, i, p, shape, x, what="unsorted, duplicates")
    assert y[1].item() == 0.0 and y[4].item() == 0.0 and y[11].item() == 0.0


def test_split_is_not_used_when_it_cannot_pay(cuda, fsb_lib):
    # real limits: a matrix of this size keeps the stream kernel alone
    spec = S.config_spec("c3").scaled(1 << 16)
    d, i, p = S.generate_csr(spec, None)
    pr = _prepared(d, i, p, (spec.n_rows, spec.n_cols))
    assert pr.long_rows is None
    x = S.dense_vector(spec, spec.n_cols)
    y = fs.flagsparse_spmv_csr(x=dev(x), prepared=pr)
    assert_spmv_ok(y.cpu().numpy(), d, i, p, (spec.n_rows, spec.n_cols), x)
