"""Seeded generators: numpy / torch twins give the same bits, row ranges are independent, and the
distributions are the ones the benchmark configurations ask for.  CPU only."""

import numpy as np
import pytest
import torch

from flagsparse_b200 import synthetic as S

SMALL = {"c1": 4096, "c2": 1 << 13, "c3": 1 << 15, "c4": 1 << 12, "c5": 1 << 13}


def _spec(name):
    spec = S.config_spec(name)
    return spec if spec.n_rows == SMALL[name] else spec.scaled(SMALL[name])


@pytest.mark.parametrize("name", sorted(SMALL))
def test_numpy_and_torch_twins_agree(name):
    spec = _spec(name)
    a = S.generate_csr(spec, None)
    b = S.generate_csr(spec, "cpu")
    for u, v in zip(a, b):
        assert np.array_equal(u, v.numpy())
    assert a[0].dtype == np.float32 and a[1].dtype == np.int32 and a[2].dtype == np.int32


@pytest.mark.parametrize("name", sorted(SMALL))
def test_row_ranges_are_independent(name):
    spec = _spec(name)
    d, i, p = S.generate_csr(spec, None, value_dtype="float64", index_dtype="int64", indptr_dtype="int64")
    assert d.dtype == np.float64 and i.dtype == np.int64 and p.dtype == np.int64
    n = spec.n_rows
    for r0, r1 in ((0, 17), (n // 3, n // 3 + 301), (n - 5, n)):
        d2, i2, p2 = S.generate_csr(spec, None, value_dtype="float64", index_dtype="int64", indptr_dtype="int64",
                                    row_range=(r0, r1))
        assert np.array_equal(d2, d[p[r0]:p[r1]])
        assert np.array_equal(i2, i[p[r0]:p[r1]])
        assert np.array_equal(p2, p[r0:r1 + 1] - p[r0])
    # small chunks give the same matrix as one big chunk
    d3, i3, p3 = S.generate_csr(spec, None, value_dtype="float64", index_dtype="int64", indptr_dtype="int64",
                                chunk_nnz=5000)
    assert np.array_equal(d3, d) and np.array_equal(i3, i) and np.array_equal(p3, p)


def test_structure_of_each_config():
    d, i, p = S.generate_csr(_spec("c1"), None)
    lens = np.diff(p)
    assert np.all(lens == 16) and i.min() >= 0 and i.max() < 4096
    assert np.all(np.diff(i.reshape(-1, 16), axis=1) > 0)  # sorted, distinct
    assert d.min() >= -1 and d.max() < 1

    spec = _spec("c2")
    d, i, p = S.generate_csr(spec, None)
    lens = np.diff(p)
    assert abs(lens.mean() - 32) < 0.5 and 20 < lens.var() < 45
    rows = np.repeat(np.arange(spec.n_rows), lens)
    w = spec.columns[1]
    lo = np.clip(rows - w, 0, spec.n_cols - (2 * w + 1))
    assert np.all(i >= lo) and np.all(i <= lo + 2 * w)
    same_row = rows[1:] == rows[:-1]
    assert np.all(np.diff(i)[same_row] > 0)  # sorted and deduplicated

    spec = _spec("c3")
    d, i, p = S.generate_csr(spec, None)
    lens = np.diff(p)
    assert lens.min() >= 1 and lens.max() > 50 * lens.mean()  # heavy tail
    assert 0.8 < p[-1] / (spec.lengths[3]) < 1.1

    d, i, p = S.generate_csr(_spec("c4"), None)
    assert np.all(np.diff(p) == 16)
    assert np.all(np.diff(i.reshape(-1, 16), axis=1) >= 0)  # sorted, duplicates allowed

    spec = _spec("c5")
    d, i, p = S.generate_csr(spec, None, indptr_dtype="int64")
    assert p.dtype == np.int64
    assert np.array_equal(np.diff(p), S.row_lengths(spec, S._ops(None), 0, spec.n_rows))  # lengths known up front


def test_seed_changes_the_matrix_and_dense_operands_match():
    a = S.generate_csr(S.config_spec("c1", seed=0), None)
    b = S.generate_csr(S.config_spec("c1", seed=1), None)
    assert not np.array_equal(a[1], b[1]) and not np.array_equal(a[0], b[0])
    x = S.dense_vector(0, 1000)
    assert np.array_equal(x, S.dense_vector(0, 1000, "cpu").numpy())
    assert np.array_equal(S.dense_vector(0, 1000, row_range=(100, 200)), x[100:200])
    B = S.dense_vector(0, 300, n_dense=12)
    assert B.shape == (300, 12) and B.dtype == np.float32
    assert np.array_equal(B, S.dense_vector(0, 300, "cpu", n_dense=12).numpy())
    assert np.array_equal(S.dense_vector(0, 300, n_dense=12, row_range=(7, 90)), B[7:90])
    x64 = S.dense_vector(0, 50, value_dtype="float64")
    assert x64.dtype == np.float64 and np.all(np.abs(x64) <= 1)
    assert isinstance(S.dense_vector(0, 5, "cpu"), torch.Tensor)
