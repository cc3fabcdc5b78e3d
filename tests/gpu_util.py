"""Helpers shared by the GPU tests: numpy <-> device, calls through the public API, sampled checks."""

import contextlib
import os

import numpy as np
import torch

import flagsparse_b200 as fs
from flagsparse_b200 import synthetic as S
from helpers import assert_spmm_ok, assert_spmv_ok


def dev(a, device="cuda:0"):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


@contextlib.contextmanager
def env(**kw):
    old = {k: os.environ.get(k) for k in kw}
    try:
        for k, v in kw.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = str(v)
        yield
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


def spmv(data, indices, indptr, shape, x, algo=None, tuning=0, **kw):
    """numpy in, numpy out, through flagsparse_spmv_csr; algo None = the package's own choice."""
    with env(FSB_SPMV_ALGO=algo, FSB_SPMV_TUNING=tuning):
        y = fs.flagsparse_spmv_csr(dev(data), dev(indices), dev(indptr), dev(x), shape, **kw)
    return y.cpu().numpy()


def spmm(data, indices, indptr, shape, b, algo=None, opt=False, **kw):
    with env(FSB_SPMM_ALGO=algo):
        if opt:
            c = fs.flagsparse_spmm_csr_opt(dev(data), dev(indices), dev(indptr), dev(b), shape, **kw)
        else:
            c = fs.flagsparse_spmm_csr(dev(data), dev(indices), dev(indptr), dev(b), shape, **kw)
    return c.cpu().numpy()


def sample_blocks(n_rows, n_blocks, block_rows, seed=0):
    rng = np.random.default_rng(seed)
    starts = sorted(set([0, max(0, n_rows - block_rows)] + rng.integers(0, max(1, n_rows - block_rows), n_blocks).tolist()))
    return [(s, min(n_rows, s + block_rows)) for s in starts]


def check_spmv_blocks(spec, y_dev, x_host, blocks, value_dtype="float32", index_dtype="int32", indptr_dtype="int32"):
    """Regenerate a few row blocks of a synthetic matrix on the host and hold y[rows] to the oracle bound."""
    worst = 0.0
    for r0, r1 in blocks:
        d, i, p = S.generate_csr(spec, None, value_dtype=value_dtype, index_dtype=index_dtype,
                                 indptr_dtype=indptr_dtype, row_range=(r0, r1))
        y = y_dev[r0:r1].cpu().numpy()
        worst = max(worst, assert_spmv_ok(y, d, i, p, (r1 - r0, spec.n_cols), x_host, what=f"{spec.name} rows {r0}:{r1}"))
    return worst


def check_spmm_blocks(spec, c_dev, b_host, blocks):
    worst = 0.0
    for r0, r1 in blocks:
        d, i, p = S.generate_csr(spec, None, row_range=(r0, r1))
        c = c_dev[r0:r1].cpu().numpy()
        worst = max(worst, assert_spmm_ok(c, d, i, p, (r1 - r0, spec.n_cols), b_host, what=f"{spec.name} rows {r0}:{r1}"))
    return worst
