"""Host-logic tests without a GPU: a context in which CPU tensors claim to be CUDA tensors and the CUDA launches of
the package are replaced by host stand-ins (scipy products, a numpy tile plan, torch reductions for the analysis
pass).  Everything above the C ABI -- validation, kernel selection, the regrouped layouts, the COO / wide-dtype /
long-row paths, `out=` and `return_time` handling -- then runs on CPU exactly as it runs on the GPU.  Test
infrastructure only."""

import contextlib
from unittest import mock

import numpy as np
import scipy.sparse as sp
import torch

from flagsparse_b200 import _common, coo, spmm_csr, spmv_csr


def fake_analyze(indices, indptr, n_rows):
    """What fsb_csr_analyze returns (include/fsb.h), with torch reductions."""
    p = indptr.to(torch.int64)
    lens = p[1:] - p[:-1]
    nnz = indices.numel()
    mean_up = (nnz + n_rows - 1) // n_rows if n_rows > 0 else 0
    long_len = max(64, mean_up * 32)
    return _common.CsrStats([
        int(p[0]), int(p[-1]), int((lens < 0).sum()),
        int(indices.min()) if nnz else 2**63 - 1, int(indices.max()) if nnz else -2**63,
        int(lens.max()) if n_rows > 0 else 0, int((lens == 0).sum()), int((lens > long_len).sum()),
    ])


def fake_tile_plan(indptr, n_rows, nnz, tile_nnz):
    """What fsb_csr_tile_plan writes: tile_row[t] = row holding entry t * tile_nnz."""
    n_tiles = (nnz + tile_nnz - 1) // tile_nnz if nnz > 0 else 0
    p = indptr.to(torch.int64).numpy()
    plan = np.zeros(n_tiles + 1, dtype=np.int32)
    if n_tiles > 1:
        plan[1:n_tiles] = np.searchsorted(p, np.arange(1, n_tiles, dtype=np.int64) * tile_nnz, side="right") - 1
    plan[n_tiles] = n_rows
    return torch.from_numpy(plan)


def _matrix(p):
    return sp.csr_matrix((p.data.numpy(), p.kernel_indices.numpy(), p.kernel_indptr.numpy()), shape=(p.n_rows, p.n_cols))


class Launches:
    """Stand-ins for _spmv_launch / _spmm_launch that also record what they were asked to run."""

    def __init__(self):
        self.spmv, self.spmm = [], []

    def spmv_launch(self, prepared, x, y):
        assert prepared.data.dtype in (torch.float32, torch.float64), "the kernels compute float32 / float64 only"
        assert x.dtype == prepared.data.dtype == y.dtype and x.is_contiguous() and y.is_contiguous()
        assert x.numel() == prepared.n_cols and y.numel() == prepared.n_rows
        kind = "panel" if prepared.panel is not None else "long rows" if prepared.long_rows is not None else \
            {1: "vector", 2: "stream"}.get(prepared.algo if prepared.tile_row is not None else 1, "vector")
        self.spmv.append(kind)
        if prepared.n_rows:
            y.copy_(torch.from_numpy(np.asarray(_matrix(prepared) @ x.numpy(), dtype=x.numpy().dtype)))

    def spmv_launch_wide(self, prepared, x, y):
        """Stand-in for fsb_spmv_csr_wide: the matrix as stored, x and y float32 (half precisions) or complex."""
        dt = prepared.data.dtype
        half = dt in (torch.float16, torch.bfloat16)
        assert dt in (torch.float16, torch.bfloat16, torch.complex64, torch.complex128)
        assert x.dtype == y.dtype == (torch.float32 if half else dt) and x.is_contiguous() and y.is_contiguous()
        self.spmv.append("wide")
        vals = prepared.data.to(torch.float32 if half else dt).numpy()
        a = sp.csr_matrix((vals, prepared.kernel_indices.numpy(), prepared.kernel_indptr.numpy()),
                          shape=(prepared.n_rows, prepared.n_cols))
        if prepared.n_rows:
            y.copy_(torch.from_numpy(np.asarray(a @ x.numpy(), dtype=x.numpy().dtype)))

    def spmm_launch_wide(self, prepared, B, C):
        """Stand-in for fsb_spmm_csr_wide."""
        dt = prepared.data.dtype
        half = dt in (torch.float16, torch.bfloat16)
        assert B.dtype == C.dtype == (torch.float32 if half else dt) and B.stride(-1) == 1
        self.spmm.append(("wide", int(B.shape[1])))
        vals = prepared.data.to(torch.float32 if half else dt).numpy()
        a = sp.csr_matrix((vals, prepared.kernel_indices.numpy(), prepared.kernel_indptr.numpy()),
                          shape=(prepared.n_rows, prepared.n_cols))
        if prepared.n_rows and B.shape[1]:
            C.copy_(torch.from_numpy(np.asarray(a @ B.numpy(), dtype=B.numpy().dtype)))

    def spmm_launch(self, prepared, B, C):
        assert prepared.data.dtype in (torch.float32, torch.float64)
        assert B.dtype == prepared.data.dtype == C.dtype and C.shape == (prepared.n_rows, B.shape[1])
        self.spmm.append(int(B.shape[1]))
        if prepared.n_rows and B.shape[1]:
            C.copy_(torch.from_numpy(np.asarray(_matrix(prepared) @ B.numpy(), dtype=B.numpy().dtype)))


@contextlib.contextmanager
def fake_cuda():
    launches = Launches()
    patches = [
        mock.patch.object(torch.Tensor, "is_cuda", new_callable=mock.PropertyMock, return_value=True),
        mock.patch.object(spmv_csr, "_analyze_csr", fake_analyze),
        mock.patch.object(spmm_csr, "_analyze_csr", fake_analyze),
        mock.patch.object(spmv_csr, "_tile_plan", fake_tile_plan),
        mock.patch.object(spmm_csr, "_tile_plan", fake_tile_plan),
        mock.patch.object(spmv_csr, "_spmv_launch", launches.spmv_launch),
        mock.patch.object(spmv_csr, "_spmv_launch_wide", launches.spmv_launch_wide),
        mock.patch.object(coo, "_spmv_launch", launches.spmv_launch),
        mock.patch.object(spmm_csr, "_spmm_launch", launches.spmm_launch),
        mock.patch.object(spmm_csr, "_spmm_launch_wide", launches.spmm_launch_wide),
        mock.patch.object(torch.cuda, "synchronize", lambda *a, **k: None),
    ]
    for p in patches:
        p.start()
    try:
        yield launches
    finally:
        for p in reversed(patches):
            p.stop()
