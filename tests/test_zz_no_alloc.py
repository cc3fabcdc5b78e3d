"""fsb_spmv_csr_noalloc: the SpMV entry point for callers that cannot allocate device memory.

Who needs it: code that runs while its framework's memory pool is frozen or capped, plugins that are handed
every buffer by their host and own no allocator, and latency-critical loops that cannot afford cudaMalloc's
device-wide synchronisation.  The entry point keeps its per-tile partial sums in an array built into
libfsb.so instead of caller scratch, so it must give exactly what fsb_spmv_csr gives -- checked here on two
calls in a row (the second call finds the first call's leftovers in the shared array), straight through the
C ABI.  This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""

import numpy as np
import pytest
import torch

from flagsparse_b200 import _lib
from flagsparse_b200 import synthetic as S
from helpers import assert_spmv_ok

pytestmark = pytest.mark.gpu

NOALLOC_MAX_TILES = 262144


def _run_both(L, vtype, d, i, p, x, n_rows, n_cols, tuning=0):
    nnz = d.numel()
    st = torch.cuda.current_stream().cuda_stream
    T = L.fsb_spmv_tile_nnz(vtype, tuning)
    n_tiles = L.fsb_csr_num_tiles(nnz, T)
    plan = torch.empty(n_tiles + 1, dtype=torch.int32, device=d.device)
    assert L.fsb_csr_tile_plan(_lib.FSB_I32, p.data_ptr(), n_rows, nnz, T, plan.data_ptr(), st) == 0
    nbytes = L.fsb_spmv_csr_scratch_bytes(vtype, nnz, tuning)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=d.device)
    y_ref = torch.full((n_rows,), float("nan"), dtype=d.dtype, device=d.device)
    y_new = torch.full((n_rows,), float("nan"), dtype=d.dtype, device=d.device)
    rc = L.fsb_spmv_csr(vtype, _lib.FSB_I32, _lib.FSB_I32, d.data_ptr(), i.data_ptr(), p.data_ptr(), x.data_ptr(),
                        y_ref.data_ptr(), n_rows, n_cols, nnz, _lib.FSB_SPMV_STREAM, tuning, plan.data_ptr(),
                        scratch.data_ptr(), nbytes, st)
    assert rc == 0
    rc = L.fsb_spmv_csr_noalloc(vtype, _lib.FSB_I32, _lib.FSB_I32, d.data_ptr(), i.data_ptr(), p.data_ptr(),
                                x.data_ptr(), y_new.data_ptr(), n_rows, n_cols, nnz, tuning, plan.data_ptr(), st)
    assert rc == 0
    torch.cuda.synchronize()
    return y_ref, y_new, plan


@pytest.mark.parametrize("vdt", ["float32", "float64"])
def test_noalloc_matches_the_scratch_entry_point_twice_in_a_row(cuda, fsb_lib, vdt):
    L = fsb_lib
    vtype = _lib.FSB_F32 if vdt == "float32" else _lib.FSB_F64
    # a skewed matrix: rows cross tile boundaries, so the partial-sum slots are really used
    spec = S.config_spec("c3").scaled(1 << 16)
    d, i, p = S.generate_csr(spec, "cuda:0", value_dtype=vdt)
    host = (d.cpu().numpy(), i.cpu().numpy(), p.cpu().numpy(), (spec.n_rows, spec.n_cols))
    x1 = S.dense_vector(spec, spec.n_cols, "cuda:0", value_dtype=vdt)
    x2 = S.dense_vector(spec.seed + 1, spec.n_cols, "cuda:0", value_dtype=vdt)
    for x in (x1, x2):  # second call: the built-in array still holds the first call's partial sums
        y_ref, y_new, _ = _run_both(L, vtype, d, i, p, x, spec.n_rows, spec.n_cols)
        assert torch.equal(y_ref, y_new)  # same kernels, same order of additions: the same bits
        assert_spmv_ok(y_new.cpu().numpy(), *host, x.cpu().numpy(), what="noalloc")
        del y_ref, y_new
    # another tile size shares the same array
    y_ref, y_new, _ = _run_both(L, vtype, d, i, p, x1, spec.n_rows, spec.n_cols, tuning=(1 << 8))
    assert torch.equal(y_ref, y_new)


def test_noalloc_limits_and_degenerate_inputs(cuda, fsb_lib):
    L = fsb_lib
    st = torch.cuda.current_stream().cuda_stream
    spec = S.config_spec("c1")
    d, i, p = S.generate_csr(spec, "cuda:0")
    x = S.dense_vector(spec, spec.n_cols, "cuda:0")
    y = torch.empty(spec.n_rows, dtype=torch.float32, device="cuda:0")
    plan = torch.zeros(64, dtype=torch.int32, device="cuda:0")
    args = (_lib.FSB_F32, _lib.FSB_I32, _lib.FSB_I32, d.data_ptr(), i.data_ptr(), p.data_ptr(), x.data_ptr(),
            y.data_ptr(), spec.n_rows, spec.n_cols)
    # one tile more than the built-in array holds: refused on the host, nothing is launched
    too_many = (NOALLOC_MAX_TILES * 2048) + 1
    assert L.fsb_spmv_csr_noalloc(*args, too_many, 0, plan.data_ptr(), st) == -5
    assert L.fsb_spmv_csr_noalloc(*args, NOALLOC_MAX_TILES * 1024 + 1, 1 << 8, plan.data_ptr(), st) == -5
    # missing plan, bad dtype tag
    assert L.fsb_spmv_csr_noalloc(*args, d.numel(), 0, None, st) == -1
    assert L.fsb_spmv_csr_noalloc(9, *args[1:], d.numel(), 0, plan.data_ptr(), st) == -1
    # an all-empty matrix needs no plan and gives exact zeros
    zptr = torch.zeros(spec.n_rows + 1, dtype=torch.int32, device="cuda:0")
    y.fill_(5.0)
    assert L.fsb_spmv_csr_noalloc(_lib.FSB_F32, _lib.FSB_I32, _lib.FSB_I32, None, None, zptr.data_ptr(), x.data_ptr(),
                                  y.data_ptr(), spec.n_rows, spec.n_cols, 0, 0, None, st) == 0
    torch.cuda.synchronize()
    assert torch.count_nonzero(y) == 0
