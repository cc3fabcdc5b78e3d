"""CSR SDDMM host code: out[p] = alpha * dot(x[row(p)], y[col(p)]) + beta * data[p] on a CSR pattern.

Entry points, arguments, defaults, exception types and the order of the checks follow the reference's
src/flagsparse/sparse_operations/sddmm_csr.py (SDDMMPrepared :9-33, prepare_sddmm_csr :93-104, the pattern checks
:46-80, the dense-operand checks :206-228, the `out` checks :231-242, flagsparse_sddmm_csr :350-422).  Below the
boundary one CUDA kernel (csrc/sddmm_csr.cu) does the work; there is no fallback path, so `allow_fallback` is
accepted and reported as unused.
"""

import time

import torch

from . import _lib
from ._common import _VTYPE, _stream_ptr

SUPPORTED_SDDMM_VALUE_DTYPES = (torch.float32, torch.float64)


class SDDMMPrepared:
    """The checked CSR pattern plus the row of every entry (the reference's class of this name, :9-33; block_k and
    num_warps are kept as the bookkeeping they are there)."""

    __slots__ = ("indices", "indptr", "shape", "n_rows", "n_cols", "nnz", "row_ids", "block_k", "num_warps")

    def __init__(self, indices, indptr, shape, row_ids, block_k, num_warps):
        self.indices = indices
        self.indptr = indptr
        self.shape = (int(shape[0]), int(shape[1]))
        self.n_rows, self.n_cols = self.shape
        self.nnz = int(indices.numel())
        self.row_ids = row_ids
        self.block_k = int(block_k)
        self.num_warps = int(num_warps)


def _launch_bookkeeping(k):
    """(block_k, num_warps) the reference would launch its Triton kernel with (:36-43); reported, not used."""
    if k <= 32:
        return 32, 2
    return (64, 4) if k <= 128 else (128, 8)


def _check_pattern(indices, indptr, shape):
    if len(shape) != 2:
        raise ValueError("shape must have two entries: (n_rows, n_cols)")
    if indices.ndim != 1 or indptr.ndim != 1:
        raise ValueError("indices and indptr must be one-dimensional")
    n_rows, n_cols = int(shape[0]), int(shape[1])
    if n_rows < 0 or n_cols < 0:
        raise ValueError("shape must not be negative")
    if indptr.numel() != n_rows + 1:
        raise ValueError(f"indptr needs n_rows + 1 = {n_rows + 1} entries, it has {indptr.numel()}")
    if not (indices.is_cuda and indptr.is_cuda):
        raise ValueError("indices and indptr must live on a CUDA device")
    if indices.dtype != torch.int32:
        raise TypeError("indices must be int32")
    if indptr.dtype not in (torch.int32, torch.int64):
        raise TypeError("indptr must be int32 or int64")
    indptr64 = indptr.to(torch.int64).contiguous()
    indices = indices.contiguous()
    nnz = int(indices.numel())
    # one read-back for all structural facts
    facts = torch.stack([
        indptr64[0], indptr64[-1],
        (indptr64[1:] < indptr64[:-1]).sum() if n_rows > 0 else indptr64.new_zeros(()),
        indices.min().to(torch.int64) if nnz > 0 else indptr64.new_zeros(()),
        indices.max().to(torch.int64) if nnz > 0 else indptr64.new_zeros(()),
    ]).tolist()
    first, last, n_decreasing, lo, hi = (int(v) for v in facts)
    if first != 0:
        raise ValueError("indptr must start at 0")
    if last != nnz:
        raise ValueError(f"indptr must end at nnz = {nnz}")
    if n_decreasing > 0:
        raise ValueError("indptr must not decrease")
    if nnz > 0 and (lo < 0 or hi >= n_cols):
        raise IndexError("a column index lies outside shape[1]")
    return indices, indptr64, (n_rows, n_cols)


def prepare_sddmm_csr(indices, indptr, shape, k_hint=64):
    """Check a CSR pattern once and build the row of every entry (reference: :93-104)."""
    indices, indptr, shape = _check_pattern(indices, indptr, shape)
    n_rows = shape[0]
    if n_rows > 0:
        row_ids = torch.repeat_interleave(torch.arange(n_rows, dtype=torch.int32, device=indptr.device),
                                          indptr[1:] - indptr[:-1])
    else:
        row_ids = torch.empty(0, dtype=torch.int32, device=indptr.device)
    block_k, num_warps = _launch_bookkeeping(int(k_hint))
    return SDDMMPrepared(indices, indptr, shape, row_ids, block_k, num_warps)


def _check_dense(data, prepared, x, y):
    if x.ndim != 2 or y.ndim != 2:
        raise ValueError("x and y must be two-dimensional")
    if not (x.is_cuda and y.is_cuda):
        raise ValueError("x and y must live on a CUDA device")
    if x.device != y.device or x.device != prepared.indices.device:
        raise ValueError("x, y and the pattern must share one CUDA device")
    if x.dtype not in SUPPORTED_SDDMM_VALUE_DTYPES:
        raise TypeError("x must be float32 or float64")
    if y.dtype != x.dtype:
        raise TypeError("y must have the dtype of x")
    if data is not None and data.dtype != x.dtype:
        raise TypeError("data must have the dtype of x and y")
    if x.shape[0] != prepared.n_rows:
        raise ValueError(f"x needs n_rows = {prepared.n_rows} rows, it has {x.shape[0]}")
    if y.shape[0] != prepared.n_cols:
        raise ValueError(f"y needs n_cols = {prepared.n_cols} rows, it has {y.shape[0]}")
    if x.shape[1] != y.shape[1]:
        raise ValueError("x and y must have the same number of columns (K)")
    if data is not None and data.numel() != prepared.nnz:
        raise ValueError("data needs one value per entry of the pattern")
    return int(x.shape[1])


def _resolve_out(prepared, x, out):
    if out is None:
        return torch.empty(prepared.nnz, dtype=x.dtype, device=x.device)
    if out.ndim != 1 or out.numel() != prepared.nnz:
        raise ValueError("out must be one-dimensional with nnz elements")
    if not out.is_cuda or out.device != x.device:
        raise ValueError("out must live on the CUDA device of x")
    if out.dtype != x.dtype:
        raise TypeError("out must have the dtype of x")
    return out


def _unit_rows(t):
    """t as the kernel reads it: unit stride along a row, any stride between rows."""
    if t.shape[1] <= 1 or t.stride(1) == 1:
        if t.shape[0] <= 1 or t.stride(0) >= t.shape[1]:
            return t
    return t.contiguous()


def _sddmm_launch(prepared, x, y, data, alpha, beta, out):
    """Enqueue the product on the current stream; `out` may be a strided-free 1-D tensor only (contiguous)."""
    p = prepared
    dev = x.device
    with torch.cuda.device(dev):
        rc = _lib.lib().fsb_sddmm_csr(
            _VTYPE[x.dtype], p.indices.data_ptr(), p.row_ids.data_ptr(), x.data_ptr(), x.stride(0), y.data_ptr(),
            y.stride(0), None if data is None else data.data_ptr(), out.data_ptr(), p.n_rows, p.n_cols, p.nnz,
            int(x.shape[1]), float(alpha), float(beta), _stream_ptr(dev),
        )
    _lib.check(rc, "fsb_sddmm_csr")


def flagsparse_sddmm_csr(data=None, indices=None, indptr=None, x=None, y=None, shape=None, alpha=1.0, beta=0.0,
                         prepared=None, out=None, return_time=False, return_meta=False, allow_fallback=False):
    """CSR SDDMM: out[p] = alpha * dot(x[row(p)], y[col(p)]) + beta * data[p] (reference: :350-422, same arguments
    and defaults).  Returns `out` (a new tensor unless one was given), followed by the elapsed milliseconds and / or
    a dictionary of launch facts when return_time / return_meta ask for them.  Unlike the reference the call only
    synchronises the device when return_time is set."""
    prepare_ms = 0.0
    if prepared is None:
        if any(v is None for v in (indices, indptr, shape)):
            raise ValueError("indices, indptr and shape are needed when no prepared pattern is given")
        t0 = time.perf_counter()
        k_hint = int(x.shape[1]) if (x is not None and x.ndim == 2) else 64
        prepared = prepare_sddmm_csr(indices, indptr, shape, k_hint=k_hint)
        prepare_ms = (time.perf_counter() - t0) * 1000.0
    elif not isinstance(prepared, SDDMMPrepared):
        raise TypeError("prepared must be an SDDMMPrepared")
    if x is None or y is None:
        raise ValueError("x and y are needed")
    if data is None and float(beta) != 0.0:
        raise ValueError("beta is non-zero, so data is needed")
    k_dim = _check_dense(data, prepared, x, y)
    block_k, num_warps = _launch_bookkeeping(k_dim) if k_dim > 0 else (prepared.block_k, prepared.num_warps)
    meta = {"prepare_ms": prepare_ms, "block_k": block_k, "num_warps": num_warps, "fallback_used": False,
            "variant": "baseline", "acc_dtype": str(x.dtype).replace("torch.", ""),
            "out_dtype": str(x.dtype).replace("torch.", "")}
    result = _resolve_out(prepared, x, out)
    elapsed_ms = 0.0
    if k_dim == 0 or prepared.nnz == 0:
        if prepared.nnz > 0:
            if beta == 0.0 or data is None:
                result.zero_()
            else:
                result.copy_(data * beta)
    else:
        target = result if result.is_contiguous() else torch.empty_like(result, memory_format=torch.contiguous_format)
        if return_time:
            torch.cuda.synchronize(x.device)
            t0 = time.perf_counter()
        _sddmm_launch(prepared, _unit_rows(x), _unit_rows(y), None if data is None else data.contiguous(), alpha,
                      beta, target)
        if return_time:
            torch.cuda.synchronize(x.device)
            elapsed_ms = (time.perf_counter() - t0) * 1000.0
        if target is not result:
            result.copy_(target)
    if return_time and return_meta:
        return result, elapsed_ms, meta
    if return_time:
        return result, elapsed_ms
    if return_meta:
        return result, meta
    return result
