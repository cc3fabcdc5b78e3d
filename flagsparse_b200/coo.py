"""Native COO entry points over the CSR kernels: flagsparse_spmv_coo, prepare_spmv_coo, flagsparse_spmm_coo.

Same names, arguments, defaults, validation and exception types as the reference's
src/flagsparse/sparse_operations/spmv_coo.py (PreparedCoo :20-50, _prepare_coo_tensors :183-222,
prepare_spmv_coo :225-230, _validate_x_coo :233-249, flagsparse_spmv_coo :292-347) and spmm_coo.py
(_prepare_spmm_coo_inputs :312-371, _resolve_spmm_coo_launch_config :374-391, flagsparse_spmm_coo :671-694).

The reference keeps COO storage and runs one Triton program per run of equal rows (`seg_starts`), or one
atomic add per entry when the entries are not sorted.  Here the entries are ordered by row once, at prepare
time, the row runs become a row-pointer array, and the product runs on the same sm_100a kernels as the CSR
entry points: the sum over an output row is the same set of products either way.  The unsorted form gives
the same result on every call (a stable sort by row replaces the atomics).  PreparedCoo keeps the
reference's attributes (sorted data/row/col, seg_starts, n_segs, use_seg_kernel).
"""

import time

import torch

from ._common import SUPPORTED_INDEX_DTYPES, _INDEX_LIMIT_INT32, _check_value_dtype
from .spmm_csr import _alg1_shape, _check_out, _run_spmm, prepare_spmm_csr_opt
from .spmv_csr import _prepare_spmv_csr, _spmv_launch


class PreparedCoo:
    """Sorted COO entries and the bounds of their row runs (reference: spmv_coo.py:20-50), plus the prepared
    row-pointer form the kernels read."""

    __slots__ = ("data", "row", "col", "shape", "n_rows", "n_cols", "nnz", "seg_starts", "n_segs",
                 "use_seg_kernel", "_csr")

    def __init__(self, data, row, col, shape, seg_starts=None, csr=None):
        self.data = data
        self.row = row
        self.col = col
        self.shape = (int(shape[0]), int(shape[1]))
        self.n_rows, self.n_cols = self.shape
        self.nnz = int(data.numel())
        self.seg_starts = seg_starts
        if seg_starts is None:
            self.n_segs = 0
            self.use_seg_kernel = False
        else:
            self.n_segs = int(seg_starts.numel()) - 1
            self.use_seg_kernel = self.n_segs > 0
        self._csr = csr


def _sort_coo_lex(data, row64, col64, n_cols):
    """Entries in (row, col) order (reference: spmv_coo.py:153-165)."""
    if data.numel() == 0:
        return data.contiguous(), row64, col64
    order = torch.argsort(row64 * max(1, int(n_cols)) + col64)
    return data[order].contiguous(), row64[order].contiguous(), col64[order].contiguous()


def _seg_starts_from_sorted_rows(row_sorted, nnz, device):
    """int32[n_runs + 1] bounds of the runs of equal rows (reference: spmv_coo.py:168-180)."""
    if nnz == 0:
        return None
    breaks = torch.nonzero(row_sorted[1:] != row_sorted[:-1], as_tuple=False).flatten().to(torch.int32) + 1
    ends = torch.tensor([nnz], dtype=torch.int32, device=device)
    return torch.cat([torch.zeros(1, dtype=torch.int32, device=device), breaks, ends])


def _check_index_range(row64, col64, n_rows, n_cols):
    if row64.numel() == 0:
        return
    lo = torch.stack([row64.min(), col64.min(), row64.max(), col64.max()]).tolist()  # one host sync
    min_row, min_col, max_row, max_col = (int(v) for v in lo)
    if min_row < 0 or max_row >= n_rows:
        raise IndexError("row indices out of range")
    if min_col < 0 or max_col >= n_cols:
        raise IndexError("col indices out of range")
    if max_row > _INDEX_LIMIT_INT32 or max_col > _INDEX_LIMIT_INT32:
        raise ValueError("indices exceed the int32 range of the kernels")


def _row_pointer(row_sorted64, n_rows):
    indptr = torch.zeros(n_rows + 1, dtype=torch.int64, device=row_sorted64.device)
    if row_sorted64.numel():
        indptr[1:] = torch.cumsum(torch.bincount(row_sorted64, minlength=n_rows), dim=0)
    return indptr


def _prepare_coo_tensors(data, row, col, shape, sort_by_row, reuse_expected):
    if not all(torch.is_tensor(t) for t in (data, row, col)):
        raise TypeError("data, row and col have to be torch.Tensor objects")
    if data.ndim != 1 or row.ndim != 1 or col.ndim != 1:
        raise ValueError("data, row and col have to be one-dimensional")
    if not all(t.is_cuda for t in (data, row, col)):
        raise ValueError("data, row and col have to live on a CUDA device")
    n_rows, n_cols = int(shape[0]), int(shape[1])
    if data.numel() != row.numel() or data.numel() != col.numel():
        raise ValueError(f"{data.numel()} values, {row.numel()} row ids, {col.numel()} column ids: the counts differ")
    if data.dtype not in (torch.float32, torch.float64):
        raise TypeError(f"COO SpMV takes float32 or float64 values, not {data.dtype} (the CSR entry points take more)")
    row64 = row.to(torch.int64)
    col64 = col.to(torch.int64)
    _check_index_range(row64, col64, n_rows, n_cols)
    if sort_by_row:
        data_k, row_k, col_k = _sort_coo_lex(data, row64, col64, n_cols)
        seg = _seg_starts_from_sorted_rows(row_k, data_k.numel(), data_k.device)
        csr_data, csr_row, csr_col = data_k, row_k, col_k
    else:
        # the reference leaves the entries as they are and adds them with atomics; the kernels here need
        # them grouped by row, so a stable sort on the row alone keeps the caller's order inside each row
        data_k, row_k, col_k, seg = data.contiguous(), row64.contiguous(), col64.contiguous(), None
        if data_k.numel() > 1 and not bool((row_k[1:] >= row_k[:-1]).all().item()):
            csr_row, order = torch.sort(row_k, stable=True)
            csr_data, csr_col = data_k[order], col_k[order]
        else:
            csr_data, csr_row, csr_col = data_k, row_k, col_k
    kr = row_k.to(torch.int32)
    kc = col_k.to(torch.int32)
    csr = _prepare_spmv_csr(csr_data, csr_col.to(torch.int32), _row_pointer(csr_row, n_rows), (n_rows, n_cols),
                            256, None, reuse_expected=reuse_expected)
    return data_k, kr, kc, seg, csr


def prepare_spmv_coo(data, row, col, shape, sort_by_row=True):
    """Order the entries once for repeated products (reference: spmv_coo.py:225-230)."""
    d, kr, kc, seg, csr = _prepare_coo_tensors(data, row, col, shape, sort_by_row, reuse_expected=True)
    return PreparedCoo(d, kr, kc, shape, seg_starts=seg, csr=csr)


def _validate_x_coo(x, prepared):
    """x against a prepared COO matrix: same checks, order and exception types as for the CSR entry points (the
    reference's spmv_coo.py:232-249 repeats them)."""
    from .spmv_csr import _validate_spmv_x

    return _validate_spmv_x(x, prepared)


def flagsparse_spmv_coo(data=None, row=None, col=None, x=None, shape=None, out=None, return_time=False,
                        prepared=None, sort_by_row=True, block_size=256, num_warps=4, block_inner=128):
    """COO SpMV: y = A @ x (reference: spmv_coo.py:292-347, same arguments and defaults).

    block_size, num_warps and block_inner shape the reference's Triton launches; here they are validated
    the same way and otherwise unused.  Rows without entries give exact zeros; duplicates are summed.
    """
    if prepared is None:
        if any(a is None for a in (data, row, col, x, shape)):
            raise ValueError("data, row, col, x, shape required when prepared is None")
        d, kr, kc, seg, csr = _prepare_coo_tensors(data, row, col, shape, sort_by_row, reuse_expected=False)
        prepared = PreparedCoo(d, kr, kc, shape, seg_starts=seg, csr=csr)
    else:
        if not isinstance(prepared, PreparedCoo) or prepared._csr is None:
            raise TypeError("prepared must come from prepare_spmv_coo")
        if x is None:
            raise TypeError("x is required when prepared is set")
        if shape is None:
            shape = prepared.shape
        sh = (int(shape[0]), int(shape[1]))
        if sh != prepared.shape:
            raise ValueError(f"shape {sh} does not match prepared.shape {prepared.shape}")
    x = _validate_x_coo(x, prepared)
    if num_warps not in (1, 2, 4, 8, 16, 32):
        raise ValueError("num_warps must be a power of 2 in [1, 32]")
    if block_inner <= 0 or (block_inner & (block_inner - 1)) != 0:
        raise ValueError("block_inner must be a positive power of 2")
    dev, dtype = prepared.data.device, prepared.data.dtype
    if out is not None and (out.shape != (prepared.n_rows,) or out.dtype != dtype):
        raise ValueError("out shape/dtype must match result")
    direct = out is not None and out.is_cuda and out.device == dev and out.is_contiguous()
    y = out if direct else torch.empty(prepared.n_rows, dtype=dtype, device=dev)
    t0 = None
    if return_time:
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
    _spmv_launch(prepared._csr, x, y)
    elapsed_ms = None
    if return_time:
        torch.cuda.synchronize(dev)
        elapsed_ms = (time.perf_counter() - t0) * 1000.0
    if out is not None and not direct:
        out.copy_(y)
        y = out
    if return_time:
        return y, elapsed_ms
    return y


# ---------------------------------------------------------------------------------------------------
# COO SpMM
# ---------------------------------------------------------------------------------------------------
def _prepare_spmm_coo_inputs(data, row, col, B, shape):
    """Argument checks of the reference (spmm_coo.py:312-371), in its order."""
    if len(shape) != 2:
        raise ValueError("shape must be a 2-tuple: (n_rows, n_cols)")
    if data.ndim != 1 or row.ndim != 1 or col.ndim != 1:
        raise ValueError("data, row, and col must be 1D tensors")
    if B.ndim != 2:
        raise ValueError("B must be a 2D dense tensor")
    n_rows, n_cols = int(shape[0]), int(shape[1])
    if n_rows < 0 or n_cols < 0:
        raise ValueError("shape dimensions must be non-negative")
    if data.numel() != row.numel() or data.numel() != col.numel():
        raise ValueError("data, row, and col must have the same length (nnz)")
    if B.shape[0] != n_cols:
        raise ValueError(f"B.shape[0] must be n_cols={n_cols}, got {B.shape[0]}")
    if not all(t.is_cuda for t in (data, row, col, B)):
        raise ValueError("data, row, col, and B must be CUDA tensors")
    if not all(t.device == data.device for t in (row, col, B)):
        raise ValueError("data, row, col, and B must be on the same CUDA device")
    _check_value_dtype(data.dtype)
    if B.dtype != data.dtype:
        raise TypeError("B dtype must match data dtype")
    if row.dtype not in SUPPORTED_INDEX_DTYPES:
        raise TypeError("row dtype must be torch.int32 or torch.int64")
    if col.dtype not in SUPPORTED_INDEX_DTYPES:
        raise TypeError("col dtype must be torch.int32 or torch.int64")
    if data.numel() > _INDEX_LIMIT_INT32:
        raise ValueError("nnz exceeds the int32 range supported by the COO entry point")
    row64 = row.to(torch.int64)
    col64 = col.to(torch.int64)
    if data.numel() > 0:
        lo = torch.stack([row64.min(), col64.min(), row64.max(), col64.max()]).tolist()
        min_row, min_col, max_row, max_col = (int(v) for v in lo)
        if min_row < 0 or max_row >= n_rows:
            raise IndexError("row indices out of range for n_rows")
        if min_col < 0 or max_col >= n_cols:
            raise IndexError("col indices out of range for n_cols")
        if max_row > _INDEX_LIMIT_INT32:
            raise ValueError("row indices exceed the int32 range supported by the kernels")
        if max_col > _INDEX_LIMIT_INT32:
            raise ValueError("column indices exceed the int32 range supported by the kernels")
    return data.contiguous(), row64, col64, n_rows, n_cols, int(B.shape[1])


def _resolve_spmm_coo_launch_config(n_dense_cols, nnz, block_n=None, block_nnz=256):
    """The reference's launch bookkeeping (spmm_coo.py:374-391); validated, not used by the kernels."""
    warp_size, factor = _alg1_shape(n_dense_cols)
    if block_n is None:
        block_n = warp_size * factor
    if block_nnz is None:
        block_nnz = 256
    if block_n <= 0 or block_nnz <= 0:
        raise ValueError("block_n and block_nnz must be positive when provided")
    return {
        "block_n": int(block_n),
        "block_nnz": int(block_nnz),
        "required_nnz_tiles": int(-(-nnz // block_nnz) if nnz > 0 else 0),
        "heuristic_warp_size": int(warp_size),
        "heuristic_factor": int(factor),
    }


def flagsparse_spmm_coo(data, row, col, B, shape, block_n=None, block_nnz=256, out=None, return_time=False):
    """COO SpMM: C = A @ B (reference: spmm_coo.py:671-694, same arguments and defaults).

    The reference merges duplicate (row, col) entries, sorts and runs a kernel per row run, computing
    float32 inputs in float64.  Here the entries are sorted into row-pointer form and the SpMM kernel sums
    duplicates as it goes, in the value dtype.  No device synchronisation unless return_time is set.
    """
    if block_n is not None and block_n <= 0:
        raise ValueError("block_n must be positive when provided")
    if block_nnz is not None and block_nnz <= 0:
        raise ValueError("block_nnz must be positive when provided")
    data, row64, col64, n_rows, n_cols, n_dense_cols = _prepare_spmm_coo_inputs(data, row, col, B, shape)
    _resolve_spmm_coo_launch_config(n_dense_cols, data.numel(), block_n=block_n, block_nnz=block_nnz)
    if out is not None:
        _check_out(out, data.device, (n_rows, n_dense_cols), data.dtype,
                   "out must be on the same CUDA device as the inputs")
    data_s, row_s, col_s = _sort_coo_lex(data, row64, col64, n_cols)
    prepared = prepare_spmm_csr_opt(data_s, col_s.to(torch.int32), _row_pointer(row_s, n_rows), (n_rows, n_cols))
    return _run_spmm(prepared, B.contiguous(), out, return_time)
