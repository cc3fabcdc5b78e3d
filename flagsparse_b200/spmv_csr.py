"""CSR SpMV host code: the reference's entry points over hand-written sm_100a kernels.

Same names, arguments, defaults, validation order and exception types as the reference's
src/flagsparse/sparse_operations/spmv_csr.py (PreparedCsrSpmv :9-58, _prepare_spmv_csr_matrix :379-436,
_validate_spmv_x :439-452, prepare_spmv_csr :455-495, flagsparse_spmv_csr :557-610, the COO front-end
:613-758).  What differs is below the boundary: one fused analysis pass instead of six reductions, an
nnz-tile plan instead of row-length buckets, and CUDA kernels (libfsb.so) instead of Triton launches.
"""

import os
import time

import torch

from . import _lib, widetypes
from ._common import (
    SUPPORTED_INDEX_DTYPES,
    _INDEX_LIMIT_INT32,
    _ITYPE,
    _VTYPE,
    _analyze_csr,
    _check_value_dtype,
    _ptr,
    _stream_ptr,
    _tile_plan,
)

# matrices below this many nnz are a handful of tiles: the single-launch vector kernel wins on latency
_STREAM_MIN_NNZ = 1 << 18
# the vector kernel gives a row to at most 32 lanes, so it is kept away from very long rows
_VECTOR_MAX_ROW_NNZ = 4096
# "uniform" rows: the longest row is within this factor (plus a small allowance) of the mean row length
_UNIFORM_ROW_FACTOR = 8
_UNIFORM_ROW_SLACK = 64
# regroup banded matrices for the panel kernel (costs a second copy of the entries); FSB_SPMV_PANEL=0 turns it off
_PANEL_ENABLED = os.environ.get("FSB_SPMV_PANEL", "1") != "0"


def _long_rows_enabled():
    """Split the long rows of skewed matrices off to the row-group panel kernel; FSB_SPMV_LONG_ROWS=0 turns it off."""
    return os.environ.get("FSB_SPMV_LONG_ROWS", "1") != "0"


_ALGO_NAMES = {"auto": _lib.FSB_SPMV_AUTO, "vector": _lib.FSB_SPMV_VECTOR, "stream": _lib.FSB_SPMV_STREAM,
               "panel": _lib.FSB_SPMV_PANEL}


def _resolve_block_nnz(max_row_nnz, block_nnz, max_segments):
    """block_nnz / max_segments bookkeeping of the reference (spmv_csr.py:465-475).  The CUDA kernels do
    not use either number; they are kept as attributes of the prepared object."""
    block_nnz_use = block_nnz
    if max_segments is None:
        max_segments_use = max((max_row_nnz + block_nnz_use - 1) // block_nnz_use, 1)
        while max_segments_use > 2048 and block_nnz_use < 65536:
            block_nnz_use *= 2
            max_segments_use = max((max_row_nnz + block_nnz_use - 1) // block_nnz_use, 1)
    else:
        max_segments_use = max_segments
    return block_nnz_use, max_segments_use


def _select_spmv_algo(n_rows, nnz, max_row_nnz):
    """Kernel choice from indptr statistics.  Rows of about equal length (longest row within a small
    factor of the mean) go to the lanes-per-row vector kernel, which needs one launch, no scratch, and leaves
    the whole L1 to the gathers of x; skewed row lengths go to the nnz-tiled stream kernel, whose work per
    CTA does not depend on the row structure.  Small matrices take the vector kernel unless a row is long."""
    forced = os.environ.get("FSB_SPMV_ALGO", "").strip().lower()
    if forced in ("vector", "stream", "panel"):
        return _ALGO_NAMES[forced]
    if max_row_nnz > _VECTOR_MAX_ROW_NNZ:
        return _lib.FSB_SPMV_STREAM
    if nnz < _STREAM_MIN_NNZ:
        return _lib.FSB_SPMV_VECTOR
    mean = nnz / max(n_rows, 1)
    if max_row_nnz <= _UNIFORM_ROW_FACTOR * mean + _UNIFORM_ROW_SLACK:
        return _lib.FSB_SPMV_VECTOR
    return _lib.FSB_SPMV_STREAM


class PreparedCsrSpmv:
    """Cached CSR metadata for repeated SpMV calls on the same sparse matrix.

    Carries the attributes of the reference's class (spmv_csr.py:9-58) plus the tile plan and scratch of
    the stream kernel.  `opt_buckets` describes the plan (the reference lists row ids per length bucket
    there).  One prepared object owns one scratch buffer: calls that share it must not overlap on the GPU.
    """

    __slots__ = (
        "data", "kernel_indices", "kernel_indptr", "shape", "n_rows", "n_cols", "block_nnz",
        "max_segments", "max_row_nnz", "opt_buckets", "supports_opt", "stats", "algo", "tuning",
        "tile_nnz", "tile_row", "scratch", "panel", "long_rows", "wide",
    )

    def __init__(self, data, kernel_indices, kernel_indptr, shape, n_rows, n_cols, block_nnz,
                 max_segments, max_row_nnz, stats, algo, tuning, tile_nnz, tile_row, scratch, panel=None,
                 long_rows=None, wide=None):
        self.data = data
        self.kernel_indices = kernel_indices
        self.kernel_indptr = kernel_indptr
        self.shape = (int(shape[0]), int(shape[1]))
        self.n_rows = n_rows
        self.n_cols = n_cols
        self.block_nnz = block_nnz
        self.max_segments = max_segments
        self.max_row_nnz = max_row_nnz
        self.supports_opt = data.dtype in (torch.float32, torch.float64)
        self.stats = stats
        self.algo = algo
        self.tuning = tuning
        self.tile_nnz = tile_nnz
        self.tile_row = tile_row
        self.scratch = scratch
        self.panel = panel
        self.long_rows = long_rows   # (prepared short-row part, LongRowLayout) when the long rows were split off
        # float16 / bfloat16 / complex values: ("native", []) -- the product goes through fsb_spmv_csr_wide
        self.wide = wide
        n_tiles = 0 if tile_row is None else tile_row.numel() - 1
        kind = {_lib.FSB_SPMV_STREAM: "stream", _lib.FSB_SPMV_PANEL: "panel"}.get(algo, "vector")
        if long_rows is not None:
            kind = "long-row panel + " + long_rows[0].opt_buckets[0]["kind"]
        self.opt_buckets = [{"kind": kind, "tile_nnz": tile_nnz, "n_tiles": n_tiles, "n_rows": n_rows}]

    def _status_words(self):
        if self.panel is not None:
            yield self.panel.status
        if self.long_rows is not None:
            yield self.long_rows[1].status
            yield from self.long_rows[0]._status_words()
        if self.wide is not None:
            for part in self.wide[1]:
                yield from part._status_words()

    def check_status(self):
        """Wait for the last product on this matrix and raise RuntimeError if one of its kernels gave up on a
        bounded device-side wait (its rows of y are then incomplete).  Every product also looks, without waiting,
        at how the previous one ended."""
        for word in self._status_words():
            word.check()


def _prepare_spmv_csr_matrix(data, indices, indptr, shape):
    """Validate and normalise the CSR arrays; same checks, order and exception types as the reference's
    function of this name (spmv_csr.py:379-436).  Returns (data, kernel_indices, kernel_indptr, n_rows,
    n_cols, stats)."""
    if not all(torch.is_tensor(t) for t in (data, indices, indptr)):
        raise TypeError("data, indices and indptr have to be torch.Tensor objects")
    if data.ndim != 1 or indices.ndim != 1 or indptr.ndim != 1:
        raise ValueError("data, indices and indptr have to be one-dimensional")
    n_rows, n_cols = int(shape[0]), int(shape[1])
    if indptr.numel() != n_rows + 1:
        raise ValueError(f"indptr has {indptr.numel()} entries, {n_rows} rows need {n_rows + 1}")
    if data.numel() != indices.numel():
        raise ValueError(f"{data.numel()} values but {indices.numel()} column indices")
    if not all(t.is_cuda for t in (data, indices, indptr)):
        raise ValueError("data, indices and indptr have to live on a CUDA device")
    _check_value_dtype(data.dtype)
    if indices.dtype not in SUPPORTED_INDEX_DTYPES:
        raise TypeError(f"indices are {indices.dtype}; int32 or int64 is needed")

    data = data.contiguous()
    indices = indices.contiguous()
    indptr = indptr.contiguous()
    if indptr.dtype not in SUPPORTED_INDEX_DTYPES:
        # the reference accepts any integer indptr and converts it (:423-425)
        indptr = indptr.to(torch.int64)

    nnz = data.numel()
    stats = _analyze_csr(indices, indptr, n_rows)
    if stats.ptr_first != 0:
        raise ValueError("indptr[0] is not 0")
    if stats.ptr_last != nnz:
        raise ValueError(f"indptr[-1] is {stats.ptr_last}, the arrays hold {nnz} entries")
    if stats.n_decreasing > 0:
        raise ValueError("indptr decreases somewhere")
    if nnz > 0:
        if stats.min_index < 0 or stats.max_index >= n_cols:
            raise IndexError(f"column indices span [{stats.min_index}, {stats.max_index}], the matrix has {n_cols} columns")
        if stats.max_index > _INDEX_LIMIT_INT32:
            raise ValueError(f"int64 column index {stats.max_index} exceeds the int32 kernel range")
    # same narrowing as the reference (:422-425): 32-bit column indices always, 32-bit indptr when it fits
    kernel_indices = indices.to(torch.int32) if indices.dtype == torch.int64 else indices
    kernel_indptr = indptr.to(torch.int32) if nnz <= _INDEX_LIMIT_INT32 else indptr.to(torch.int64)
    return data, kernel_indices, kernel_indptr, n_rows, n_cols, stats


def _validate_spmv_x(x, prepared):
    """x against a prepared matrix: the checks of the reference's _validate_spmv_x (spmv_csr.py:439-452) in its
    order, each with the exception type it raises there.  Returns x, contiguous."""
    if not torch.is_tensor(x):            # None included
        raise TypeError("x has to be a torch.Tensor")
    a = prepared.data
    for failed, exc, why in (
        (x.ndim != 1, ValueError, "x has to be one-dimensional"),
        (not x.is_cuda, ValueError, "x has to live on a CUDA device"),
        (x.dtype != a.dtype, TypeError, f"x is {x.dtype}, the matrix holds {a.dtype}"),
        (x.numel() != prepared.n_cols, ValueError, f"x has {x.numel()} elements, the matrix {prepared.n_cols} columns"),
        (x.device != a.device, ValueError, f"x is on {x.device}, the matrix on {a.device}"),
    ):
        if failed:
            raise exc(why)
    return x.contiguous()


def prepare_spmv_csr(data, indices, indptr, shape, block_nnz=256, max_segments=None):
    """Analyse a CSR matrix once for repeated SpMV calls (reference: spmv_csr.py:455-495)."""
    return _prepare_spmv_csr(data, indices, indptr, shape, block_nnz, max_segments, reuse_expected=True)


def _split_long_rows(data, kernel_indices, kernel_indptr, n_rows, n_cols, shape, block_nnz, max_segments):
    """(prepared short-row part, LongRowLayout) for a skewed matrix whose long rows hold a large share of the
    entries, else None."""
    from . import longrows

    nnz = data.numel()
    threshold = longrows.long_row_threshold()
    lens, candidates, cand_nnz = longrows.split_rows(kernel_indptr, n_rows, threshold or longrows.MIN_CANDIDATE_LEN)
    enough = lambda k: k >= longrows.MIN_LONG_NNZ and k >= longrows.MIN_LONG_SHARE * nnz  # noqa: E731
    if not enough(cand_nnz) or cand_nnz > longrows.MAX_CANDIDATE_NNZ:
        return None
    built = longrows.build_long_row_layout(data, kernel_indices, kernel_indptr, lens, candidates, n_cols,
                                           min_unit_entries=0 if threshold else longrows.MIN_UNIT_ENTRIES)
    if built is None or not enough(built[0].nnz):
        return None
    layout, is_long = built
    d_s, i_s, p_s = longrows.short_part(data, kernel_indices, kernel_indptr, lens, is_long)
    short = _prepare_spmv_csr(d_s, i_s, p_s, shape, block_nnz, max_segments, reuse_expected=True, allow_split=False)
    return short, layout


def _prepare_spmv_csr(data, indices, indptr, shape, block_nnz, max_segments, reuse_expected, allow_split=True):
    """reuse_expected=False (a one-shot product) skips the panel regrouping, which costs about as much as a
    hundred products and only pays when the prepared matrix is used again."""
    data, kernel_indices, kernel_indptr, n_rows, n_cols, stats = _prepare_spmv_csr_matrix(
        data, indices, indptr, shape
    )
    max_row_nnz = stats.max_row_nnz
    block_nnz_use, max_segments_use = _resolve_block_nnz(max_row_nnz, block_nnz, max_segments)
    nnz = data.numel()
    if data.dtype in widetypes.WIDE_DTYPES:
        # float16 / bfloat16 / complex values are read as they are stored by a kernel of their own (fsb_spmv_csr_wide):
        # nothing to plan, no second copy of the matrix
        return PreparedCsrSpmv(
            data=data, kernel_indices=kernel_indices, kernel_indptr=kernel_indptr, shape=shape, n_rows=n_rows,
            n_cols=n_cols, block_nnz=block_nnz_use, max_segments=max_segments_use, max_row_nnz=max_row_nnz,
            stats=stats, algo=_lib.FSB_SPMV_VECTOR, tuning=0, tile_nnz=0, tile_row=None, scratch=None,
            wide=("native", []),
        )
    algo = _select_spmv_algo(n_rows, nnz, max_row_nnz)
    tuning = int(os.environ.get("FSB_SPMV_TUNING", "0"))
    tile_nnz, tile_row, scratch, panel_layout = 0, None, None, None
    # rows of about equal length whose columns stay within a few chunks: regroup once, keep x in shared memory
    want_panel = algo == _lib.FSB_SPMV_PANEL or (
        reuse_expected and algo == _lib.FSB_SPMV_VECTOR and os.environ.get("FSB_SPMV_ALGO", "") == ""
        and _PANEL_ENABLED)
    if want_panel:
        from . import panel

        panel_layout = panel.build_panel_layout(data, kernel_indices, kernel_indptr, n_rows, n_cols, max_row_nnz,
                                                force=algo == _lib.FSB_SPMV_PANEL)
        algo = _lib.FSB_SPMV_PANEL if panel_layout is not None else _lib.FSB_SPMV_VECTOR
    if algo == _lib.FSB_SPMV_STREAM and nnz > 0 and n_rows > 0:
        L = _lib.lib()
        vt = _VTYPE[data.dtype]
        tile_nnz = int(L.fsb_spmv_tile_nnz(vt, tuning))
        tile_row = _tile_plan(kernel_indptr, n_rows, nnz, tile_nnz)
        scratch = torch.empty(int(L.fsb_spmv_csr_scratch_bytes(vt, nnz, tuning)), dtype=torch.uint8,
                              device=data.device)
    # skewed rows: the long ones leave for the row-group panel kernel, the CSR kernels keep the short ones
    long_rows = None
    if (algo == _lib.FSB_SPMV_STREAM and allow_split and reuse_expected and _long_rows_enabled()
            and os.environ.get("FSB_SPMV_ALGO", "") == ""):
        long_rows = _split_long_rows(data, kernel_indices, kernel_indptr, n_rows, n_cols, shape, block_nnz,
                                     max_segments)
    return PreparedCsrSpmv(
        data=data, kernel_indices=kernel_indices, kernel_indptr=kernel_indptr, shape=shape, n_rows=n_rows,
        n_cols=n_cols, block_nnz=block_nnz_use, max_segments=max_segments_use, max_row_nnz=max_row_nnz,
        stats=stats, algo=algo, tuning=tuning, tile_nnz=tile_nnz, tile_row=tile_row, scratch=scratch,
        panel=panel_layout, long_rows=long_rows,
    )


def _spmv_launch(prepared, x, y):
    """Enqueue y = A x on the current stream of the matrix's device.  Stands in for both of the
    reference's launch helpers (_triton_spmv_csr_impl_opt_prepared :329-376 and
    _triton_spmv_csr_impl_prepared :510-554): float32 and float64 accumulate natively either way."""
    L = _lib.lib()
    p = prepared
    dev = p.data.device
    if p.algo == _lib.FSB_SPMV_PANEL and p.panel is not None:
        from . import panel

        with torch.cuda.device(dev):
            panel.launch_panel(p.panel, x, y, p.n_rows, p.n_cols, _stream_ptr(dev))
        return
    if p.long_rows is not None:
        from . import longrows

        short, layout = p.long_rows
        _spmv_launch(short, x, y)      # every row of y; the long rows get zeros here
        with torch.cuda.device(dev):
            longrows.launch_long_rows(layout, x, y, p.n_cols, _stream_ptr(dev))
        return
    algo = p.algo if p.tile_row is not None else _lib.FSB_SPMV_VECTOR
    lanes = p.tuning & 0xFF
    tuning = p.tuning if algo == _lib.FSB_SPMV_STREAM else (lanes if lanes in (2, 4, 8, 16, 32) else 0)
    with torch.cuda.device(dev):
        rc = L.fsb_spmv_csr(
            _VTYPE[p.data.dtype], _ITYPE[p.kernel_indices.dtype], _ITYPE[p.kernel_indptr.dtype],
            _ptr(p.data), _ptr(p.kernel_indices), p.kernel_indptr.data_ptr(), _ptr(x), _ptr(y),
            p.n_rows, p.n_cols, p.data.numel(), algo, tuning,
            None if p.tile_row is None else p.tile_row.data_ptr(),
            None if p.scratch is None else p.scratch.data_ptr(),
            0 if p.scratch is None else p.scratch.numel(), _stream_ptr(dev),
        )
    _lib.check(rc, "fsb_spmv_csr")


_WIDE_VTYPE = {torch.float16: _lib.FSB_F16, torch.bfloat16: _lib.FSB_BF16, torch.complex64: _lib.FSB_C64,
               torch.complex128: _lib.FSB_C128}


def _spmv_launch_wide(prepared, x, y):
    """Enqueue y = A x for float16 / bfloat16 / complex values (fsb_spmv_csr_wide): x and y are float32 for the
    half precisions and of the matrix's own type for complex values.  Stands in for the reference's base launch
    helper on these types (_triton_spmv_csr_impl_prepared, :510-554)."""
    p = prepared
    dev = p.data.device
    if p.n_rows == 0:
        return
    with torch.cuda.device(dev):
        rc = _lib.lib().fsb_spmv_csr_wide(
            _WIDE_VTYPE[p.data.dtype], _ITYPE[p.kernel_indptr.dtype], _ptr(p.data), _ptr(p.kernel_indices),
            p.kernel_indptr.data_ptr(), _ptr(x), _ptr(y), p.n_rows, p.n_cols, p.data.numel(), _stream_ptr(dev),
        )
    _lib.check(rc, "fsb_spmv_csr_wide")


def flagsparse_spmv_csr(data=None, indices=None, indptr=None, x=None, shape=None, block_nnz=256,
                        max_segments=None, out=None, return_time=False, use_opt=False, prepared=None):
    """CSR SpMV: y = A @ x (reference: spmv_csr.py:557-610, same arguments and defaults).

    data, indices, indptr: CSR arrays; x: dense vector; shape: (n_rows, n_cols).
    prepared: result of prepare_spmv_csr for steady-state calls.  block_nnz, max_segments and use_opt
    select Triton launch shapes in the reference; here they are validated bookkeeping only -- both
    settings of use_opt run the same CUDA kernels.  Returns a new tensor, or `out` when it is given.
    """
    if prepared is None:
        if any(arg is None for arg in (data, indices, indptr, shape)):
            raise ValueError("data, indices, indptr, and shape are required when prepared is not provided")
        prepared = _prepare_spmv_csr(data, indices, indptr, shape, block_nnz, max_segments, reuse_expected=False)
    x = _validate_spmv_x(x, prepared)
    dev = prepared.data.device
    dtype = prepared.data.dtype
    if out is not None and (out.shape != (prepared.n_rows,) or out.dtype != dtype):
        raise ValueError("out shape/dtype must match result")
    if prepared.wide is not None:
        t0 = None
        if return_time:
            torch.cuda.synchronize(dev)
            t0 = time.perf_counter()
        y = widetypes.run(prepared, x, _spmv_launch_wide, (prepared.n_rows,))
        elapsed_ms = None
        if return_time:
            torch.cuda.synchronize(dev)
            elapsed_ms = (time.perf_counter() - t0) * 1000.0
        if out is not None:
            out.copy_(y)
            y = out
        return (y, elapsed_ms) if return_time else y
    # write straight into `out` when that is safe, else into a fresh vector that is copied over
    direct = out is not None and out.is_cuda and out.device == dev and out.is_contiguous()
    y = out if direct else torch.empty(prepared.n_rows, dtype=dtype, device=dev)
    t0 = None
    if return_time:
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
    _spmv_launch(prepared, x, y)
    elapsed_ms = None
    if return_time:
        torch.cuda.synchronize(dev)
        elapsed_ms = (time.perf_counter() - t0) * 1000.0
        prepared.check_status()
    if out is not None and not direct:
        out.copy_(y)
        y = out
    if return_time:
        return y, elapsed_ms
    return y


# ---------------------------------------------------------------------------------------------------
# COO front-end: convert to CSR, then the same kernels (reference: spmv_csr.py:613-758)
# ---------------------------------------------------------------------------------------------------
def coo_to_csr_for_spmv(data, row, col, shape, assume_sorted=False):
    """COO triple -> (values, int32 column indices, int64 row pointer) with the entries in (row, column) order,
    which is what the reference's function of this name returns (spmv_csr.py:623-647).  Entries already in order
    (or declared so) are not touched; otherwise one sort on the combined key.  The row pointer is read off
    the ordered row ids by binary search."""
    n_rows, n_cols = int(shape[0]), int(shape[1])
    dev = data.device
    rows, cols = row.to(torch.int64), col.to(torch.int64)
    if rows.numel() == 0:
        return data, cols.to(torch.int32), torch.zeros(n_rows + 1, dtype=torch.int64, device=dev)
    if not assume_sorted and rows.numel() > 1:
        key = rows * max(1, n_cols) + cols
        if bool((key[1:] < key[:-1]).any()):
            order = torch.argsort(key)     # entries with one (row, column) keep the order torch's default sort gives
            rows, cols, data = rows[order], cols[order], data[order]
        del key
    indptr = torch.searchsorted(rows.contiguous(), torch.arange(n_rows + 1, dtype=torch.int64, device=dev))
    return data, cols.to(torch.int32), indptr


def _check_coo_triple(data, row, col, extra=()):
    names = "data, row, col" + (", x" if extra else "")
    tensors = (data, row, col) + tuple(extra)
    if not all(torch.is_tensor(t) for t in tensors):
        raise TypeError(f"{names} must all be torch.Tensor")
    if not all(t.is_cuda for t in tensors):
        raise ValueError(f"{names} must all be CUDA tensors")
    if any(t.ndim != 1 for t in tensors):
        raise ValueError(f"{names} must all be 1D tensors")


def prepare_spmv_coo_tocsr(data, row, col, shape, block_nnz=256, max_segments=None, assume_sorted=False):
    """One-time COO -> CSR + analysis; use with flagsparse_spmv_coo_tocsr(..., prepared=p)
    (reference :650-684)."""
    _check_coo_triple(data, row, col)
    _check_value_dtype(data.dtype)
    if row.numel() != col.numel() or data.numel() != row.numel():
        raise ValueError("data, row, col must have the same length")
    data_s, indices, indptr = coo_to_csr_for_spmv(data, row, col, shape, assume_sorted=assume_sorted)
    return prepare_spmv_csr(data_s, indices, indptr, shape, block_nnz=block_nnz, max_segments=max_segments)


def flagsparse_spmv_coo_tocsr(data=None, row=None, col=None, x=None, shape=None, block_nnz=256,
                              max_segments=None, out=None, return_time=False, use_opt=True, prepared=None,
                              assume_sorted=False):
    """COO SpMV via CSR conversion: y = A @ x (reference :687-758, same arguments and defaults)."""
    if prepared is not None:
        if x is None:
            raise TypeError("x is required")
        if shape is None:
            shape = prepared.shape
        sh = (int(shape[0]), int(shape[1]))
        if sh != prepared.shape:
            raise ValueError(f"shape {sh} does not match prepared.shape {prepared.shape}")
        return flagsparse_spmv_csr(x=x, shape=shape, block_nnz=block_nnz, max_segments=max_segments, out=out,
                                   return_time=return_time, use_opt=use_opt, prepared=prepared)
    _check_coo_triple(data, row, col, extra=(x,))
    _check_value_dtype(data.dtype)
    if x.dtype != data.dtype:
        raise TypeError("x dtype must match data dtype")
    data_s, indices, indptr = coo_to_csr_for_spmv(data, row, col, shape, assume_sorted=assume_sorted)
    return flagsparse_spmv_csr(data_s, indices, indptr, x, shape, block_nnz=block_nnz,
                               max_segments=max_segments, out=out, return_time=return_time, use_opt=use_opt)
