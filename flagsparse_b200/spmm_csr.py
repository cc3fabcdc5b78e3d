"""CSR SpMM host code: the reference's entry points over the hand-written sm_100a kernel.

Same names, arguments, defaults, validation order and exception types as the reference's
src/flagsparse/sparse_operations/spmm_csr.py (_prepare_spmm_csr_matrix :197-255,
_prepare_spmm_csr_inputs :258-281, the launch-override checks :284-334, PreparedCsrSpmmOpt
:337-392, prepare_spmm_csr_opt :480-522, flagsparse_spmm_csr :1057-1126, flagsparse_spmm_csr_opt
:1129-1183).  Both entry points run the same nnz-tiled CUDA kernel; the reference's row-length buckets
and its split workspace for rows over 2048 nnz are replaced by the tile plan and per-tile partial rows.
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
    StatusWord,
    _stream_ptr,
    _tile_plan,
)

_SPMM_ALGO_NAMES = {"auto": _lib.FSB_SPMM_AUTO, "plain": _lib.FSB_SPMM_PLAIN, "bulk": _lib.FSB_SPMM_BULK}

# A product whose gathers range over more of B than stays in L2 can be split: A into column panels (each panel's
# slice of B at most this many bytes per column tile, so that it is fetched from DRAM about once) and B / C into
# column tiles of one 128-byte line per row; passes after the first add to C.  Off by default (0): on the 2^20-row
# matrix with 16 uniform entries per row every split measured slower than the single pass (width 32: 0.31 ms with
# two panels, 0.43 ms with four, against 0.23 ms) -- a pass over rows of a few entries each is bound by the latency
# of its read-add-write of C, not by the bytes it saves.  FSB_SPMM_PANEL_MB=<MiB> or FSB_SPMM_PANELS=<n> turn it on.
PANEL_BYTES = 0
COL_TILE_BYTES = 128
SPAN_WINDOW = 1 << 20        # consecutive entries over which the column span is sampled


def _panel_bytes():
    v = os.environ.get("FSB_SPMM_PANEL_MB")
    return PANEL_BYTES if v is None else int(float(v) * (1 << 20))


class _CsrPart:
    """CSR arrays of one column panel of A (or of all of A) plus the tile plan and scratch the kernel needs."""

    __slots__ = ("data", "kernel_indices", "kernel_indptr", "n_rows", "tile_row", "_scratch")

    def __init__(self, data, kernel_indices, kernel_indptr, n_rows, tile_nnz):
        self.data, self.kernel_indices, self.kernel_indptr, self.n_rows = data, kernel_indices, kernel_indptr, n_rows
        self.tile_row = _tile_plan(kernel_indptr, n_rows, data.numel(), tile_nnz) if data.numel() > 0 and n_rows > 0 \
            else None
        self._scratch = {}

    def scratch_for(self, n_dense):
        buf = self._scratch.get(n_dense)
        if buf is None:
            nbytes = int(_lib.lib().fsb_spmm_csr_scratch_bytes(_VTYPE[self.data.dtype], self.data.numel(), n_dense))
            buf = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=self.data.device)
            self._scratch = {n_dense: buf}  # keep one width at a time
        return buf


def split_by_column_panels(data, indices, indptr, n_rows, n_cols, n_panels):
    """CSR arrays (data, indices, indptr) of the n_panels column panels of A: panel p holds the entries whose
    column lies in [p * w, (p + 1) * w), w = ceil(n_cols / n_panels), in their original order; every panel keeps
    all n_rows rows (rows without entries in a panel are empty there)."""
    w = -(-n_cols // n_panels)
    lens = (indptr[1:] - indptr[:-1]).to(torch.int64)
    rows = torch.repeat_interleave(torch.arange(n_rows, device=data.device), lens)
    panel_of = torch.div(indices.to(torch.int64), w, rounding_mode="floor")
    out = []
    for p in range(n_panels):
        keep = panel_of == p
        counts = torch.bincount(rows[keep], minlength=n_rows)
        ptr = torch.zeros(n_rows + 1, dtype=indptr.dtype, device=data.device)
        ptr[1:] = torch.cumsum(counts, 0).to(indptr.dtype)
        out.append((data[keep].contiguous(), indices[keep].contiguous(), ptr))
    return out


def _prepare_spmm_csr_matrix(data, indices, indptr, shape):
    """Checks of the reference's function of this name (spmm_csr.py:197-255), in its order.  Returns
    (data, kernel_indices, kernel_indptr, n_rows, n_cols, stats); unlike the reference the indptr keeps
    its 32-bit width when it has one (the kernels read either)."""
    if len(shape) != 2:
        raise ValueError("shape must be a 2-tuple: (n_rows, n_cols)")
    if data.ndim != 1 or indices.ndim != 1 or indptr.ndim != 1:
        raise ValueError("data, indices, and indptr must be 1D tensors")
    n_rows, n_cols = int(shape[0]), int(shape[1])
    if n_rows < 0 or n_cols < 0:
        raise ValueError("shape dimensions must be non-negative")
    if indptr.numel() != n_rows + 1:
        raise ValueError(f"indptr length must be n_rows+1={n_rows + 1}, got {indptr.numel()}")
    if data.numel() != indices.numel():
        raise ValueError("data and indices must have the same length (nnz)")
    if not all(t.is_cuda for t in (data, indices, indptr)):
        raise ValueError("data, indices, and indptr must be CUDA tensors")
    if not all(t.device == data.device for t in (indices, indptr)):
        raise ValueError("data, indices, and indptr must be on the same CUDA device")
    _check_value_dtype(data.dtype)
    if indices.dtype not in SUPPORTED_INDEX_DTYPES:
        raise TypeError("indices dtype must be torch.int32 or torch.int64")
    if indptr.dtype not in SUPPORTED_INDEX_DTYPES:
        raise TypeError("indptr dtype must be torch.int32 or torch.int64")

    data = data.contiguous()
    indices = indices.contiguous()
    indptr = indptr.contiguous()
    nnz = data.numel()
    stats = _analyze_csr(indices, indptr, n_rows)
    if stats.ptr_first != 0:
        raise ValueError("indptr[0] must be 0")
    if stats.ptr_last != nnz:
        raise ValueError(f"indptr[-1] must equal nnz={nnz}, got {stats.ptr_last}")
    if stats.n_decreasing > 0:
        raise ValueError("indptr must be nondecreasing")
    if nnz > 0:
        if stats.min_index < 0 or stats.max_index >= n_cols:
            raise IndexError("indices out of range for n_cols")
        if stats.max_index > _INDEX_LIMIT_INT32:
            raise ValueError("column indices exceed the int32 range supported by the kernel")
    kernel_indices = indices.to(torch.int32) if indices.dtype == torch.int64 else indices
    return data, kernel_indices, indptr, n_rows, n_cols, stats


def _check_spmm_dense(B, data, n_cols):
    """Checks on B of the reference's _prepare_spmm_csr_inputs (spmm_csr.py:271-280)."""
    if B.shape[0] != n_cols:
        raise ValueError(f"B.shape[0] must be n_cols={n_cols}, got {B.shape[0]}")
    if not B.is_cuda:
        raise ValueError("B must be a CUDA tensor")
    if B.device != data.device:
        raise ValueError("B must be on the same CUDA device as the sparse matrix")
    if B.dtype != data.dtype:
        raise TypeError("B dtype must match data dtype")
    return _row_major(B)


def _row_major(B):
    """B as the kernel can read it: unit stride along a row, any stride between rows (the reference copies every
    non-contiguous B, spmm_csr.py:280; a row-strided view needs no copy here)."""
    if B.shape[1] <= 1 or B.stride(1) == 1:
        if B.shape[0] <= 1 or B.stride(0) >= B.shape[1]:
            return B
    return B.contiguous()


# (dense columns above which the shape applies, lanes, column factor): the launch shapes the reference picks for its
# base SpMM kernel (spmm_csr.py:284-296).  The CUDA kernel does not use them; they only give the defaults against
# which explicit overrides are checked, and the bookkeeping dictionary callers may look at.
_ALG1_SHAPES = ((64, 32, 4), (32, 32, 2), (16, 32, 1), (8, 16, 1), (4, 8, 1))


def _alg1_shape(n_dense_cols):
    for above, lanes, factor in _ALG1_SHAPES:
        if n_dense_cols > above:
            return lanes, factor
    return 4, 1


def _check_launch_overrides(n_dense_cols, max_row_nnz, block_n=None, block_nnz=None, max_segments=None):
    """The two ways a call can be refused for its launch overrides, as in the reference (spmm_csr.py:299-334): a
    non-positive block size or segment count, and a max_segments that cannot hold the longest row.  Returns the
    reference's bookkeeping for the accepted values."""
    lanes, factor = _alg1_shape(n_dense_cols)
    tile_cols = lanes * factor if block_n is None else block_n
    seg_len = lanes if block_nnz is None else block_nnz
    if min(tile_cols, seg_len) <= 0:
        raise ValueError("block_n and block_nnz, when given, must be positive")
    needed = -(-max_row_nnz // seg_len) if max_row_nnz > 0 else 0
    if max_segments is not None:
        if max_segments <= 0:
            raise ValueError("max_segments, when given, must be positive")
        if needed > int(max_segments):
            raise ValueError(f"the longest row needs {needed} segments of {seg_len} entries; max_segments allows "
                             f"{int(max_segments)}")
    return {"block_n": int(tile_cols), "block_nnz": int(seg_len),
            "max_segments": None if max_segments is None else int(max_segments), "required_segments": int(needed),
            "warp_size": int(lanes), "factor": int(factor), "max_row_nnz": int(max_row_nnz),
            "auto_max_segments": max_segments is None}


def _select_spmm_opt_block_n(n_dense_cols):
    """Column-tile table of the reference's opt path (spmm_csr.py:405-414); informational here."""
    for bound in (8, 16, 32, 64):
        if n_dense_cols <= bound:
            return bound
    return 128


class PreparedCsrSpmmOpt:
    """Cached CSR metadata for repeated SpMM calls on the same sparse matrix.

    Attribute names follow the reference's class (spmm_csr.py:337-392).  `row_buckets` describes the tile
    plan; the `long_*` split tables of the reference stay empty because rows of any length go through the
    same tiles.  Scratch (two partial rows per tile) depends on the width of B and is cached per width:
    calls that share a prepared object must not overlap on the GPU.
    """

    __slots__ = (
        "data", "kernel_indices", "kernel_indptr", "shape", "n_rows", "n_cols", "max_row_nnz",
        "row_buckets", "supports_opt", "long_part_rows", "long_part_starts", "long_part_ends",
        "long_row_ids", "long_row_part_ptr", "long_row_fallback_only", "stats", "tile_nnz", "tile_row",
        "_scratch", "_status", "_row_lengths", "wide", "_whole", "_panels", "_span",
    )

    def __init__(self, data, kernel_indices, kernel_indptr, shape, n_rows, n_cols, stats, tile_nnz, tile_row,
                 wide=None):
        dev = data.device
        self.data = data
        self.kernel_indices = kernel_indices
        self.kernel_indptr = kernel_indptr
        self.shape = (int(shape[0]), int(shape[1]))
        self.n_rows = int(n_rows)
        self.n_cols = int(n_cols)
        self.max_row_nnz = int(stats.max_row_nnz)
        self.stats = stats
        self.tile_nnz = tile_nnz
        self.tile_row = tile_row
        n_tiles = 0 if tile_row is None else tile_row.numel() - 1
        self.row_buckets = [{"kind": "tiles", "tile_nnz": tile_nnz, "n_tiles": n_tiles, "n_rows": self.n_rows}]
        self._scratch = None
        self.supports_opt = data.dtype in (torch.float32, torch.float64)
        self.long_part_rows = torch.empty((0,), dtype=torch.int32, device=dev)
        self.long_part_starts = torch.empty((0,), dtype=torch.int64, device=dev)
        self.long_part_ends = torch.empty((0,), dtype=torch.int64, device=dev)
        self.long_row_ids = torch.empty((0,), dtype=torch.int32, device=dev)
        self.long_row_part_ptr = torch.zeros(1, dtype=torch.int64, device=dev)
        self.long_row_fallback_only = False
        self._status = None
        self._row_lengths = None
        self._whole = None       # the matrix as one _CsrPart (shares the tile plan)
        self._panels = {}        # number of column panels -> list of _CsrPart
        self._span = None        # columns spanned by a window of consecutive entries (median over samples)
        # float16 / bfloat16 / complex values: ("native", []) -- the product goes through fsb_spmm_csr_wide
        self.wide = wide

    @property
    def row_lengths(self):
        if self._row_lengths is None:
            p = self.kernel_indptr.to(torch.int64)
            self._row_lengths = p[1:] - p[:-1] if self.n_rows > 0 else p.new_empty((0,))
        return self._row_lengths

    # -- how a product of a given width is run --------------------------------------------------------------
    def column_span(self):
        """Median number of columns between the smallest and the largest column index inside windows of
        SPAN_WINDOW consecutive entries: about how many rows of B the CTAs running at one time gather from."""
        if self._span is None:
            idx = self.kernel_indices
            nnz = idx.numel()
            if nnz == 0:
                self._span = 0
            else:
                k = max(1, min(64, nnz // SPAN_WINDOW))
                win = min(SPAN_WINDOW, nnz)
                starts = [(nnz - win) * j // max(1, k - 1) if k > 1 else 0 for j in range(k)]
                spans = [int(idx[s0:s0 + win].max()) - int(idx[s0:s0 + win].min()) + 1 for s0 in starts[:8]]
                spans.sort()
                self._span = spans[len(spans) // 2]
        return self._span

    def n_panels_for(self, n_dense):
        """Column panels of A for a product of this width (1 = the matrix as it is)."""
        forced = int(os.environ.get("FSB_SPMM_PANELS", "0"))
        if forced > 0:
            return forced
        limit = _panel_bytes()
        if limit <= 0 or self.tile_row is None:
            return 1
        sv = self.data.element_size()
        row_bytes = min(n_dense * sv, COL_TILE_BYTES)
        if self.column_span() * row_bytes <= limit:
            return 1                                  # the gathers of concurrent CTAs stay within what L2 holds
        return max(1, min(16, -(-self.n_cols * row_bytes // limit)))

    def parts_for(self, n_panels):
        if n_panels == 1:
            if self._whole is None:
                part = _CsrPart.__new__(_CsrPart)
                part.data, part.kernel_indices, part.kernel_indptr = self.data, self.kernel_indices, self.kernel_indptr
                part.n_rows, part.tile_row, part._scratch = self.n_rows, self.tile_row, {}
                self._whole = part
            return [self._whole]
        parts = self._panels.get(n_panels)
        if parts is None:
            triples = split_by_column_panels(self.data, self.kernel_indices, self.kernel_indptr, self.n_rows,
                                             self.n_cols, n_panels)
            parts = [_CsrPart(d, i, p, self.n_rows, self.tile_nnz) for d, i, p in triples]
            self._panels = {n_panels: parts}          # keep one split at a time
        return parts

    def passes_for(self, n_dense):
        """[(part, first column, width, accumulate)]: the launches of one product, in order."""
        n_panels = self.n_panels_for(n_dense)
        parts = self.parts_for(n_panels)
        sv = self.data.element_size()
        tile = n_dense if n_panels == 1 else max(1, COL_TILE_BYTES // sv)
        out = []
        for c0 in range(0, n_dense, tile):
            for k, part in enumerate(parts):
                out.append((part, c0, min(tile, n_dense - c0), k > 0))
        return out

    def launches_per_product(self, n_dense):
        return sum(2 if (part.tile_row is not None and part.tile_row.numel() > 2) else 1
                   for part, _, _, _ in self.passes_for(n_dense))

    def plan_summary(self, n_dense):
        passes = self.passes_for(n_dense)
        return {"column_panels_of_A": self.n_panels_for(n_dense), "column_tiles_of_B": len({c for _, c, _, _ in passes}),
                "passes": len(passes), "column_span": self.column_span(), "panel_bytes_limit": _panel_bytes()}

    def status_word(self):
        if self._status is None:
            self._status = StatusWord(self.data.device)
        return self._status

    def check_status(self):
        """Wait for the last product on this matrix and raise RuntimeError if its kernel gave up on a bounded
        device-side wait (tiles of C are then unwritten).  Every product also looks, without waiting, at how the
        previous one ended."""
        if self._status is not None:
            self._status.check()
        if self.wide is not None:
            for part in self.wide[1]:
                part.check_status()


def prepare_spmm_csr_opt(data, indices, indptr, shape):
    """Analyse a CSR matrix once for repeated SpMM calls (reference: spmm_csr.py:480-522)."""
    data, kernel_indices, kernel_indptr, n_rows, n_cols, stats = _prepare_spmm_csr_matrix(
        data, indices, indptr, shape
    )
    nnz = data.numel()
    if data.dtype in widetypes.WIDE_DTYPES:
        # read as stored by fsb_spmm_csr_wide: nothing to plan, no second copy of the matrix
        return PreparedCsrSpmmOpt(data, kernel_indices, kernel_indptr, shape, n_rows, n_cols, stats, 0, None,
                                  wide=("native", []))
    tile_nnz, tile_row = 0, None
    if nnz > 0 and n_rows > 0:
        tile_nnz = int(_lib.lib().fsb_spmm_tile_nnz(_VTYPE[data.dtype]))
        tile_row = _tile_plan(kernel_indptr, n_rows, nnz, tile_nnz)
    return PreparedCsrSpmmOpt(data, kernel_indices, kernel_indptr, shape, n_rows, n_cols, stats, tile_nnz, tile_row)


def _spmm_launch(prepared, B, C):
    """Enqueue C = A B on the current stream.  Stands in for _triton_spmm_csr_impl (spmm_csr.py:525-599)
    and _triton_spmm_csr_impl_opt_prepared (:1033-1055).  One launch of the tiled kernel per pass: the whole
    product, or (column panel of A) x (column tile of B) passes when B is too large to be gathered from L2."""
    L = _lib.lib()
    p = prepared
    dev = p.data.device
    n_dense = int(B.shape[1])
    if p.n_rows == 0 or n_dense == 0:
        return
    algo = _SPMM_ALGO_NAMES.get(os.environ.get("FSB_SPMM_ALGO", "auto").strip().lower(), _lib.FSB_SPMM_AUTO)
    status = p.status_word()
    status.poll()
    sv = B.element_size()
    vt, it, pt = _VTYPE[p.data.dtype], _ITYPE[p.kernel_indices.dtype], _ITYPE[p.kernel_indptr.dtype]
    ldb, ldc = B.stride(0), C.stride(0)
    stream = _stream_ptr(dev)
    with torch.cuda.device(dev):
        for part, c0, width, accumulate in p.passes_for(n_dense):
            scratch = part.scratch_for(width) if part.tile_row is not None else None
            rc = L.fsb_spmm_csr(
                vt, it, pt, _ptr(part.data), _ptr(part.kernel_indices), part.kernel_indptr.data_ptr(),
                B.data_ptr() + c0 * sv, ldb, C.data_ptr() + c0 * sv, ldc, p.n_rows, p.n_cols, width,
                part.data.numel(), algo | (_lib.FSB_SPMM_ACCUMULATE if accumulate else 0),
                None if part.tile_row is None else part.tile_row.data_ptr(),
                None if scratch is None else scratch.data_ptr(), 0 if scratch is None else scratch.numel(),
                status.data_ptr(), stream,
            )
            _lib.check(rc, "fsb_spmm_csr")
    status.posted("fsb_spmm_csr")


def _check_out(out, device, shape, dtype, device_msg):
    if not out.is_cuda:
        raise ValueError("out must be a CUDA tensor")
    if out.device != device:
        raise ValueError(device_msg)
    if out.shape != shape or out.dtype != dtype:
        raise ValueError("out shape/dtype must match result")


def _spmm_launch_wide(prepared, B, C):
    """Enqueue C = A B for float16 / bfloat16 / complex values (fsb_spmm_csr_wide): B and C are float32 for the half
    precisions and of the matrix's own type for complex values; B may have any row stride.  Stands in for the
    reference's base launch helper on these types (_triton_spmm_csr_impl, spmm_csr.py:525-599)."""
    from .spmv_csr import _WIDE_VTYPE

    p = prepared
    dev = p.data.device
    if p.n_rows == 0 or B.shape[1] == 0:
        return
    with torch.cuda.device(dev):
        rc = _lib.lib().fsb_spmm_csr_wide(
            _WIDE_VTYPE[p.data.dtype], _ITYPE[p.kernel_indptr.dtype], _ptr(p.data), _ptr(p.kernel_indices),
            p.kernel_indptr.data_ptr(), _ptr(B), B.stride(0) if B.shape[0] > 1 else B.shape[1], _ptr(C), C.stride(0),
            p.n_rows, p.n_cols, int(B.shape[1]), p.data.numel(), _stream_ptr(dev),
        )
    _lib.check(rc, "fsb_spmm_csr_wide")


def _run_spmm(prepared, B, out, return_time):
    dev, dtype = prepared.data.device, prepared.data.dtype
    shape = (prepared.n_rows, int(B.shape[1]))
    if prepared.wide is not None:
        t0 = None
        if return_time:
            torch.cuda.synchronize(dev)
            t0 = time.perf_counter()
        C = widetypes.run(prepared, B, _spmm_launch_wide, shape)
        elapsed_ms = None
        if return_time:
            torch.cuda.synchronize(dev)
            elapsed_ms = (time.perf_counter() - t0) * 1000.0
        if out is not None:
            out.copy_(C)
            C = out
        return (C, elapsed_ms) if return_time else C
    direct = out is not None and out.is_contiguous()
    C = out if direct else torch.empty(shape, dtype=dtype, device=dev)
    t0 = None
    if return_time:
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
    _spmm_launch(prepared, B, C)
    elapsed_ms = None
    if return_time:
        torch.cuda.synchronize(dev)
        elapsed_ms = (time.perf_counter() - t0) * 1000.0
        prepared.check_status()
    if out is not None and not direct:
        out.copy_(C)
        C = out
    if return_time:
        return C, elapsed_ms
    return C


def flagsparse_spmm_csr(data, indices, indptr, B, shape, block_n=None, block_nnz=None, max_segments=None,
                        out=None, return_time=False):
    """CSR SpMM: C = A @ B (reference: spmm_csr.py:1057-1126, same arguments and defaults).

    A is given as CSR arrays; B is a dense CUDA tensor of shape (n_cols, n_dense_cols), any strides.
    block_n / block_nnz / max_segments are the reference's Triton launch overrides: validated the same
    way, otherwise unused.  Unlike the reference this call does not synchronise the device unless
    return_time is set.
    """
    if block_n is not None and block_n <= 0:
        raise ValueError("block_n must be positive when provided")
    if block_nnz is not None and block_nnz <= 0:
        raise ValueError("block_nnz must be positive when provided")
    if max_segments is not None and max_segments <= 0:
        raise ValueError("max_segments must be positive when provided")
    if B.ndim != 2:
        raise ValueError("B must be a 2D dense tensor")
    prepared = prepare_spmm_csr_opt(data, indices, indptr, shape)
    B = _check_spmm_dense(B, prepared.data, prepared.n_cols)
    n_dense_cols = int(B.shape[1])
    _check_launch_overrides(n_dense_cols, prepared.max_row_nnz, block_n=block_n, block_nnz=block_nnz,
                                     max_segments=max_segments)
    if out is not None:
        _check_out(out, prepared.data.device, (prepared.n_rows, n_dense_cols), prepared.data.dtype,
                   "out must be on the same CUDA device as the inputs")
    return _run_spmm(prepared, B, out, return_time)


def flagsparse_spmm_csr_opt(data=None, indices=None, indptr=None, B=None, shape=None, prepared=None, out=None,
                            return_time=False):
    """CSR SpMM on a prepared matrix (reference: spmm_csr.py:1129-1183, same arguments and defaults)."""
    if prepared is not None and not isinstance(prepared, PreparedCsrSpmmOpt):
        raise TypeError("prepared must be a PreparedCsrSpmmOpt instance")
    if prepared is None:
        if any(arg is None for arg in (data, indices, indptr, shape)):
            raise ValueError("data, indices, indptr, and shape are required when prepared is not provided")
        prepared = prepare_spmm_csr_opt(data, indices, indptr, shape)
    elif shape is not None:
        resolved_shape = (int(shape[0]), int(shape[1]))
        if resolved_shape != prepared.shape:
            raise ValueError(f"shape {resolved_shape} does not match prepared.shape {prepared.shape}")
    if B is None:
        raise ValueError("B is required")
    if not prepared.supports_opt:
        raise TypeError("flagsparse_spmm_csr_opt only supports float32 and float64")
    if not B.is_cuda:
        raise ValueError("B must be a CUDA tensor")
    if B.device != prepared.data.device:
        raise ValueError("B must be on the same CUDA device as sparse matrix data")
    if out is not None:
        _check_out(out, prepared.data.device, (prepared.n_rows, int(B.shape[1])), prepared.data.dtype,
                   "out must be on the same CUDA device as sparse matrix data")
    # checks the reference makes inside its launch helper (:1040-1046)
    if B.dtype != prepared.data.dtype:
        raise TypeError("B dtype must match sparse matrix dtype")
    if B.shape[0] != prepared.n_cols:
        raise ValueError(f"B.shape[0] must be n_cols={prepared.n_cols}, got {B.shape[0]}")
    if B.ndim != 2:
        raise ValueError("B must be a 2D dense tensor")
    return _run_spmm(prepared, _row_major(B), out, return_time)
