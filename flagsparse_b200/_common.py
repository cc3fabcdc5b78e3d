"""Dtype tables, limits and tolerances shared by the CSR SpMV / SpMM host code.

Mirrors the conventions of the reference's src/flagsparse/sparse_operations/_common.py:22-31 (dtype
whitelists, int32 index limit) and :76-85 (allclose tolerances).  The CUDA kernels compute float32 and float64;
the other four value dtypes of the reference's whitelist run through them by widening or by splitting complex
values into real and imaginary matrices (widetypes.py), on the entry points where the reference accepts them.
"""

import torch

from . import _lib

SUPPORTED_VALUE_DTYPES = (torch.float16, torch.bfloat16, torch.float32, torch.float64, torch.complex64,
                          torch.complex128)
# what the kernels themselves compute in; the other value dtypes are widened or split on the host
NATIVE_VALUE_DTYPES = (torch.float32, torch.float64)
SUPPORTED_INDEX_DTYPES = (torch.int32, torch.int64)
_INDEX_LIMIT_INT32 = 2**31 - 1

_VTYPE = {torch.float32: _lib.FSB_F32, torch.float64: _lib.FSB_F64}
_ITYPE = {torch.int32: _lib.FSB_I32, torch.int64: _lib.FSB_I64}


def _check_value_dtype(dtype, what="data"):
    if dtype in SUPPORTED_VALUE_DTYPES:
        return
    raise TypeError(
        f"{what} dtype must be one of: float16, bfloat16, float32, float64, complex64, complex128"
    )


def _tolerance_for_dtype(value_dtype):
    """(atol, rtol) used by the reference's allclose checks (_common.py:76-85)."""
    if value_dtype == torch.float16:
        return 2e-3, 2e-3
    if value_dtype == torch.bfloat16:
        return 1e-1, 1e-1
    if value_dtype in (torch.float32, torch.complex64):
        return 1e-6, 1e-5
    if value_dtype in (torch.float64, torch.complex128):
        return 1e-10, 1e-8
    return 1e-6, 1e-5


def _stream_ptr(device):
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t):
    return t.data_ptr() if t is not None and t.numel() > 0 else None


class CsrStats:
    """The eight numbers fsb_csr_analyze produces, read back with a single device-to-host copy."""

    __slots__ = ("ptr_first", "ptr_last", "n_decreasing", "min_index", "max_index", "max_row_nnz",
                 "n_empty_rows", "n_long_rows")

    def __init__(self, values):
        (self.ptr_first, self.ptr_last, self.n_decreasing, self.min_index, self.max_index,
         self.max_row_nnz, self.n_empty_rows, self.n_long_rows) = (int(v) for v in values)


def _analyze_csr(indices, indptr, n_rows):
    """One fused device pass over indptr and indices (the reference does six reductions with six host
    syncs, spmv_csr.py:404-427); returns CsrStats."""
    L = _lib.lib()
    stats = torch.empty(8, dtype=torch.int64, device=indptr.device)
    with torch.cuda.device(indptr.device):
        rc = L.fsb_csr_analyze(
            _ITYPE[indices.dtype], _ITYPE[indptr.dtype], _ptr(indices), indptr.data_ptr(),
            n_rows, indices.numel(), stats.data_ptr(), _stream_ptr(indptr.device),
        )
    _lib.check(rc, "fsb_csr_analyze")
    return CsrStats(stats.cpu().tolist())


def _tile_plan(indptr, n_rows, nnz, tile_nnz):
    """int32 tile_row[n_tiles + 1] on the device (see fsb_csr_tile_plan in include/fsb.h)."""
    L = _lib.lib()
    n_tiles = int(L.fsb_csr_num_tiles(nnz, tile_nnz))
    plan = torch.empty(n_tiles + 1, dtype=torch.int32, device=indptr.device)
    with torch.cuda.device(indptr.device):
        rc = L.fsb_csr_tile_plan(
            _ITYPE[indptr.dtype], indptr.data_ptr(), n_rows, nnz, tile_nnz, plan.data_ptr(),
            _stream_ptr(indptr.device),
        )
    _lib.check(rc, "fsb_csr_tile_plan")
    return plan


class StatusWord:
    """The word through which a kernel reports that one of its bounded waits ran out, and the host side of it.
    The word lives in pinned host memory that the GPU writes directly (only when a wait does run out), so looking
    at it costs neither a copy nor a synchronisation: every call on the same object polls it, and check() waits
    for the last launch first.  A set word is reset and turned into a RuntimeError, so a product whose kernel gave
    up is never handed on silently."""

    def __init__(self, device):
        device = torch.device(device)
        self._cuda = device.type == "cuda"
        self.word = torch.zeros(1, dtype=torch.int32)
        if self._cuda:
            self.word = self.word.pin_memory()       # page-locked: the same address is valid on the device
        self._event = None
        self._what = None

    def data_ptr(self):
        return self.word.data_ptr()

    def item(self):
        return int(self.word[0])

    def posted(self, what, stream=None):
        """Call right after a launch that may set the word; `stream` is the torch stream of that launch (default:
        the current one)."""
        if not self._cuda:
            return
        if self._event is None:
            self._event = torch.cuda.Event()
        self._event.record(stream or torch.cuda.current_stream())
        self._what = what

    def poll(self):
        """Raise if a launch is known to have failed; never waits for the GPU."""
        if int(self.word[0]) != 0:
            self._raise()

    def check(self):
        """Wait for the last launch and raise if it (or an earlier one) failed."""
        if self._event is not None:
            self._event.synchronize()
        if int(self.word[0]) != 0:
            self._raise()

    def _raise(self):
        code, what = int(self.word[0]), self._what or "a kernel of this matrix"
        self.word.zero_()
        raise RuntimeError(f"{what}: a device-side wait ran out (status {code}); the result of that call is "
                           "incomplete")
