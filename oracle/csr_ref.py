"""ctypes wrapper of oracle/libcsr_ref.so (built by oracle/Makefile) -- TEST INFRASTRUCTURE ONLY."""

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libcsr_ref.so")
_lib = None


def build(force=False):
    src = os.path.join(_HERE, "csr_ref.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libcsr_ref.so"], check=True, stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.csr_ref_max_threads.restype = ctypes.c_int
        _lib.csr_ref_spmv.restype = None
        _lib.csr_ref_spmm.restype = None
    return _lib


def max_threads():
    return int(lib().csr_ref_max_threads())


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _split_indices(indices):
    indices = np.ascontiguousarray(indices)
    if indices.dtype == np.int32:
        return indices, _p(indices), None
    indices = indices.astype(np.int64, copy=False)
    return indices, None, _p(indices)


def spmv(data, indices, indptr, shape, x, native=False, threads=1):
    """y = A x on `threads` host threads; float64 accumulation unless native=True."""
    data = np.ascontiguousarray(data)
    x = np.ascontiguousarray(x, dtype=data.dtype)
    ptr = np.ascontiguousarray(indptr, dtype=np.int64)
    keep, i32, i64 = _split_indices(indices)
    y = np.empty(shape[0], dtype=data.dtype)
    lib().csr_ref_spmv(ctypes.c_int(int(data.dtype == np.float64)), _p(data), i32, i64, _p(ptr), _p(x), _p(y),
                       ctypes.c_int64(shape[0]), ctypes.c_int(int(native)), ctypes.c_int(int(threads)))
    return y


def spmm(data, indices, indptr, shape, b, native=False, threads=1):
    """C = A B (B row-major) on `threads` host threads; float64 accumulation unless native=True."""
    data = np.ascontiguousarray(data)
    b = np.ascontiguousarray(b, dtype=data.dtype)
    ptr = np.ascontiguousarray(indptr, dtype=np.int64)
    keep, i32, i64 = _split_indices(indices)
    n_dense = b.shape[1]
    c = np.empty((shape[0], n_dense), dtype=data.dtype)
    lib().csr_ref_spmm(ctypes.c_int(int(data.dtype == np.float64)), _p(data), i32, i64, _p(ptr), _p(b),
                       ctypes.c_int64(n_dense), _p(c), ctypes.c_int64(n_dense), ctypes.c_int64(shape[0]),
                       ctypes.c_int64(n_dense), ctypes.c_int(int(native)), ctypes.c_int(int(threads)))
    return c
