"""ctypes binding of libfsb.so (declared in include/fsb.h).

The library is the only compute backend of this package: there is no Triton path and no CPU fallback.
`lib()` raises if the shared library has not been built (python -m flagsparse_b200.build), so a missing
extension is loud, never silent.
"""

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# FSB_BOUNDS_CHECK=1 in the environment selects the checking build (python -m flagsparse_b200.build --check): every
# product entry point then walks its index arrays first and refuses, with a record, a call that would leave them
CHECKING = os.environ.get("FSB_BOUNDS_CHECK", "") not in ("", "0")
LIB_PATH = os.path.join(_HERE, "csrc", "libfsb_check.so" if CHECKING else "libfsb.so")

FSB_F32, FSB_F64 = 0, 1
FSB_F16, FSB_BF16, FSB_C64, FSB_C128 = 2, 3, 4, 5     # fsb_spmv_csr_wide only
FSB_I32, FSB_I64 = 0, 1
FSB_SPMV_AUTO, FSB_SPMV_VECTOR, FSB_SPMV_STREAM = 0, 1, 2
FSB_SPMV_PANEL = 3  # host-side tag only: the panel kernel has its own entry point
FSB_SPMM_AUTO, FSB_SPMM_PLAIN, FSB_SPMM_BULK = 0, 1, 2
FSB_SPMM_ACCUMULATE = 16  # or-ed into the selector: C += A B
FSB_CUDA_ERROR_BASE = 1000

_ERRORS = {
    -1: "FSB_EINVAL (bad enum, negative size or missing pointer)",
    -2: "FSB_ERANGE (dimension outside the supported range)",
    -3: "FSB_EALIGN (pointer not aligned to its element size)",
    -4: "FSB_ESCRATCH (scratch buffer too small)",
    -5: "FSB_ENOSPACE (matrix too large for the built-in scratch array)",
    -6: "FSB_EBOUNDS (checking build: an index array would take a kernel out of bounds; nothing was launched)",
}
FSB_EBOUNDS = -6
BAD_KINDS = {
    1: "column index outside [0, n_cols)",
    2: "row pointer outside [0, nnz]",
    3: "row pointer smaller than the one before it",
    4: "row id outside [0, n_rows)",
    5: "panel slot with an accumulator beyond the spare one",
    6: "panel slot with an x position beyond the x buffers",
    7: "unit with a column chunk beyond n_cols",
    8: "unit or piece pointer table negative or decreasing",
}

_c = ctypes
_vp, _i64, _i32, _sz = _c.c_void_p, _c.c_int64, _c.c_int, _c.c_size_t

# name -> (restype, argtypes); must list every symbol include/fsb.h declares
SIGNATURES = {
    "fsb_version": (_i32, []),
    "fsb_spmv_tile_nnz": (_i32, [_i32, _i32]),
    "fsb_spmm_tile_nnz": (_i32, [_i32]),
    "fsb_csr_analyze": (_i32, [_i32, _i32, _vp, _vp, _i64, _i64, _vp, _vp]),
    "fsb_csr_num_tiles": (_i64, [_i64, _i32]),
    "fsb_csr_tile_plan": (_i32, [_i32, _vp, _i64, _i64, _i32, _vp, _vp]),
    "fsb_spmv_csr_scratch_bytes": (_sz, [_i32, _i64, _i32]),
    "fsb_spmv_csr": (_i32, [_i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _vp, _vp, _sz, _vp]),
    "fsb_spmv_csr_scatter": (
        _i32,
        [_i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i64, _i64, _i64, _i64, _i32, _i32, _vp, _vp, _sz, _vp],
    ),
    "fsb_spmv_csr_noalloc": (_i32, [_i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp, _vp]),
    "fsb_spmv_panel_piece_slots": (_i32, [_i32]),
    "fsb_spmv_panel_smem_bytes": (_sz, [_i32, _i32, _i32, _i32]),
    "fsb_spmv_panel_static_smem_bytes": (_sz, []),
    "fsb_spmv_csr_panel": (_i32, [_i32, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp,
                                  _i64, _i64, _vp, _vp]),
    "fsb_spmv_csr_panel_groups": (_i32, [_i32, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp,
                                         _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i64, _vp, _vp]),
    "fsb_spmm_csr_scratch_bytes": (_sz, [_i32, _i64, _i64]),
    "fsb_spmm_csr": (
        _i32,
        [_i32, _i32, _i32, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _vp, _sz, _vp, _vp],
    ),
    "fsb_spmv_csr_wide": (_i32, [_i32, _i32, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "fsb_spmm_csr_wide": (_i32, [_i32, _i32, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _i64, _vp]),
    "fsb_sddmm_csr": (_i32, [_i32, _vp, _vp, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _c.c_double,
                             _c.c_double, _vp]),
    "fsb_panel_build_max_chunks": (_i32, []),
    "fsb_panel_build_count": (_i32, [_i32, _i32, _vp, _vp, _i64, _i64, _i32, _i32, _vp, _vp]),
    "fsb_panel_build_sort": (_i32, [_i32, _i32, _i32, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp,
                                    _vp]),
    "fsb_panel_build_window": (_i32, [_i32]),
    "fsb_panel_build_core_count": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp]),
    "fsb_panel_build_core_place": (_i32, [_i32, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp,
                                          _vp, _vp, _vp, _vp, _vp, _vp]),
    "fsb_panel_build_runs": (_i32, [_vp, _vp, _i64, _i32, _vp, _vp]),
    "fsb_panel_build_cut": (_i32, [_vp, _vp, _i32, _i32, _vp, _vp, _vp, _vp, _vp]),
    "fsb_panel_build_fill": (_i32, [_i32, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp,
                                    _vp]),
    "fsb_bounds_check_enabled": (_i32, []),
    "fsb_bounds_check_report": (_i32, [_vp]),
}

_lib = None


def lib():
    """Load libfsb.so once and attach the prototypes.  Raises RuntimeError when it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m flagsparse_b200.build"
                f"{' --check' if CHECKING else ''}` (this package has no fallback path)"
            )
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(rc, what):
    """Turn a non-zero return code of the C ABI into a RuntimeError."""
    if rc == 0:
        return
    if rc >= FSB_CUDA_ERROR_BASE:
        raise RuntimeError(f"{what}: CUDA error {rc - FSB_CUDA_ERROR_BASE}")
    if rc == FSB_EBOUNDS:
        seen, kind, where, value, limit = bounds_report()
        raise IndexError(f"{what}: {_ERRORS[rc]}: {BAD_KINDS.get(kind, kind)} at position {where} "
                         f"(value {value}, limit {limit}; {seen} violation(s) seen)")
    raise RuntimeError(f"{what}: {_ERRORS.get(rc, rc)}")


def bounds_report():
    """(violations seen, kind, position, value, limit) of the last call the checking build refused; clears it."""
    out = (ctypes.c_int64 * 5)()
    lib().fsb_bounds_check_report(ctypes.cast(out, ctypes.c_void_p))
    return tuple(int(v) for v in out)
