"""float16, bfloat16, complex64 and complex128 values: the host side of fsb_spmv_csr_wide / fsb_spmm_csr_wide.

The reference's base paths take these four value types by computing in a wider real type and casting back:
half precisions run its float32 kernel on `data.to(float32)` and `x.to(float32)` and round the result
(src/flagsparse/sparse_operations/spmv_csr.py:496-535, spmm_csr.py:525-560 of the reference), complex values run a
kernel over the interleaved real view (spmv_csr.py:123-155, 536-554; spmm_csr.py:138-195).  Here one kernel per
product reads the matrix as it is stored (2 bytes per half-precision value, interleaved pairs for complex values):
  * float16 / bfloat16: the dense operand is widened to float32 once per call, products and sums are float32, the
    float32 result is rounded once to the caller's type;
  * complex: operand and result stay in the caller's type.
`dense_dtype` says which type the kernel's dense operand and result have; `run` does the widening, the launch and
the rounding around a caller-supplied `launch(prepared, dense operand, dense result)`, which is the CUDA launch in
the package and a host stand-in in the CPU tests.
"""

import torch

HALF_DTYPES = (torch.float16, torch.bfloat16)
COMPLEX_DTYPES = (torch.complex64, torch.complex128)
WIDE_DTYPES = HALF_DTYPES + COMPLEX_DTYPES


def dense_dtype(dtype):
    """Type of the dense operand and of the result as the kernel sees them, for matrix values of `dtype`."""
    if dtype in HALF_DTYPES:
        return torch.float32
    if dtype in COMPLEX_DTYPES:
        return dtype
    raise TypeError(f"{dtype} has kernels of its own")


def run(prepared, operand, launch, out_shape):
    """prepared.data @ operand for a matrix of one of the four types; operand is x (1-D) or B (2-D, unit stride
    along a row) of the matrix's dtype.  Returns a new tensor of that dtype."""
    dtype = prepared.data.dtype
    dense = dense_dtype(dtype)
    o = operand if operand.dtype == dense else operand.to(dense)
    if o.ndim == 1 or o.stride(-1) != 1 or (o.shape[0] > 1 and o.stride(0) < o.shape[1]):
        o = o.contiguous()
    result = torch.empty(out_shape, dtype=dense, device=operand.device)
    launch(prepared, o, result)
    return result if dense == dtype else result.to(dtype)
