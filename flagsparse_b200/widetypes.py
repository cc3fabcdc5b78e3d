"""float16, bfloat16, complex64 and complex128 values through the float32 / float64 kernels.

The reference's base paths take these four value types by computing in a wider real type and casting back:
half precisions run its float32 kernel on `data.to(float32)` and `x.to(float32)` and round the result
(src/flagsparse/sparse_operations/spmv_csr.py:496-535, spmm_csr.py:525-560 of the reference), complex values run a
kernel over the interleaved real view (spmv_csr.py:123-155, 536-554; spmm_csr.py:138-195).  Here the same results
come from the real kernels of this package without new device code:
  * float16 / bfloat16: one float32 copy of the values made at prepare time, x (or B) widened per call, the
    float32 result rounded once to the caller's type;
  * complex: the values split into a real and an imaginary matrix at prepare time (same indices), and
        Re y = A_re x_re - A_im x_im,   Im y = A_re x_im + A_im x_re
    as four real products per call, in the component precision (float32 for complex64, float64 for complex128).
The functions below hold the arithmetic only; the caller passes `launch(part, operand, result)`, which is the CUDA
launch in the package and a host stand-in in the tests of this module.
"""

import torch

HALF_DTYPES = (torch.float16, torch.bfloat16)
COMPLEX_DTYPES = (torch.complex64, torch.complex128)
WIDE_DTYPES = HALF_DTYPES + COMPLEX_DTYPES


def compute_dtype(dtype):
    """The real type the kernels run in for values of `dtype`."""
    if dtype in HALF_DTYPES:
        return torch.float32
    if dtype == torch.complex64:
        return torch.float32
    if dtype == torch.complex128:
        return torch.float64
    return dtype


def split_values(data):
    """(kind, real value arrays) of a value array: ('cast', [float32 copy]) or ('complex', [re, im])."""
    if data.dtype in HALF_DTYPES:
        return "cast", [data.to(torch.float32)]
    if data.dtype in COMPLEX_DTYPES:
        ri = torch.view_as_real(data.contiguous())
        return "complex", [ri[..., 0].contiguous(), ri[..., 1].contiguous()]
    raise TypeError(f"{data.dtype} needs no widening")


def _split_operand(v):
    ri = torch.view_as_real(v.contiguous())
    return ri[..., 0].contiguous(), ri[..., 1].contiguous()


def product(kind, parts, operand, launch, out_shape, dtype):
    """A @ operand for a matrix held as `parts` (see split_values); operand is x (1-D) or B (2-D) of the caller's
    dtype.  launch(part, real operand, real result) must fill `result` with part @ operand."""
    dev = operand.device
    comp = compute_dtype(dtype)
    if kind == "cast":
        y = torch.empty(out_shape, dtype=comp, device=dev)
        launch(parts[0], operand.to(comp).contiguous(), y)
        return y.to(dtype)
    if kind == "complex":
        o_re, o_im = _split_operand(operand)
        t = [torch.empty(out_shape, dtype=comp, device=dev) for _ in range(4)]
        launch(parts[0], o_re, t[0])
        launch(parts[1], o_im, t[1])
        launch(parts[0], o_im, t[2])
        launch(parts[1], o_re, t[3])
        return torch.complex(t[0] - t[1], t[2] + t[3])
    raise ValueError(f"unknown kind {kind!r}")
