"""CPU oracle for CSR SpMV / SpMM -- TEST INFRASTRUCTURE ONLY.

Nothing in the flagsparse_b200 package imports this directory; only tests/, the smoke check and the CPU
legs of bench.py do, and only as the checker or the timed CPU baseline.

What it restates (paths relative to the reference project root):
  * the reference's definition of the result, y_i = sum_p data_p * x[indices_p] over
    p in [indptr_i, indptr_{i+1}) with duplicates summed and empty rows exactly 0
    (src/flagsparse/sparse_operations/spmv_csr.py:94-120), and C[i, :] = sum_p data_p * B[indices_p, :]
    (src/flagsparse/sparse_operations/spmm_csr.py:92-134);
  * its base-path arithmetic: float32 inputs are promoted to float64, accumulated in float64 and rounded
    once to float32 (spmv_csr.py:54-55, 516-535; spmm_csr.py:548-573) -- `spmv_base` / `spmm_base`;
  * its own correctness recipe: a float64 result for float32 inputs as the yardstick
    (tests/test_spmv.py:143-174, tests/test_spmm.py:286-288) -- `spmv_f64` / `spmm_f64`, computed with
    scipy.sparse, together with the row-wise magnitude |A| |x| that the acceptance bound
    |y - y_ref| <= tol * (|A| |x|) is stated against.
Pinned by tests/test_oracle.py against tests/golden/*.npz, which hold outputs of the reference's own
Triton kernels (run under Triton's interpreter by tests/golden/make_golden.py).
"""

import numpy as np
import scipy.sparse as sp

TOL = {np.dtype(np.float32): 1e-5, np.dtype(np.float64): 1e-13}


def _csr64(data, indices, indptr, shape, absolute=False):
    # Private copies of all three arrays: some scipy operations canonicalise a matrix in place, which
    # would rewrite the caller's arrays.  A matvec sums duplicate entries as the definition asks.
    d = np.array(data, dtype=np.float64, copy=True)
    if absolute:
        np.abs(d, out=d)
    return sp.csr_matrix((d, np.array(indices, copy=True), np.array(indptr, copy=True)), shape=shape)


def spmv_f64(data, indices, indptr, shape, x):
    """(y_ref, magnitude): float64 product and |A| |x|, both length n_rows."""
    x64 = np.asarray(x, dtype=np.float64)
    y = _csr64(data, indices, indptr, shape) @ x64
    mag = _csr64(data, indices, indptr, shape, absolute=True) @ np.abs(x64)
    return np.asarray(y).reshape(-1), np.asarray(mag).reshape(-1)


def spmm_f64(data, indices, indptr, shape, b):
    """(C_ref, magnitude): float64 product and |A| |B|, both (n_rows, n_dense)."""
    b64 = np.asarray(b, dtype=np.float64)
    if b64.shape[1] == 0:
        z = np.zeros((shape[0], 0))
        return z, z
    c = _csr64(data, indices, indptr, shape) @ b64
    mag = _csr64(data, indices, indptr, shape, absolute=True) @ np.abs(b64)
    return np.asarray(c), np.asarray(mag)


def spmv_base(data, indices, indptr, shape, x):
    """The reference's base path: float64 accumulate, one rounding to the input dtype."""
    y, _ = spmv_f64(data, indices, indptr, shape, x)
    return y.astype(np.asarray(data).dtype)


def spmm_base(data, indices, indptr, shape, b):
    c, _ = spmm_f64(data, indices, indptr, shape, b)
    return c.astype(np.asarray(data).dtype)


def spmv_rowloop(data, indices, indptr, shape, x, acc_dtype=None):
    """Plain-Python row loop of the definition (small cases only); accumulates in `acc_dtype`
    (default: the value dtype, i.e. the reference's opt path, spmv_csr.py:161-279)."""
    data, indices, indptr, x = map(np.asarray, (data, indices, indptr, x))
    acc_dtype = np.dtype(acc_dtype or data.dtype)
    y = np.zeros(shape[0], dtype=data.dtype)
    for i in range(shape[0]):
        acc = acc_dtype.type(0)
        for p in range(int(indptr[i]), int(indptr[i + 1])):
            acc = acc_dtype.type(acc + acc_dtype.type(data[p]) * acc_dtype.type(x[int(indices[p])]))
        y[i] = acc
    return y


def sddmm_f64(data, indices, indptr, x, y, alpha=1.0, beta=0.0):
    """(out_ref, magnitude) of out[p] = alpha * dot(x[row(p)], y[col(p)]) + beta * data[p] in float64, and
    |alpha| * dot(|x[row]|, |y[col]|) + |beta| * |data[p]| -- the definition the reference's kernel implements
    (src/flagsparse/sparse_operations/sddmm_csr.py:107-152) and checks itself against (:424-440)."""
    indptr = np.asarray(indptr, dtype=np.int64)
    rows = np.repeat(np.arange(indptr.shape[0] - 1), np.diff(indptr))
    cols = np.asarray(indices, dtype=np.int64)
    x64, y64 = np.asarray(x, dtype=np.float64), np.asarray(y, dtype=np.float64)
    out = alpha * np.einsum("pk,pk->p", x64[rows], y64[cols])
    mag = abs(alpha) * np.einsum("pk,pk->p", np.abs(x64[rows]), np.abs(y64[cols]))
    if data is not None:
        d64 = np.asarray(data, dtype=np.float64)
        out = out + beta * d64
        mag = mag + abs(beta) * np.abs(d64)
    return out, mag


def max_bound_ratio(got, ref, mag):
    """max_i |got_i - ref_i| / mag_i with 0/0 = 0: the quantity the acceptance bound limits by `tol`."""
    got = np.asarray(got, dtype=np.float64)
    err = np.abs(got - ref)
    with np.errstate(divide="ignore", invalid="ignore"):
        ratio = np.where(mag > 0, err / mag, np.where(err > 0, np.inf, 0.0))
    return float(ratio.max()) if ratio.size else 0.0


def within_bound(got, ref, mag, dtype):
    """|got - ref| <= tol * mag element-wise, tol = 1e-5 (float32) or 1e-13 (float64)."""
    return max_bound_ratio(got, ref, mag) <= TOL[np.dtype(dtype)]
