"""Seeded synthetic CSR matrices for the benchmark configurations, on the host (numpy) or on a GPU (torch).

Every quantity is a pure function of (seed, row, position) through a 64-bit integer mix, computed with
wrap-around int64 arithmetic that numpy and torch implement identically.  Consequences:
  * the numpy generator and the torch generator produce bit-identical matrices, so a matrix generated on
    the GPU can be checked against a host oracle that regenerates only a few row blocks;
  * any row range can be generated on its own (row shards of the multi-GPU driver, sampled checks).
Row lengths and columns are drawn with integer comparisons and integer modulo only -- no floating point
takes part in the structure.

The reference has no seeded generator (its _build_random_csr, src/flagsparse/sparse_operations/_common.py:
166-181, uses unseeded torch.randint); the shapes and distributions here are the ones the benchmark
configurations name.
"""

import math
from dataclasses import dataclass, replace
from functools import lru_cache

import numpy as np

try:  # torch is needed only for the GPU twin
    import torch
except ImportError:  # pragma: no cover
    torch = None

_MASK64 = (1 << 64) - 1


def _s64(v):
    """Python int -> the same 64 bits as a signed int64 value."""
    v &= _MASK64
    return v - (1 << 64) if v >= (1 << 63) else v


_M1 = _s64(0xBF58476D1CE4E5B9)
_M2 = _s64(0x94D049BB133111EB)
_GOLD = _s64(0x9E3779B97F4A7C15)
_KMUL = _s64(0xD1B54A32D192ED03)

TAG_LEN, TAG_COL, TAG_VAL, TAG_X, TAG_B = 1, 2, 3, 4, 5


def _lsr(z, s):
    """Logical right shift of int64 lanes (both libraries shift arithmetically)."""
    return (z >> s) & ((1 << (64 - s)) - 1)


def _mix(z):
    """splitmix64 finaliser on int64 lanes (array of either library)."""
    z = (z ^ _lsr(z, 30)) * _M1
    z = (z ^ _lsr(z, 27)) * _M2
    return z ^ _lsr(z, 31)


def _mix_int(z):
    """Same finaliser on one Python int."""
    z &= _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    return z ^ (z >> 31)


def _stream_base(seed, tag):
    return _s64(_mix_int(seed * 0x9E3779B97F4A7C15 + tag))


def _hash2(base, a, b):
    """64-bit hash of the integer pair (a, b) in stream `base`; a and b are int64 arrays."""
    return _mix(_mix(a * _GOLD + base) + b * _KMUL)


# ---------------------------------------------------------------------------------------------------
# the two array backends
# ---------------------------------------------------------------------------------------------------
class _NumpyOps:
    name = "numpy"

    def arange(self, a, b=None):
        return np.arange(a, b, dtype=np.int64) if b is not None else np.arange(a, dtype=np.int64)

    def asarray_i64(self, a):
        return np.asarray(a, dtype=np.int64)

    def repeat(self, x, counts):
        return np.repeat(x, counts)

    def cumsum0(self, counts):
        out = np.zeros(counts.shape[0] + 1, dtype=np.int64)
        np.cumsum(counts, out=out[1:])
        return out

    def searchsorted_right(self, table, v):
        return np.searchsorted(table, v, side="right").astype(np.int64)

    def sort(self, x):
        return np.sort(x)

    def argsort_stable(self, x):
        return np.argsort(x, kind="stable")

    def clip(self, x, lo, hi):
        return np.clip(x, lo, hi)

    def bincount(self, x, n):
        return np.bincount(x, minlength=n).astype(np.int64)

    def keep_mask_unique_sorted(self, x):
        m = np.ones(x.shape[0], dtype=bool)
        if x.shape[0] > 1:
            m[1:] = x[1:] != x[:-1]
        return m

    def to_f32(self, i24):
        return (i24.astype(np.float32) * np.float32(2.0**-23)) - np.float32(1.0)

    def to_f64(self, i53):
        return (i53.astype(np.float64) * (2.0**-52)) - 1.0

    def cast(self, x, dtype):
        return x.astype(_np_dtype(dtype))

    def concat(self, xs, dtype):
        return np.concatenate(xs) if xs else np.zeros(0, dtype=_np_dtype(dtype))

    def cumsum_rows_lt(self, m):  # running count along axis 1
        return np.cumsum(m, axis=1)

    def lower_triangle(self, m):  # [j, i] true for i < j
        return np.tril(np.ones((m, m), dtype=bool), -1)


class _TorchOps:
    name = "torch"

    def __init__(self, device):
        self.device = torch.device(device)

    def arange(self, a, b=None):
        if b is None:
            return torch.arange(a, dtype=torch.int64, device=self.device)
        return torch.arange(a, b, dtype=torch.int64, device=self.device)

    def asarray_i64(self, a):
        return torch.as_tensor(np.asarray(a, dtype=np.int64), device=self.device)

    def repeat(self, x, counts):
        return torch.repeat_interleave(x, counts)

    def cumsum0(self, counts):
        out = torch.zeros(counts.shape[0] + 1, dtype=torch.int64, device=self.device)
        torch.cumsum(counts, dim=0, out=out[1:])
        return out

    def searchsorted_right(self, table, v):
        return torch.searchsorted(table, v, right=True)

    def sort(self, x):
        return torch.sort(x).values

    def argsort_stable(self, x):
        return torch.sort(x, stable=True).indices

    def clip(self, x, lo, hi):
        return torch.clamp(x, lo, hi)

    def bincount(self, x, n):
        return torch.bincount(x, minlength=n)

    def keep_mask_unique_sorted(self, x):
        m = torch.ones(x.shape[0], dtype=torch.bool, device=self.device)
        if x.shape[0] > 1:
            m[1:] = x[1:] != x[:-1]
        return m

    def to_f32(self, i24):
        return i24.to(torch.float32) * (2.0**-23) - 1.0

    def to_f64(self, i53):
        return i53.to(torch.float64) * (2.0**-52) - 1.0

    def cast(self, x, dtype):
        return x.to(_torch_dtype(dtype))

    def concat(self, xs, dtype):
        if not xs:
            return torch.zeros(0, dtype=_torch_dtype(dtype), device=self.device)
        return torch.cat(xs)

    def cumsum_rows_lt(self, m):
        return torch.cumsum(m.to(torch.int64), dim=1)

    def lower_triangle(self, m):
        return torch.tril(torch.ones((m, m), dtype=torch.bool, device=self.device), -1)


def _np_dtype(name):
    return {"float32": np.float32, "float64": np.float64, "int32": np.int32, "int64": np.int64}[name]


def _torch_dtype(name):
    return {"float32": torch.float32, "float64": torch.float64, "int32": torch.int32, "int64": torch.int64}[name]


def _ops(device):
    return _NumpyOps() if device is None or device == "numpy" else _TorchOps(device)


# ---------------------------------------------------------------------------------------------------
# specification of a matrix
# ---------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class CsrSpec:
    """A synthetic CSR matrix: shape, row-length law, column law, whether duplicate columns are merged."""

    name: str
    n_rows: int
    n_cols: int
    lengths: tuple  # ("const", k) | ("poisson", mean) | ("zipf", alpha, max_len, target_nnz)
    columns: tuple  # ("band", half_width) | ("uniform",) | ("distinct",)
    dedup: bool
    seed: int = 0

    def scaled(self, n_rows, name=None):
        """The same laws on a smaller (or larger) square matrix -- used by tests to shrink a config."""
        lengths = self.lengths
        if lengths[0] == "zipf":
            lengths = (lengths[0], lengths[1], min(lengths[2], n_rows), int(lengths[3] * n_rows / self.n_rows))
        columns = self.columns
        if columns[0] == "band":
            columns = ("band", max(1, min(columns[1], (n_rows - 1) // 2)))
        return replace(self, name=name or f"{self.name}@{n_rows}", n_rows=n_rows, n_cols=n_rows, lengths=lengths,
                       columns=columns)


def config_spec(config, seed=0):
    """The five benchmark configurations: 'c1' .. 'c5'."""
    c = config.lower()
    if c == "c1":  # 4096^2, exactly 16 distinct sorted columns per row
        return CsrSpec("c1", 4096, 4096, ("const", 16), ("distinct",), False, seed)
    if c == "c2":  # 2^22 rows, Poisson(32) row lengths, band of +-2^16, sorted and deduplicated
        return CsrSpec("c2", 1 << 22, 1 << 22, ("poisson", 32.0), ("band", 1 << 16), True, seed)
    if c == "c3":  # 2^24 rows, Zipf(2) row lengths clipped to [1, 2^17] scaled to ~256M nnz, uniform columns
        return CsrSpec("c3", 1 << 24, 1 << 24, ("zipf", 2.0, 1 << 17, 256_000_000), ("uniform",), True, seed)
    if c == "c4":  # 2^20 rows, exactly 16 sorted uniform columns per row (duplicates kept)
        return CsrSpec("c4", 1 << 20, 1 << 20, ("const", 16), ("uniform",), False, seed)
    if c == "c5":  # 2^26 rows, Poisson(32), band of +-2^20, sorted, duplicates kept (lengths known up front)
        return CsrSpec("c5", 1 << 26, 1 << 26, ("poisson", 32.0), ("band", 1 << 20), False, seed)
    raise ValueError(f"unknown config {config!r}")


# ---------------------------------------------------------------------------------------------------
# row lengths
# ---------------------------------------------------------------------------------------------------
@lru_cache(maxsize=None)
def _poisson_thresholds(mean):
    """floor(cdf(k) * 2^53) for k = 0.. until the cdf saturates (host table, int64)."""
    out, p, cdf, k = [], math.exp(-mean), 0.0, 0
    while True:
        cdf += p
        out.append(min(int(cdf * (1 << 53)), (1 << 53) - 1))
        k += 1
        p *= mean / k
        if (1.0 - cdf) < 2.0**-54 or k > 100000:
            break
    out[-1] = (1 << 53)  # u53 < 2^53 always lands at or below the last length
    return np.asarray(out, dtype=np.int64)


@lru_cache(maxsize=None)
def _zipf_table(alpha, max_len, target_nnz, n_rows):
    """(thresholds, scale_q16): inverse-cdf table of pmf ~ k^-alpha on [1, max_len] and the fixed-point
    factor that brings the expected total to target_nnz."""
    k = np.arange(1, max_len + 1, dtype=np.float64)
    pmf = k ** (-alpha)
    pmf /= pmf.sum()
    cdf = np.cumsum(pmf)
    thr = np.minimum((cdf * float(1 << 53)).astype(np.int64), (1 << 53) - 1)
    thr[-1] = 1 << 53
    mean = float((k * pmf).sum())
    scale_q16 = max(1, int(round(target_nnz / (n_rows * mean) * 65536.0)))
    return thr, scale_q16


def row_lengths(spec, ops, r0, r1):
    """Row lengths BEFORE deduplication for rows [r0, r1), int64 array of the backend."""
    rows = ops.arange(r0, r1)
    kind = spec.lengths[0]
    if kind == "const":
        return rows * 0 + int(spec.lengths[1])
    u53 = _lsr(_hash2(_stream_base(spec.seed, TAG_LEN), rows, rows * 0), 11)
    if kind == "poisson":
        table = ops.asarray_i64(_poisson_thresholds(float(spec.lengths[1])))
        n = ops.searchsorted_right(table, u53)
        if spec.columns[0] == "band":
            n = ops.clip(n, 0, 2 * spec.columns[1] + 1)
        return n
    if kind == "zipf":
        _, alpha, max_len, target = spec.lengths
        thr, scale_q16 = _zipf_table(float(alpha), int(max_len), int(target), int(spec.n_rows))
        raw = ops.searchsorted_right(ops.asarray_i64(thr), u53) + 1
        scaled = (raw * scale_q16 + 32768) >> 16
        return ops.clip(scaled, 1, min(int(max_len), spec.n_cols))
    raise ValueError(kind)


# ---------------------------------------------------------------------------------------------------
# one block of rows
# ---------------------------------------------------------------------------------------------------
def _block(spec, ops, r0, r1):
    """Rows [r0, r1): returns (columns sorted within each row, per-row counts)."""
    n = r1 - r0
    if spec.columns[0] == "distinct":
        k = int(spec.lengths[1])
        m = 2 * k  # candidates per row; the first k distinct ones in draw order are kept
        flat = ops.arange(n * m)
        rloc = flat // m
        pos = flat % m
        cand = _lsr(_hash2(_stream_base(spec.seed, TAG_COL), rloc + r0, pos), 1) % spec.n_cols
        cand2 = cand.reshape(n, m)
        # dup[i, j]: candidate j of row i repeats an earlier candidate of the same row
        eq = cand2.reshape(n, m, 1) == cand2.reshape(n, 1, m)
        earlier = ops.lower_triangle(m)
        dup = (eq & earlier.reshape(1, m, m)).sum(2) > 0
        fresh = ~dup
        keep = (fresh & (ops.cumsum_rows_lt(fresh) <= k)).reshape(n * m)
        if int(keep.sum()) != n * k:  # 2k draws from thousands of columns: practically impossible
            raise RuntimeError("distinct-column draw ran out of candidates")
        key = ops.sort(rloc[keep] * (1 << 32) + cand[keep])
        return key & 0xFFFFFFFF, rloc[:n] * 0 + k

    lens = row_lengths(spec, ops, r0, r1)
    start = ops.cumsum0(lens)
    total = int(start[-1])
    rloc = ops.repeat(ops.arange(n), lens)
    pos = ops.arange(total) - start[rloc]
    rows = rloc + r0
    h = _lsr(_hash2(_stream_base(spec.seed, TAG_COL), rows, pos), 1)
    if spec.columns[0] == "band":
        w = int(spec.columns[1])
        span = 2 * w + 1
        lo = ops.clip(rows - w, 0, spec.n_cols - span)
        cols = lo + h % span
    else:
        cols = h % spec.n_cols
    key = ops.sort(rloc * (1 << 32) + cols)
    if spec.dedup:
        key = key[ops.keep_mask_unique_sorted(key)]
        lens = ops.bincount(key >> 32, n)
    return key & 0xFFFFFFFF, lens


def _values(spec, ops, r0, lens, value_dtype):
    n = lens.shape[0]
    start = ops.cumsum0(lens)
    total = int(start[-1])
    rloc = ops.repeat(ops.arange(n), lens)
    pos = ops.arange(total) - start[rloc]
    h = _hash2(_stream_base(spec.seed, TAG_VAL), rloc + r0, pos)
    if value_dtype == "float32":
        return ops.to_f32(_lsr(h, 40))
    return ops.to_f64(_lsr(h, 11))


def generate_csr(spec, device=None, value_dtype="float32", index_dtype="int32", indptr_dtype="int32",
                 row_range=None, chunk_nnz=1 << 26):
    """Rows `row_range` (default: all) of the matrix as (data, indices, indptr) with indptr[0] == 0.
    `device` None/"numpy" gives numpy arrays, anything else torch tensors on that device."""
    ops = _ops(device)
    r_begin, r_end = (0, spec.n_rows) if row_range is None else (int(row_range[0]), int(row_range[1]))
    mean = {"const": lambda: spec.lengths[1], "poisson": lambda: spec.lengths[1],
            "zipf": lambda: max(1.0, spec.lengths[3] / spec.n_rows)}[spec.lengths[0]]()
    rows_per_chunk = max(1, min(1 << 22, int(chunk_nnz / max(mean, 1.0))))
    if spec.columns[0] == "distinct":
        rows_per_chunk = min(rows_per_chunk, 8192)
    datas, idxs, counts = [], [], []
    for c0 in range(r_begin, r_end, rows_per_chunk):
        c1 = min(r_end, c0 + rows_per_chunk)
        cols, lens = _block(spec, ops, c0, c1)
        datas.append(_values(spec, ops, c0, lens, value_dtype))
        idxs.append(ops.cast(cols, index_dtype))
        counts.append(lens)
    lens_all = ops.concat(counts, "int64")
    indptr = ops.cast(ops.cumsum0(lens_all), indptr_dtype)
    return ops.concat(datas, value_dtype), ops.concat(idxs, index_dtype), indptr


def dense_vector(spec_or_seed, n, device=None, value_dtype="float32", tag=TAG_X, n_dense=None, row_range=None):
    """x (n,) or, with n_dense, a row-major B (n, n_dense): uniform in [-1, 1), a pure function of
    (seed, row, column)."""
    seed = spec_or_seed.seed if isinstance(spec_or_seed, CsrSpec) else int(spec_or_seed)
    ops = _ops(device)
    r0, r1 = (0, n) if row_range is None else row_range
    if n_dense is None:
        rows = ops.arange(r0, r1)
        h = _hash2(_stream_base(seed, tag), rows, rows * 0)
    else:
        flat = ops.arange(r0 * n_dense, r1 * n_dense)
        h = _hash2(_stream_base(seed, TAG_B), flat // n_dense, flat % n_dense)
    v = ops.to_f32(_lsr(h, 40)) if value_dtype == "float32" else ops.to_f64(_lsr(h, 11))
    return v if n_dense is None else v.reshape(r1 - r0, n_dense)
