"""Matrix Market (.mtx) coordinate files -> CSR tensors for the SpMV / SpMM entry points.

Same name, arguments and result as the loader the reference's benchmark scripts use
(tests/test_spmv.py:29-103 and tests/test_spmm.py:163-268 of the reference: load_mtx_to_csr_torch):
  * `pattern` files get the value 1 for every entry; `integer` files are read as reals;
  * `symmetric`, `hermitian` and `skew-symmetric` files are expanded (an off-diagonal entry (r, c, v) also gives
    (c, r, v), or (c, r, -v) for skew-symmetric) when the mirrored position lies inside the matrix;
  * only the first `nnz` data lines count; entries outside the matrix are dropped;
  * entries that land on the same (row, column) are summed, in file order and in double precision;
  * columns come out sorted inside each row; column indices and the row pointer are int64.
The reference walks the file entry by entry through Python dictionaries; this loader parses the entries with
numpy's text reader and does the same arithmetic with arrays (one stable sort).  Complex files are refused: the
kernels here take float32 and float64 values.
"""

import numpy as np
import torch

_FIELDS = ("real", "integer", "pattern", "complex", "double")
_SYMMETRIES = ("general", "symmetric", "skew-symmetric", "hermitian")


def _parse(file_path):
    """(field, symmetry, n_rows, n_cols, nnz, rows, cols, vals) with 0-based rows/cols of the first nnz data lines."""
    field, symmetry = "real", "general"
    size = None
    data_lines = []
    with open(file_path, "r", encoding="utf-8") as handle:
        for line in handle:
            stripped = line.strip()
            if stripped.startswith("%%MatrixMarket"):
                tokens = stripped.split()
                if len(tokens) >= 3 and tokens[2].lower() != "coordinate":
                    raise ValueError(f"only coordinate Matrix Market files are supported, got {tokens[2]!r}: {file_path}")
                if len(tokens) >= 5:
                    field, symmetry = tokens[3].lower(), tokens[4].lower()
                continue
            if stripped.startswith("%") or not stripped:
                continue
            if size is None:
                parts = stripped.split()
                size = (int(parts[0]), int(parts[1]), int(parts[2]) if len(parts) > 2 else 0)
                continue
            data_lines.append(stripped)
    if size is None:
        raise ValueError(f"Cannot parse .mtx header: {file_path}")
    n_rows, n_cols, nnz = size
    data_lines = data_lines[:nnz]
    is_pattern = field == "pattern"
    if field == "complex":
        raise TypeError(f"Matrix Market file {file_path} stores complex values; float32/float64 only here")
    rows, cols, vals = _parse_entries(data_lines, is_pattern)
    return field, symmetry, n_rows, n_cols, nnz, rows, cols, vals


def _parse_entries(data_lines, is_pattern):
    """0-based rows and columns and float64 values of the data lines.  numpy's text reader takes the regular case
    (every line with the same number of fields); anything else goes line by line, which also finds the line to
    name in an error."""
    if not data_lines:
        return np.zeros(0, dtype=np.int64), np.zeros(0, dtype=np.int64), np.zeros(0, dtype=np.float64)
    try:
        table = np.loadtxt(data_lines, dtype=np.float64, ndmin=2, comments=None)
        if table.shape[0] == len(data_lines) and table.shape[1] >= (2 if is_pattern else 3):
            rows = table[:, 0].astype(np.int64) - 1
            cols = table[:, 1].astype(np.int64) - 1
            vals = np.ones(len(data_lines), dtype=np.float64) if is_pattern else np.ascontiguousarray(table[:, 2])
            if np.array_equal(rows + 1, table[:, 0]) and np.array_equal(cols + 1, table[:, 1]):
                return rows, cols, vals
    except ValueError:
        pass
    rows = np.empty(len(data_lines), dtype=np.int64)
    cols = np.empty(len(data_lines), dtype=np.int64)
    vals = np.ones(len(data_lines), dtype=np.float64)
    for k, line in enumerate(data_lines):
        parts = line.split()
        if len(parts) < 2:
            rows[k] = cols[k] = -1          # dropped later, like any entry outside the matrix
            continue
        rows[k] = int(parts[0]) - 1
        cols[k] = int(parts[1]) - 1
        if not is_pattern:
            if len(parts) < 3:
                raise ValueError(f"Matrix Market entry is missing a numeric value: {line}")
            vals[k] = float(parts[2])
    return rows, cols, vals


def mtx_to_csr_arrays(file_path):
    """numpy CSR (float64 data, int64 indices, int64 indptr, shape) of a Matrix Market coordinate file."""
    field, symmetry, n_rows, n_cols, nnz, rows, cols, vals = _parse(file_path)
    indptr = np.zeros(n_rows + 1, dtype=np.int64)
    if nnz == 0 or rows.size == 0:
        return np.zeros(0, dtype=np.float64), np.zeros(0, dtype=np.int64), indptr, (n_rows, n_cols)
    inside = (rows >= 0) & (rows < n_rows) & (cols >= 0) & (cols < n_cols)
    rows, cols, vals = rows[inside], cols[inside], vals[inside]
    mirror = symmetry in ("symmetric", "hermitian", "skew-symmetric")
    if mirror:
        # entry k sits at position 2k, its mirror image at 2k + 1: a stable sort then keeps the file order
        twin = (rows != cols) & (cols < n_rows) & (rows < n_cols)
        r2 = np.stack([rows, cols], axis=1).reshape(-1)
        c2 = np.stack([cols, rows], axis=1).reshape(-1)
        v2 = np.stack([vals, -vals if symmetry == "skew-symmetric" else vals], axis=1).reshape(-1)
        keep = np.stack([np.ones_like(twin), twin], axis=1).reshape(-1)
        rows, cols, vals = r2[keep], c2[keep], v2[keep]
    if rows.size == 0:
        return np.zeros(0, dtype=np.float64), np.zeros(0, dtype=np.int64), indptr, (n_rows, n_cols)
    key = rows * np.int64(max(n_cols, 1)) + cols
    order = np.argsort(key, kind="stable")
    key, vals = key[order], vals[order]
    first = np.ones(key.size, dtype=bool)
    first[1:] = key[1:] != key[:-1]
    starts = np.flatnonzero(first)
    data = np.add.reduceat(vals, starts)           # left to right inside each (row, column): the file order
    ukey = key[starts]
    out_rows = ukey // max(n_cols, 1)
    indices = ukey - out_rows * max(n_cols, 1)
    indptr[1:] = np.cumsum(np.bincount(out_rows, minlength=n_rows))
    return data, indices.astype(np.int64), indptr, (n_rows, n_cols)


def load_mtx_to_csr_torch(file_path, dtype=torch.float32, device=None):
    """Load a SuiteSparse / Matrix Market .mtx file into CSR torch tensors: (data, indices, indptr, shape), on
    `device` (default: the GPU when there is one)."""
    if dtype not in (torch.float32, torch.float64):
        raise TypeError("dtype must be torch.float32 or torch.float64")
    if device is None:
        device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    data, indices, indptr, shape = mtx_to_csr_arrays(file_path)
    return (torch.from_numpy(data).to(dtype).to(device), torch.from_numpy(indices).to(device),
            torch.from_numpy(indptr).to(device), shape)
