"""Shared helpers of the test-suite (oracle access, golden loading, a numpy model of the tiled kernels)."""

import glob
import json
import os

import numpy as np

from oracle import csr_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_files(kind):
    return sorted(glob.glob(os.path.join(GOLDEN, f"{kind}_*.npz")))


def golden_index():
    with open(os.path.join(GOLDEN, "index.json")) as f:
        return json.load(f)


def load_golden(path):
    g = np.load(path)
    d = {k: g[k] for k in g.files}
    d["shape"] = tuple(int(v) for v in d["shape"])
    return d


def handmade_csr(seed, row_lens, n_cols, value_dtype=np.float32, index_dtype=np.int32, indptr_dtype=np.int32,
                 sort=True, replace=False):
    """Random CSR with prescribed row lengths; unsorted and/or duplicate columns on request."""
    rng = np.random.default_rng(seed)
    indptr = np.zeros(len(row_lens) + 1, dtype=np.int64)
    indptr[1:] = np.cumsum(row_lens)
    cols = []
    for k in row_lens:
        c = rng.choice(n_cols, size=k, replace=replace or k > n_cols)
        cols.append(np.sort(c) if sort else c)
    cols = np.concatenate(cols) if cols else np.zeros(0)
    data = rng.uniform(-1, 1, size=int(indptr[-1])).astype(value_dtype)
    return data, cols.astype(index_dtype), indptr.astype(indptr_dtype)


def assert_spmv_ok(y, data, indices, indptr, shape, x, what=""):
    """y (numpy) against the float64 oracle with the stated bound 1e-5 / 1e-13 * (|A| |x|)."""
    ref, mag = O.spmv_f64(data, indices, indptr, shape, x)
    dtype = np.asarray(data).dtype
    assert y.shape == (shape[0],), f"{what}: shape {y.shape}"
    assert y.dtype == dtype, f"{what}: dtype {y.dtype}"
    ratio = O.max_bound_ratio(y, ref, mag)
    assert ratio <= O.TOL[np.dtype(dtype)], f"{what}: max |y-y_ref|/(|A||x|) = {ratio:.3e}"
    return ratio


def assert_spmm_ok(c, data, indices, indptr, shape, b, what=""):
    ref, mag = O.spmm_f64(data, indices, indptr, shape, b)
    dtype = np.asarray(data).dtype
    assert c.shape == (shape[0], b.shape[1]), f"{what}: shape {c.shape}"
    assert c.dtype == dtype, f"{what}: dtype {c.dtype}"
    ratio = O.max_bound_ratio(c, ref, mag)
    assert ratio <= O.TOL[np.dtype(dtype)], f"{what}: max |C-C_ref|/(|A||B|) = {ratio:.3e}"
    return ratio


# ---------------------------------------------------------------------------------------------------
# numpy model of the nnz-tiled kernels: same plan, same ownership rules, same carry / head / fix-up
# ---------------------------------------------------------------------------------------------------
def tile_plan_model(indptr, tile):
    indptr = np.asarray(indptr, dtype=np.int64)
    n_rows = indptr.shape[0] - 1
    nnz = int(indptr[-1])
    n_tiles = (nnz + tile - 1) // tile if nnz > 0 else 0
    plan = np.zeros(n_tiles + 1, dtype=np.int64)
    for t in range(1, n_tiles):
        plan[t] = np.searchsorted(indptr, t * tile, side="right") - 1
    plan[n_tiles] = n_rows
    plan[0] = 0
    return plan


def tiled_spmv_model(data, indices, indptr, x, tile):
    """Evaluate y the way the stream kernel + fix-up kernel do; returns (y, written_count_per_row)."""
    indptr = np.asarray(indptr, dtype=np.int64)
    n_rows = indptr.shape[0] - 1
    nnz = int(indptr[-1])
    y = np.full(n_rows, np.nan)
    written = np.zeros(n_rows, dtype=np.int64)
    if nnz == 0:
        return np.zeros(n_rows), written + 1
    plan = tile_plan_model(indptr, tile)
    n_tiles = plan.shape[0] - 1
    prod = np.asarray(data, dtype=np.float64) * np.asarray(x, dtype=np.float64)[np.asarray(indices, dtype=np.int64)]
    carry = np.full(n_tiles, np.nan)
    head = np.full(n_tiles, np.nan)
    for t in range(n_tiles):
        lo, cnt = t * tile, min(tile, nnz - t * tile)
        ra, rb = int(plan[t]), int(plan[t + 1])
        nrf = rb - ra
        off = [int(np.clip(indptr[ra + g] - lo, 0, cnt)) for g in range(nrf + 1)] + [cnt]
        head_partial = nrf > 0 and indptr[ra] - lo < 0
        for g in range(nrf + 1):
            acc = prod[lo + off[g]: lo + off[g + 1]].sum()
            if g == nrf:
                carry[t] = acc
            elif g == 0 and head_partial:
                head[t] = acc
            else:
                y[ra + g] = acc
                written[ra + g] += 1
    for t in range(1, n_tiles):
        ra, rb = int(plan[t]), int(plan[t + 1])
        if ra >= rb:
            continue
        p = int(indptr[ra])
        if p >= t * tile:
            continue
        t0 = p // tile
        y[ra] = head[t] + carry[t0:t].sum()
        written[ra] += 1
    return y, written
