"""Run with FSB_BOUNDS_CHECK=1 (tests/test_bounds_check_gpu.py does, in a child process): index arrays that would take
a kernel out of bounds are refused by the checking build of the library, with a record, and nothing is launched.

Every bad index used here points into memory the process owns anyway (every array sits in the middle of a larger
allocation, a bad row pointer never exceeds the spare entries, a bad x slot of a panel layout lands in the
accumulators behind the x buffers), so no case depends on the check for its memory safety.
"""

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from flagsparse_b200 import _lib, panel  # noqa: E402
from flagsparse_b200 import synthetic as S  # noqa: E402
from helpers import assert_spmv_ok  # noqa: E402

DEV = "cuda:0"
SLACK = 64


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def roomy(a):
    """The array on the device in the middle of an allocation with SLACK spare rows on either side (zeros).
    Returns (allocation, view of the array); the view keeps the allocation alive."""
    a = np.ascontiguousarray(a)
    big = torch.zeros((a.shape[0] + 2 * SLACK,) + a.shape[1:], dtype=torch.from_numpy(a).dtype, device=DEV)
    big[SLACK:SLACK + a.shape[0]] = torch.from_numpy(a).to(DEV)
    return big, big[SLACK:SLACK + a.shape[0]]


def expect_refusal(rc, kind, where, value, limit, what):
    assert rc == _lib.FSB_EBOUNDS, f"{what}: return code {rc}"
    seen, k, w, v, lim = _lib.bounds_report()
    assert (seen, k, w, v, lim) == (1, kind, where, value, limit), f"{what}: report {(seen, k, w, v, lim)}"
    assert _lib.bounds_report() == (0, 0, 0, 0, 0), f"{what}: the report is cleared by reading it"
    print(f"refused as expected: {what}")


def main():
    L = _lib.lib()
    assert _lib.CHECKING and L.fsb_bounds_check_enabled() == 1, "not the checking build"
    st = torch.cuda.current_stream().cuda_stream
    F32, I32 = _lib.FSB_F32, _lib.FSB_I32
    spec = S.config_spec("c2").scaled(3000)
    data, idx, ptr = S.generate_csr(spec, None)
    x = S.dense_vector(spec, spec.n_cols)
    n_rows, n_cols, nnz = spec.n_rows, spec.n_cols, data.size
    _, d = roomy(data)
    _, xd = roomy(x)
    y = torch.full((n_rows,), 7.0, dtype=torch.float32, device=DEV)

    def spmv(i_t, p_t):
        return L.fsb_spmv_csr(F32, I32, I32, d.data_ptr(), i_t.data_ptr(), p_t.data_ptr(), xd.data_ptr(), y.data_ptr(),
                              n_rows, n_cols, nnz, _lib.FSB_SPMV_VECTOR, 0, None, None, 0, st)

    # ---- SpMV: a column index past n_cols, a negative one, row pointers past nnz and out of order
    _, i_good = roomy(idx)
    _, p_good = roomy(ptr)
    where = nnz // 2
    for bad in (n_cols + 5, -1):
        bad_idx = idx.copy()
        bad_idx[where] = bad
        _, i_bad = roomy(bad_idx)
        rc = spmv(i_bad, p_good)
        expect_refusal(rc, 1, where, bad, n_cols, f"SpMV column {bad}")
        torch.cuda.synchronize()
        assert bool((y == 7.0).all()), "a refused call writes nothing"
    bad_ptr = ptr.copy()
    bad_ptr[-1] = nnz + 3                                 # three more entries than there are: inside the allocation
    rc = spmv(i_good, roomy(bad_ptr)[1])
    expect_refusal(rc, 2, n_rows, nnz + 3, nnz, "SpMV last row pointer past nnz")
    bad_ptr = ptr.copy()
    r = n_rows // 3
    bad_ptr[r] = bad_ptr[r - 1] - 1 if bad_ptr[r - 1] > 0 else 0
    if bad_ptr[r] < bad_ptr[r - 1]:
        rc = spmv(i_good, roomy(bad_ptr)[1])
        expect_refusal(rc, 3, r, int(bad_ptr[r]), int(bad_ptr[r - 1]), "SpMV row pointer out of order")
    # the context is intact: the same call with the good arrays computes the product
    assert spmv(i_good, p_good) == 0
    torch.cuda.synchronize()
    assert_spmv_ok(y.cpu().numpy(), data, idx, ptr, (n_rows, n_cols), x, what="after the refusals")
    assert _lib.bounds_report() == (0, 0, 0, 0, 0)

    # ---- the Python error path
    try:
        _lib.check(spmv(roomy(np.where(np.arange(nnz) == 7, n_cols, idx).astype(np.int32))[1], p_good), "fsb_spmv_csr")
    except IndexError as e:
        assert "position 7" in str(e) and f"limit {n_cols}" in str(e), str(e)
        print("IndexError:", e)
    else:
        raise AssertionError("no IndexError")

    # ---- SpMM: the same walk in front of the tile kernel (B has SLACK spare rows)
    n_dense = 8
    Bh = np.random.default_rng(3).uniform(-1, 1, (n_cols, n_dense)).astype(np.float32)
    _, B = roomy(Bh)
    C = torch.full((n_rows, n_dense), 7.0, dtype=torch.float32, device=DEV)
    T = L.fsb_spmm_tile_nnz(F32)
    n_tiles = L.fsb_csr_num_tiles(nnz, T)
    plan = torch.empty(n_tiles + 1, dtype=torch.int32, device=DEV)
    assert L.fsb_csr_tile_plan(I32, p_good.data_ptr(), n_rows, nnz, T, plan.data_ptr(), st) == 0
    nbytes = L.fsb_spmm_csr_scratch_bytes(F32, nnz, n_dense)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    bad_idx = idx.copy()
    bad_idx[11] = n_cols + 1
    _, i_bad = roomy(bad_idx)

    def spmm(i_t):
        return L.fsb_spmm_csr(F32, I32, I32, d.data_ptr(), i_t.data_ptr(), p_good.data_ptr(), B.data_ptr(), n_dense,
                              C.data_ptr(), n_dense, n_rows, n_cols, n_dense, nnz, _lib.FSB_SPMM_AUTO, plan.data_ptr(),
                              scratch.data_ptr(), nbytes, None, st)

    expect_refusal(spmm(i_bad), 1, 11, n_cols + 1, n_cols, "SpMM column past n_cols")
    torch.cuda.synchronize()
    assert bool((C == 7.0).all())
    assert spmm(i_good) == 0
    torch.cuda.synchronize()
    want = torch.sparse_csr_tensor(dev(ptr.astype(np.int64)), dev(idx.astype(np.int64)), dev(data.astype(np.float64)),
                                   size=(n_rows, n_cols)) @ dev(Bh.astype(np.float64))
    assert float((C.double() - want).abs().max()) < 1e-4

    # ---- SDDMM: row ids and column ids (X and Y have SLACK spare rows)
    K = 16
    Xh = np.random.default_rng(4).uniform(-1, 1, (n_rows, K)).astype(np.float32)
    Yh = np.random.default_rng(5).uniform(-1, 1, (n_cols, K)).astype(np.float32)
    _, X = roomy(Xh)
    _, Y = roomy(Yh)
    rows = np.repeat(np.arange(n_rows, dtype=np.int32), np.diff(ptr))
    out = torch.full((nnz,), 7.0, dtype=torch.float32, device=DEV)

    def sddmm(i_t, r_t):
        return L.fsb_sddmm_csr(F32, i_t.data_ptr(), r_t.data_ptr(), X.data_ptr(), K, Y.data_ptr(), K, None,
                               out.data_ptr(), n_rows, n_cols, nnz, K, 1.0, 0.0, st)

    bad_rows = rows.copy()
    bad_rows[nnz - 1] = n_rows + 2
    expect_refusal(sddmm(i_good, roomy(bad_rows)[1]), 4, nnz - 1, n_rows + 2, n_rows, "SDDMM row id past n_rows")
    expect_refusal(sddmm(i_bad, roomy(rows)[1]), 1, 11, n_cols + 1, n_cols, "SDDMM column past n_cols")
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())
    assert sddmm(i_good, roomy(rows)[1]) == 0
    torch.cuda.synchronize()
    want = (Xh.astype(np.float64)[rows] * Yh.astype(np.float64)[idx]).sum(axis=1)
    assert float(np.abs(out.cpu().numpy() - want).max()) < 1e-4

    # ---- a panel layout whose packed word points past the x buffers (it would read an accumulator instead)
    lay = panel.build_panel_layout(dev(data), dev(idx), dev(ptr), n_rows, n_cols, int(np.diff(ptr).max()), force=True)
    assert lay is not None
    xp = dev(x)
    yp = torch.full((n_rows,), 7.0, dtype=torch.float32, device=DEV)
    panel.launch_panel(lay, xp, yp, n_rows, n_cols, st)
    torch.cuda.synchronize()
    assert_spmv_ok(yp.cpu().numpy(), data, idx, ptr, (n_rows, n_cols), x, what="panel under the checking build")
    word = int(lay.rc[0].item()) & 0xFFFFFFFF            # the packed words are kept as int32 bit patterns
    x_slots = lay.n_buffers * lay.chunk_cols
    assert x_slots + 2 < 65536
    word = (word & 0xFFFF0000) | (x_slots + 2)
    lay.rc[0] = word - 2 ** 32 if word >= 2 ** 31 else word
    yp.fill_(7.0)
    try:
        panel.launch_panel(lay, xp, yp, n_rows, n_cols, st)
    except IndexError as e:
        assert "x position" in str(e) and f"limit {x_slots}" in str(e), str(e)
        print("IndexError:", e)
    else:
        raise AssertionError("the panel entry point took a bad packed word")
    torch.cuda.synchronize()
    assert bool((yp == 7.0).all())
    print("all cases ok")


if __name__ == "__main__":
    main()
