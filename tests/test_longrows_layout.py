"""The prepare-time split of long rows for the row-group panel kernel, checked on CPU tensors: every entry of a
long row lands in exactly one slot, packed words decode to the right (row, column), no accumulator receives more
than 16 entries of a unit or straddles two pieces, the CTA / group tables are consistent, and a plain evaluation
of (short part + long layout) equals the oracle.  No kernel is launched."""

import numpy as np
import pytest
import torch

from flagsparse_b200 import longrows
from helpers import handmade_csr
from oracle import csr_oracle as O

SLOTS = 512


def _skewed(seed, n_rows, n_cols, vdt):
    rng = np.random.default_rng(seed)
    lens = rng.integers(0, 12, n_rows)
    lens[rng.choice(n_rows, 60, replace=False)] = rng.integers(64, 400, 60)
    lens[rng.choice(n_rows, 6, replace=False)] = rng.integers(2000, min(n_cols, 30000), 6)
    return handmade_csr(seed + 1, lens.tolist(), n_cols, value_dtype=vdt)


def _evaluate_long(lay, x):
    """Partial sums the way the kernels walk the layout, then the reduction over CTAs; returns {row: value}."""
    val = lay.val.numpy().astype(np.float64)
    rc = lay.rc.numpy().astype(np.int64) & 0xFFFFFFFF
    upp, uch = lay.unit_piece_ptr.numpy(), lay.unit_chunk.numpy()
    cup, cg = lay.cta_unit_ptr.numpy(), lay.cta_group.numpy()
    gq, gc, vb = lay.group_q_ptr.numpy(), lay.group_cta_ptr.numpy(), lay.vbase.numpy()
    cpp = lay.cta_part_ptr.numpy()
    CW = lay.chunk_cols
    E = 16 // lay.val.element_size()
    part = np.zeros(lay.part.numel())
    assert cup[0] == 0 and cup[-1] == lay.n_units and upp[-1] == lay.n_pieces and gc[-1] == lay.n_ctas
    seen = 0
    sl = np.arange(SLOTS)
    ln, k = sl // 16, sl % 16
    for c in range(lay.n_ctas):
        g = cg[c]
        assert gc[g] <= c < gc[g + 1]
        q0, q1 = gq[g], gq[g + 1]
        n_acc = vb[q1] - vb[q0]
        assert 0 < n_acc <= lay.max_group_acc
        acc = np.zeros(n_acc)
        for u in range(cup[c], cup[c + 1]):
            parity = (u - cup[c]) & (lay.n_buffers - 1)
            per_acc = {}
            for pc in range(upp[u], upp[u + 1]):
                w = rc[pc * SLOTS + (k // 4) * 128 + ln * 4 + k % 4]
                vals = val[pc * SLOTS + (k // E) * 32 * E + ln * E + k % E]
                a, field = w >> 16, w & 0xFFFF
                for kk in range(16):   # race-freedom: the 32 slots of a round hold 32 different accumulators
                    ak = a[kk::16]
                    ak = ak[ak != lay.pad_row]
                    assert ak.size == np.unique(ak).size
                live = a != lay.pad_row
                assert live.any() and np.all(live[:live.sum()]) and np.all(vals[~live] == 0)
                al, fl = a[live], field[live]
                assert np.all(al < n_acc) and np.all(fl // CW == parity)
                cols = uch[u] * CW + fl % CW
                np.add.at(acc, al, vals[live] * x[cols])
                for v, n in zip(*np.unique(al, return_counts=True)):
                    assert v not in per_acc, "an accumulator straddles two pieces of a unit"
                    per_acc[v] = n
                seen += int(live.sum())
            assert not per_acc or max(per_acc.values()) <= 16
        for i in range(q1 - q0):
            part[cpp[c] + i] = acc[vb[q0 + i] - vb[q0]: vb[q0 + i + 1] - vb[q0]].sum()
    out = {}
    qg, rows = lay.q_group.numpy(), lay.long_rows.numpy()
    for q in range(lay.n_long):
        g = qg[q]
        assert gq[g] <= q < gq[g + 1]
        out[int(rows[q])] = sum(part[cpp[c] + q - gq[g]] for c in range(gc[g], gc[g + 1]))
    return out, seen


@pytest.mark.parametrize("vdt,acc_cap,n_ctas", [("float32", 640, 7), ("float64", 256, 12), ("float32", None, None)])
def test_long_row_layout(fsb_lib, vdt, acc_cap, n_ctas):
    n_rows, n_cols = 1500, 40000
    data, indices, indptr = _skewed(3, n_rows, n_cols, np.dtype(vdt))
    x = np.random.default_rng(5).uniform(-1, 1, n_cols).astype(vdt)
    td, ti, tp = torch.from_numpy(data), torch.from_numpy(indices), torch.from_numpy(indptr)
    lens, is_long, long_nnz = longrows.split_rows(tp, n_rows, 64)
    assert int(is_long.sum()) >= 60 and long_nnz == int(lens[is_long].sum())
    lay, mask = longrows.build_long_row_layout(td, ti, tp, lens, is_long, n_cols, n_ctas_target=n_ctas,
                                               acc_cap=acc_cap)
    assert torch.equal(mask, is_long) and lay.nnz == long_nnz and lay.n_long == int(is_long.sum())
    if acc_cap is not None:
        assert lay.n_groups > 1 and lay.max_group_acc <= acc_cap
        assert abs(lay.n_ctas - n_ctas) <= lay.n_groups
    # rows with more than 16 entries in a chunk need several accumulators
    assert int((lay.vbase[1:] - lay.vbase[:-1]).max()) > 1
    # longest rows first
    ll = lens[lay.long_rows.long()].numpy()
    assert np.all(np.diff(ll) <= 0)
    got, seen = _evaluate_long(lay, x.astype(np.float64))
    assert seen == long_nnz
    ref, mag = O.spmv_f64(data, indices, indptr, (n_rows, n_cols), x)
    long_ids = np.nonzero(is_long.numpy())[0]
    assert sorted(got) == long_ids.tolist()
    for r in long_ids:
        assert abs(got[r] - ref[r]) <= 1e-12 * max(mag[r], 1e-300)
    # the short part: same shape, long rows emptied, the other rows untouched
    d_s, i_s, p_s = longrows.short_part(td, ti, tp, lens, is_long)
    ps = p_s.numpy()
    assert ps.dtype == indptr.dtype and ps[-1] == data.size - long_nnz
    assert np.all(np.diff(ps)[long_ids] == 0)
    ref_s, _ = O.spmv_f64(d_s.numpy(), i_s.numpy(), ps, (n_rows, n_cols), x)
    short_ids = np.nonzero(~is_long.numpy())[0]
    assert np.array_equal(ref_s[short_ids], ref[short_ids]) and not ref_s[long_ids].any()


def test_only_dense_groups_are_kept(fsb_lib):
    """With a density requirement the longest rows stay (whole groups of them), the sparser groups go back."""
    n_rows, n_cols = 1500, 40000
    data, indices, indptr = _skewed(3, n_rows, n_cols, np.float32)
    td, ti, tp = torch.from_numpy(data), torch.from_numpy(indices), torch.from_numpy(indptr)
    lens, cand, _ = longrows.split_rows(tp, n_rows, 64)
    full, _ = longrows.build_long_row_layout(td, ti, tp, lens, cand, n_cols, n_ctas_target=7, acc_cap=640)
    assert full.n_groups >= 2
    # density of the first group only
    q1 = int(full.group_q_ptr[1])
    first_nnz = int(lens[full.long_rows[:q1].long()].sum())
    need = first_nnz // 5 - 1            # 5 chunks of 8192 columns: the first group passes, later ones do not
    lay, mask = longrows.build_long_row_layout(td, ti, tp, lens, cand, n_cols, n_ctas_target=7, acc_cap=640,
                                               min_unit_entries=need)
    assert lay.n_groups == 1 and lay.n_long == q1 and lay.nnz == first_nnz and int(mask.sum()) == q1
    assert torch.equal(lay.long_rows, full.long_rows[:q1])
    x = np.random.default_rng(5).uniform(-1, 1, n_cols)
    got, seen = _evaluate_long(lay, x)
    assert seen == first_nnz
    ref, mag = O.spmv_f64(data, indices, indptr, (n_rows, n_cols), x.astype(np.float32))
    for r, v in got.items():
        assert abs(v - ref[r]) <= 1e-6 * max(mag[r], 1e-300)
    # nothing dense enough: no layout
    assert longrows.build_long_row_layout(td, ti, tp, lens, cand, n_cols, acc_cap=640,
                                          min_unit_entries=first_nnz) is None


def test_no_candidates(fsb_lib):
    data, indices, indptr = handmade_csr(9, [5] * 100, 64)
    tp = torch.from_numpy(indptr)
    lens, is_long, long_nnz = longrows.split_rows(tp, 100, 64)
    assert long_nnz == 0 and not is_long.any()
    assert longrows.build_long_row_layout(torch.from_numpy(data), torch.from_numpy(indices), tp, lens, is_long,
                                          64) is None
