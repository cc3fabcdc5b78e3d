"""The prepare-time regrouping for the panel SpMV kernel, checked on CPU tensors: every entry lands in exactly
one tile, packed words decode back to the right (row, column), the tile tables are consistent with what the
kernel assumes, and a plain evaluation of the layout equals the oracle.  No kernel is launched."""

import numpy as np
import pytest
import torch

from flagsparse_b200 import panel
from flagsparse_b200 import synthetic as S
from helpers import handmade_csr
from oracle import csr_oracle as O


def _evaluate(lay, x, n_rows, n_cols, slots):
    """y from the layout the way the kernel walks it (row block -> units -> pieces -> slots)."""
    y = np.zeros(n_rows)
    val = lay.val.numpy().astype(np.float64)
    rc = lay.rc.numpy().astype(np.int64) & 0xFFFFFFFF
    upp, uch, rbp = lay.unit_piece_ptr.numpy(), lay.unit_chunk.numpy(), lay.rb_unit_ptr.numpy()
    CW, RB = lay.chunk_cols, lay.rb_rows
    seen = 0
    assert rbp[0] == 0 and rbp[-1] == lay.n_units and upp[-1] == lay.n_pieces
    for b in range(lay.n_row_blocks):
        assert np.all(np.diff(uch[rbp[b]:rbp[b + 1]]) > 0)   # units of a row block in chunk order
        for u in range(rbp[b], rbp[b + 1]):
            parity = (u - rbp[b]) & (lay.n_buffers - 1)
            rows_in_unit = []
            for pc in range(upp[u], upp[u + 1]):
                # undo the interleaving: slot = 16 * lane + k
                sl = np.arange(slots)
                ln, k = sl // 16, sl % 16
                E = 16 // lay.val.element_size()
                w = rc[pc * slots + (k // 4) * 128 + ln * 4 + k % 4]
                vals = val[pc * slots + (k // E) * 32 * E + ln * E + k % E]
                rloc, field = w >> 16, w & 0xFFFF
                # the kernel's race-freedom: the 32 slots of a round (same position modulo 16) hold 32 different rows
                for k in range(16):
                    rk = rloc[k::16]
                    rk = rk[rk != 0xFFFF]
                    assert rk.size == np.unique(rk).size
                live = rloc != 0xFFFF
                assert live.any() and np.all(live[:live.sum()])            # real slots first, then padding
                assert np.all(vals[~live] == 0)
                rl, fl = rloc[live], field[live]
                assert np.all(fl // CW == parity) and np.all(np.diff(rl) >= 0)
                cols = uch[u] * CW + fl % CW
                rows = b * RB + rl
                assert np.all(rows < n_rows) and np.all(cols < n_cols)
                np.add.at(y, rows, vals[live] * x[cols])
                rows_in_unit.append(np.unique(rl))
                seen += int(live.sum())
            allrows = np.concatenate(rows_in_unit)
            assert allrows.size == np.unique(allrows).size   # a row never straddles two pieces of a unit
    return y, seen


@pytest.mark.parametrize("vdt", ["float32", "float64"])
def test_layout_of_a_banded_matrix(fsb_lib, vdt):
    spec = S.config_spec("c2").scaled(120000)
    d, i, p = (torch.from_numpy(a) for a in S.generate_csr(spec, None, value_dtype=vdt))
    lay = panel.build_panel_layout(d, i, p, spec.n_rows, spec.n_cols, 70, force=True)
    assert lay is not None and lay.n_row_blocks * lay.rb_rows >= spec.n_rows
    x = S.dense_vector(spec, spec.n_cols, value_dtype=vdt).astype(np.float64)
    y, seen = _evaluate(lay, x, spec.n_rows, spec.n_cols, fsb_lib.fsb_spmv_panel_piece_slots())
    assert seen == d.numel()
    ref, mag = O.spmv_f64(d.numpy(), i.numpy(), p.numpy(), (spec.n_rows, spec.n_cols), x)
    assert np.allclose(y, ref, rtol=0, atol=1e-9)
    vt = 0 if vdt == "float32" else 1
    assert (fsb_lib.fsb_spmv_panel_smem_bytes(vt, lay.rb_rows, lay.chunk_cols, lay.n_buffers)
            + fsb_lib.fsb_spmv_panel_static_smem_bytes()) <= 227 * 1024
    assert lay.slot_overhead < 1.5  # a small matrix: the last piece of each unit is mostly padding


def test_layout_with_empty_rows_ragged_edges_and_duplicates(fsb_lib):
    lens = [0, 0, 7, 0, 15, 1, 0, 16, 0, 0, 12] * 300
    # n_cols not a multiple of 4: the last chunk of x is ragged; duplicate, unsorted columns inside rows
    data, idx, ptr = handmade_csr(5, lens, 10007, sort=False, replace=True)
    d, i, p = torch.from_numpy(data), torch.from_numpy(idx), torch.from_numpy(ptr)
    lay = panel.build_panel_layout(d, i, p, len(lens), 10007, 16, force=True)
    assert lay is not None
    x = np.random.default_rng(6).uniform(-1, 1, 10007)
    y, seen = _evaluate(lay, x, len(lens), 10007, fsb_lib.fsb_spmv_panel_piece_slots())
    assert seen == data.size
    ref, _ = O.spmv_f64(data, idx, ptr, (len(lens), 10007), x)
    assert np.allclose(y, ref, rtol=0, atol=1e-9)
    # a row with more entries inside one column chunk than a piece can hold with room to spare: refused
    data, idx, ptr = handmade_csr(7, [20, 3], 64)
    assert panel.build_panel_layout(torch.from_numpy(data), torch.from_numpy(idx), torch.from_numpy(ptr), 2, 64, 20,
                                    force=True) is None


def test_selection_rules(fsb_lib):
    # too small, too long rows, or columns spread over the whole width: no panel layout
    spec = S.config_spec("c2").scaled(4096)
    d, i, p = (torch.from_numpy(a) for a in S.generate_csr(spec, None))
    assert panel.build_panel_layout(d, i, p, spec.n_rows, spec.n_cols, 70) is None          # below MIN_NNZ
    assert panel.build_panel_layout(d, i, p, spec.n_rows, spec.n_cols, 100000) is None      # long rows
    spec3 = S.config_spec("c3").scaled(1 << 18)
    d, i, p = (torch.from_numpy(a) for a in S.generate_csr(spec3, None))
    assert panel.estimate_units(i, p, spec3.n_rows, spec3.n_cols, 2048, 4096) > 0.9 * 128 * 64


def test_layout_built_in_slabs_equals_layout_built_at_once(fsb_lib, monkeypatch):
    spec = S.config_spec("c2").scaled(120000)
    d, i, p = S.generate_csr(spec, None)
    td, ti, tp = torch.from_numpy(d), torch.from_numpy(i), torch.from_numpy(p)
    whole = panel.build_panel_layout(td, ti, tp, spec.n_rows, spec.n_cols, int(np.diff(p).max()), force=True)
    monkeypatch.setattr(panel, "SLAB_NNZ", d.size // 7)
    slabs = panel._slabs(tp, spec.n_rows, whole.rb_rows)
    assert len(slabs) > 3 and slabs[0][0] == 0 and slabs[-1][1] == spec.n_rows
    assert all(a[1] == b[0] and a[0] % whole.rb_rows == 0 for a, b in zip(slabs, slabs[1:]))
    parts = panel.build_panel_layout(td, ti, tp, spec.n_rows, spec.n_cols, int(np.diff(p).max()), force=True)
    for name in ("val", "rc", "unit_piece_ptr", "unit_chunk", "rb_unit_ptr"):
        assert torch.equal(getattr(whole, name), getattr(parts, name)), name
    assert (whole.n_units, whole.n_pieces) == (parts.n_units, parts.n_pieces)
    assert panel.estimate_units(ti, tp, spec.n_rows, spec.n_cols, whole.rb_rows, whole.chunk_cols) == whole.n_units


@pytest.mark.parametrize("n_buffers", [4, 8])
def test_layout_with_more_x_buffers(fsb_lib, monkeypatch, n_buffers):
    monkeypatch.setattr(panel, "N_BUFFERS", n_buffers)
    spec = S.config_spec("c2").scaled(120000)
    d, i, p = S.generate_csr(spec, None)
    x = S.dense_vector(spec, spec.n_cols)
    lay = panel.build_panel_layout(torch.from_numpy(d), torch.from_numpy(i), torch.from_numpy(p), spec.n_rows,
                                   spec.n_cols, int(np.diff(p).max()), force=True)
    if n_buffers == 8:
        assert lay is None          # eight float32 chunks of 8192 columns leave no room for the accumulators
        return
    assert lay.n_buffers == n_buffers
    y, seen = _evaluate(lay, x.astype(np.float64), spec.n_rows, spec.n_cols, fsb_lib.fsb_spmv_panel_piece_slots())
    assert seen == d.size
    ref, mag = O.spmv_f64(d, i, p, (spec.n_rows, spec.n_cols), x)
    assert O.max_bound_ratio(y, ref, mag) <= 1e-12
