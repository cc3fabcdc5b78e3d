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
    R = lay.rounds
    assert slots == 32 * R
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
            parity = (u - rbp[b]) % lay.n_buffers
            rows_in_unit = []
            for pc in range(upp[u], upp[u + 1]):
                # undo the interleaving: slot = R * lane + k
                sl = np.arange(slots)
                ln, k = sl // R, sl % R
                E = 16 // lay.val.element_size()
                w = rc[pc * slots + (k // 4) * 128 + ln * 4 + k % 4]
                vals = val[pc * slots + (k // E) * 32 * E + ln * E + k % E]
                rloc, field = w >> 16, w & 0xFFFF
                # the kernel's race-freedom: a lane adds to an accumulator where its row ends.  In every round but a
                # lane's last one the lanes that do so are on different rows; in the last round two lanes may meet
                # only in layouts flagged for the kernel's segmented path
                nxt = np.append(rloc[1:], lay.pad_row)
                nxt[R - 1::R] = lay.pad_row                      # a lane's run ends with its last slot
                ends = (rloc != lay.pad_row) & (nxt != rloc)
                for k in range(R):
                    rk = rloc[k::R][ends[k::R]]
                    if k < R - 1 or not (lay.flags & panel.FLAG_LONG_RUNS):
                        assert rk.size == np.unique(rk).size
                    if not (lay.flags & panel.FLAG_LONG_RUNS):
                        # the direct path adds every slot of a round: all its real rows must differ
                        ak = rloc[k::R]
                        ak = ak[ak != lay.pad_row]
                        assert ak.size == np.unique(ak).size
                live = rloc != lay.pad_row
                assert live.any() and np.all(live[:live.sum()])            # real slots first, then padding
                assert np.all(vals[~live] == 0)
                rl, fl = rloc[live], field[live]
                assert np.all(fl // CW == parity)
                # ordered by the shared-memory bank of the accumulator, rows ascending inside a bank, and the
                # entries of a row next to each other
                banks = panel.ACC_BANKS[lay.val.element_size()]
                assert np.all(np.diff((rl % banks) * (1 << 20) + rl) >= 0)
                cols = uch[u] * CW + fl % CW
                rows = b * RB + rl
                assert np.all(rows < n_rows) and np.all(cols < n_cols)
                np.add.at(y, rows, vals[live] * x[cols])
                rows_in_unit.append(np.unique(rl))
                seen += int(live.sum())
            allrows = np.concatenate(rows_in_unit)
            assert allrows.size == np.unique(allrows).size   # a row never straddles two pieces of a unit
    return y, seen


@pytest.mark.parametrize("rounds", [None, 4, 8, 16])
@pytest.mark.parametrize("vdt", ["float32", "float64"])
def test_layout_of_a_banded_matrix(fsb_lib, vdt, rounds):
    spec = S.config_spec("c2").scaled(120000)
    d, i, p = (torch.from_numpy(a) for a in S.generate_csr(spec, None, value_dtype=vdt))
    lay = panel.build_panel_layout(d, i, p, spec.n_rows, spec.n_cols, 70, force=True, rounds=rounds)
    assert lay is not None and lay.n_row_blocks * lay.rb_rows >= spec.n_rows
    assert lay.rounds == (rounds or lay.rounds) and lay.rounds in panel.ROUNDS and lay.pad_row == lay.rb_rows
    if rounds is None:
        assert lay.max_run <= lay.rounds and not (lay.flags & panel.FLAG_LONG_RUNS)  # no segmented path needed
        assert lay.flags & panel.FLAG_RUNS                       # about two entries of a row per chunk here
    # rows of this matrix have up to a dozen entries in a chunk: small pieces must carry the long-run flag
    assert bool(lay.flags & panel.FLAG_LONG_RUNS) == (lay.max_run > lay.rounds)
    if rounds == 4:
        assert lay.flags & panel.FLAG_LONG_RUNS
    x = S.dense_vector(spec, spec.n_cols, value_dtype=vdt).astype(np.float64)
    y, seen = _evaluate(lay, x, spec.n_rows, spec.n_cols, fsb_lib.fsb_spmv_panel_piece_slots(lay.rounds))
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
    y, seen = _evaluate(lay, x, len(lens), 10007, fsb_lib.fsb_spmv_panel_piece_slots(lay.rounds))
    assert seen == data.size
    ref, _ = O.spmv_f64(data, idx, ptr, (len(lens), 10007), x)
    assert np.allclose(y, ref, rtol=0, atol=1e-9)


def test_rows_with_long_runs(fsb_lib):
    # block-structured rows: 48 consecutive columns per row, i.e. runs of up to 48 entries inside one chunk.  Such a
    # layout is accepted, takes the largest piece and is flagged for the kernel's segmented path
    n, width = 3000, 48
    rng = np.random.default_rng(11)
    start = rng.integers(0, 20000 - width, n)
    idx = (start[:, None] + np.arange(width)[None, :]).reshape(-1).astype(np.int32)
    ptr = (np.arange(n + 1) * width).astype(np.int32)
    data = rng.uniform(-1, 1, idx.size).astype(np.float32)
    d, i, p = torch.from_numpy(data), torch.from_numpy(idx), torch.from_numpy(ptr)
    lay = panel.build_panel_layout(d, i, p, n, 20000, width, force=True)
    assert lay is not None and lay.rounds == 16 and lay.max_run == width and lay.flags & panel.FLAG_LONG_RUNS
    x = rng.uniform(-1, 1, 20000)
    y, seen = _evaluate(lay, x, n, 20000, fsb_lib.fsb_spmv_panel_piece_slots(lay.rounds))
    assert seen == data.size
    ref, _ = O.spmv_f64(data, idx, ptr, (n, 20000), x)
    assert np.allclose(y, ref, rtol=0, atol=1e-9)
    # asked for small pieces, a run of 48 still fits (a piece of 4 rounds has 128 slots)
    lay4 = panel.build_panel_layout(d, i, p, n, 20000, width, force=True, rounds=4)
    assert lay4 is not None and lay4.rounds == 4 and lay4.flags & panel.FLAG_LONG_RUNS
    y4, seen4 = _evaluate(lay4, x, n, 20000, 128)
    assert seen4 == data.size and np.allclose(y4, ref, rtol=0, atol=1e-9)
    # a run longer than the largest piece (512 slots) cannot be laid out
    data, idx, ptr = handmade_csr(7, [600, 3], 1024)
    assert panel.build_panel_layout(torch.from_numpy(data), torch.from_numpy(idx), torch.from_numpy(ptr), 2, 1024, 600,
                                    force=True) is None
    # ... but one that only outgrows the small piece moves the layout to the largest one
    data, idx, ptr = handmade_csr(7, [200, 3], 1024)
    lay = panel.build_panel_layout(torch.from_numpy(data), torch.from_numpy(idx), torch.from_numpy(ptr), 2, 1024, 200,
                                   force=True, rounds=4)
    assert lay is not None and lay.rounds == 16


def test_choice_of_piece_size():
    # the smallest piece whose rounds hold every run; the largest one when some run is longer than any
    assert panel.choose_rounds([0, 0, 0]) == 4
    assert panel.choose_rounds([100, 0, 0]) == 8
    assert panel.choose_rounds([1 << 22, 10, 0]) == 16
    assert panel.choose_rounds([1 << 22, 1 << 21, 5]) == 16


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
        assert lay is None          # eight float32 chunks of 10240 columns leave no room for the accumulators
        return
    assert lay.n_buffers == n_buffers
    y, seen = _evaluate(lay, x.astype(np.float64), spec.n_rows, spec.n_cols, fsb_lib.fsb_spmv_panel_piece_slots(lay.rounds))
    assert seen == d.size
    ref, mag = O.spmv_f64(d, i, p, (spec.n_rows, spec.n_cols), x)
    assert O.max_bound_ratio(y, ref, mag) <= 1e-12


def test_single_entry_rows_get_core_pieces(fsb_lib, monkeypatch):
    """A wide band (about one entry per row and unit): most pieces are "core" pieces in which lane l holds only
    accumulators congruent to l modulo 32, the rest follow them; the whole layout still evaluates to the product."""
    spec = S.config_spec("c5").scaled(600000)           # band of +-300000 columns: 0.44 entries per row and chunk
    d, i, p = (torch.from_numpy(a) for a in S.generate_csr(spec, None, indptr_dtype="int64"))
    lay = panel.build_panel_layout(d, i, p, spec.n_rows, spec.n_cols, 70, force=True, rounds=8)
    assert lay is not None and not (lay.flags & panel.FLAG_RUNS)
    slots = fsb_lib.fsb_spmv_panel_piece_slots(lay.rounds)
    x = S.dense_vector(spec, spec.n_cols).astype(np.float64)
    y, seen = _evaluate(lay, x, spec.n_rows, spec.n_cols, slots)
    assert seen == d.numel()
    ref, _ = O.spmv_f64(d.numpy(), i.numpy(), p.numpy(), (spec.n_rows, spec.n_cols), x)
    assert np.allclose(y, ref, rtol=0, atol=1e-9)
    # count the pieces whose every lane stays inside its own class
    rc = lay.rc.numpy().astype(np.int64) & 0xFFFFFFFF
    R = lay.rounds
    core = full = 0
    for pc in range(lay.n_pieces):
        sl = np.arange(slots)
        ln, k = sl // R, sl % R
        rloc = rc[pc * slots + (k // 4) * 128 + ln * 4 + k % 4] >> 16
        live = rloc != lay.pad_row
        full += int(live.all())
        core += int(live.all() and np.all(rloc % 32 == ln))
    assert core > 0.3 * lay.n_pieces and core <= full, (core, full, lay.n_pieces)
    # the same matrix without core pieces has the same number of entries in (a few) fewer, fuller pieces at most
    monkeypatch.setenv("FSB_PANEL_NO_CORE", "1")
    plain = panel.build_panel_layout(d, i, p, spec.n_rows, spec.n_cols, 70, force=True, rounds=8)
    assert plain.n_units == lay.n_units and lay.n_pieces <= plain.n_pieces * 1.1
