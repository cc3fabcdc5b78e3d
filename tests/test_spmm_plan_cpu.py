"""How a CSR SpMM is cut into passes when B is too large to be gathered from L2: column panels of A, column tiles of
B and C.  Host logic only (CPU tensors, no launch)."""

import numpy as np
import scipy.sparse as sp
import torch

from flagsparse_b200 import spmm_csr as M
from flagsparse_b200 import synthetic as S
from helpers import handmade_csr


def test_column_panels_partition_the_entries():
    lens = [0, 5, 0, 17, 1, 64, 3] * 40
    data, idx, ptr = handmade_csr(3, lens, 1000, sort=False, replace=True)
    d, i, p = torch.from_numpy(data), torch.from_numpy(idx), torch.from_numpy(ptr)
    n_rows = len(lens)
    full = sp.csr_matrix((data.astype(np.float64), idx, ptr), shape=(n_rows, 1000)).toarray()
    for n_panels in (1, 2, 3, 7):
        parts = M.split_by_column_panels(d, i, p, n_rows, 1000, n_panels)
        assert len(parts) == n_panels and sum(int(t[0].numel()) for t in parts) == data.size
        w = -(-1000 // n_panels)
        total = np.zeros_like(full)
        for k, (dk, ik, pk) in enumerate(parts):
            assert pk.dtype == p.dtype and int(pk[0]) == 0 and int(pk[-1]) == dk.numel() and pk.numel() == n_rows + 1
            if ik.numel():
                assert int(ik.min()) >= k * w and int(ik.max()) < (k + 1) * w
            total += sp.csr_matrix((dk.numpy().astype(np.float64), ik.numpy(), pk.numpy()), shape=(n_rows, 1000)).toarray()
        assert np.array_equal(total, full)          # duplicates included: every entry lands in exactly one panel


def _prepared_on_cpu(spec):
    d, i, p = (torch.from_numpy(a) for a in S.generate_csr(spec, None))

    class Stats:
        max_row_nnz = 16

    prep = M.PreparedCsrSpmmOpt(d, i, p, (spec.n_rows, spec.n_cols), spec.n_rows, spec.n_cols, Stats(), 1024,
                                torch.zeros(d.numel() // 1024 + 2, dtype=torch.int32))
    return prep


def test_pass_plan(monkeypatch):
    spec = S.config_spec("c4").scaled(1 << 14)        # uniform columns: consecutive entries span the whole width
    prep = _prepared_on_cpu(spec)
    assert prep.column_span() > 0.9 * spec.n_cols
    assert M.PANEL_BYTES == 0 and prep.n_panels_for(128) == 1            # the split is off unless asked for
    # B small enough for L2: one pass over the whole width
    monkeypatch.setattr(M, "PANEL_BYTES", 64 << 20)
    assert prep.n_panels_for(32) == 1 and prep.n_panels_for(128) == 1
    assert [(c0, w, acc) for _, c0, w, acc in prep.passes_for(128)] == [(0, 128, False)]
    # a limit of 1 MiB: 2^14 rows of 128 bytes = 2 MiB per column tile -> two panels, tiles of 32 floats
    monkeypatch.setattr(M, "PANEL_BYTES", 1 << 20)
    assert prep.n_panels_for(32) == 2 and prep.n_panels_for(8) == 1        # 2^14 x 32 B = 0.5 MiB fits
    monkeypatch.setattr(M, "_tile_plan", lambda ptr, n_rows, nnz, tile: torch.zeros(nnz // tile + 2, dtype=torch.int32))
    passes = prep.passes_for(80)
    assert [(c0, w, acc) for _, c0, w, acc in passes] == [(0, 32, False), (0, 32, True), (32, 32, False), (32, 32, True),
                                                          (64, 16, False), (64, 16, True)]
    assert passes[0][0] is passes[2][0] and passes[0][0] is not passes[1][0]
    assert sum(part.data.numel() for part, c0, _, _ in passes if c0 == 0) == prep.data.numel()
    assert prep.plan_summary(80)["passes"] == 6
    # the override, and the switch
    monkeypatch.setenv("FSB_SPMM_PANELS", "3")
    assert prep.n_panels_for(8) == 3
    monkeypatch.delenv("FSB_SPMM_PANELS")
    monkeypatch.setenv("FSB_SPMM_PANEL_MB", "0")
    assert prep.n_panels_for(128) == 1
    # a banded matrix: consecutive entries stay within a narrow range of columns -> never split
    monkeypatch.delenv("FSB_SPMM_PANEL_MB")
    monkeypatch.setattr(M, "SPAN_WINDOW", 4096)
    band = _prepared_on_cpu(S.CsrSpec("band", 1 << 14, 1 << 14, ("const", 16), ("band", 64), False, 0))
    assert band.column_span() < 1024 and band.n_panels_for(128) == 1
