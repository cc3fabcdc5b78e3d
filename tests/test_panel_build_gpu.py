"""The device-side builder of the panel layout (csrc/panel_build.cu) against the host-side one (panel.py:
_build_slab + pack_pieces): the same arrays, bit for bit, and the same decisions."""

import numpy as np
import pytest
import torch

import flagsparse_b200 as fs
from flagsparse_b200 import panel as P
from flagsparse_b200 import synthetic as S
from gpu_util import dev, env
from helpers import assert_spmv_ok, handmade_csr

pytestmark = pytest.mark.gpu


def _both(d, i, p, n_rows, n_cols, rounds=None, **envs):
    """(layout of the device-side builder, layout of the host-side builder) for the same matrix."""
    mx = int((p[1:] - p[:-1]).max().item()) if p.numel() > 1 else 0
    with env(FSB_PANEL_BUILDER="device", **envs):
        fused = P.build_panel_layout(d, i, p, n_rows, n_cols, mx, force=True, rounds=rounds)
    with env(FSB_PANEL_BUILDER="torch", **envs):
        host = P.build_panel_layout(d, i, p, n_rows, n_cols, mx, force=True, rounds=rounds)
    return fused, host


def _assert_same(a, b, what):
    assert (a is None) == (b is None), what
    if a is None:
        return
    for name in ("n_row_blocks", "rb_rows", "chunk_cols", "n_buffers", "rounds", "flags", "max_run", "pad_row", "n_units",
                 "n_pieces"):
        assert getattr(a, name) == getattr(b, name), f"{what}: {name} {getattr(a, name)} != {getattr(b, name)}"
    for name in ("unit_piece_ptr", "unit_chunk", "rb_unit_ptr", "rc", "val"):
        ta, tb = getattr(a, name), getattr(b, name)
        assert ta.dtype == tb.dtype and ta.shape == tb.shape, f"{what}: {name} {ta.dtype}{tuple(ta.shape)} {tb.dtype}{tuple(tb.shape)}"
        if not torch.equal(ta, tb):
            bad = torch.nonzero(ta != tb).flatten()
            raise AssertionError(f"{what}: {name} differs at {bad.numel()} places, first {bad[:5].tolist()}")
    assert abs(a.x_overhead - b.x_overhead) < 1e-12 and abs(a.slot_overhead - b.slot_overhead) < 1e-12


def _is_fused(d, i, p, n_rows, n_cols, **envs):
    geometry = P._geometry(d.dtype, n_rows, d.device, P.default_buffers())
    with env(FSB_PANEL_BUILDER="device", **envs):
        if not P._fused_applicable(d, i, p, n_rows, n_cols, geometry[3], geometry[2]):
            return "not applicable"
        lay = P._build_fused(d, i, p, n_rows, n_cols, geometry, P.default_buffers(), None, True)
    return lay if isinstance(lay, str) else "fused"


@pytest.mark.parametrize("vdt", ["float32", "float64"])
@pytest.mark.parametrize("name,rows", [("c2", 300000), ("c5", 400000)])
def test_banded_matrices(cuda, fsb_lib, vdt, name, rows):
    spec = S.config_spec(name).scaled(rows)
    idt = "int64" if vdt == "float64" else "int32"
    d, i, p = S.generate_csr(spec, "cuda:0", value_dtype=vdt, index_dtype=idt, indptr_dtype=idt)
    envs = dict(FSB_PANEL_NO_CORE="1")          # the core pieces of float32 single-entry layouts are host-only
    assert _is_fused(d, i, p, spec.n_rows, spec.n_cols, **envs) == "fused"
    for rounds in (None, 4, 8, 16):
        a, b = _both(d, i, p, spec.n_rows, spec.n_cols, rounds=rounds, **envs)
        _assert_same(a, b, f"{name} {vdt} rounds {rounds}")
    # and the product from the device-built layout
    x = S.dense_vector(spec, spec.n_cols, "cuda:0", value_dtype=vdt)
    with env(FSB_SPMV_ALGO="panel", FSB_PANEL_BUILDER="device", **envs):
        prep = fs.prepare_spmv_csr(d, i, p, (spec.n_rows, spec.n_cols))
    assert prep.panel is not None
    y = fs.flagsparse_spmv_csr(x=x, prepared=prep)
    assert_spmv_ok(y.cpu().numpy(), d.cpu().numpy(), i.cpu().numpy(), p.cpu().numpy(), (spec.n_rows, spec.n_cols),
                   x.cpu().numpy(), what=f"{name} {vdt} device-built layout")
    prep.check_status()


@pytest.mark.parametrize("rows", [400000, 1 << 22])
def test_core_pieces(cuda, fsb_lib, rows):
    """float32 layouts with mostly one entry per row and unit: core pieces + rest, as pack_pieces_core makes them.
    The larger case has some 200 chunks per row block: the sort pass takes its wide window."""
    spec = S.config_spec("c5").scaled(rows)
    d, i, p = S.generate_csr(spec, "cuda:0", indptr_dtype="int64")
    assert _is_fused(d, i, p, spec.n_rows, spec.n_cols) == "fused"
    for rounds in ((None, 4, 16) if rows < (1 << 22) else (None,)):
        a, b = _both(d, i, p, spec.n_rows, spec.n_cols, rounds=rounds)
        assert a is not None and not a.flags & P.FLAG_RUNS
        _assert_same(a, b, f"c5 float32 with core pieces, {rows} rows, rounds {rounds}")


def test_long_runs_every_piece_size(cuda, fsb_lib):
    n, width, n_cols = 200000, 48, 300000
    rng = np.random.default_rng(3)
    start = np.clip(np.arange(n) * n_cols // n + rng.integers(-2000, 2000, n), 0, n_cols - width)
    idx = (start[:, None] + np.arange(width)[None, :]).reshape(-1).astype(np.int32)
    ptr = (np.arange(n + 1, dtype=np.int64) * width).astype(np.int32)
    data = rng.uniform(-1, 1, idx.size).astype(np.float32)
    d, i, p = dev(data), dev(idx), dev(ptr)
    assert _is_fused(d, i, p, n, n_cols) == "fused"
    for rounds in (None, 4, 8, 16):
        a, b = _both(d, i, p, n, n_cols, rounds=rounds)
        assert a is not None and a.max_run == width and a.flags & P.FLAG_LONG_RUNS
        _assert_same(a, b, f"48-entry runs, rounds {rounds}")


@pytest.mark.parametrize("vdt,idt,pdt", [(np.float32, np.int64, np.int64), (np.float64, np.int32, np.int64),
                                         (np.float32, np.int32, np.int32)])
def test_ragged_unsorted_duplicates(cuda, fsb_lib, vdt, idt, pdt):
    """Empty rows, rows of very different lengths, unsorted and repeated columns inside a band, sizes that are no
    multiple of the row block or the chunk."""
    rng = np.random.default_rng(11)
    n_rows, n_cols = 180001, 200003
    lens = rng.poisson(9, n_rows)
    lens[rng.integers(0, n_rows, 4000)] = 0
    lens[rng.integers(0, n_rows, 50)] = 300
    ptr = np.zeros(n_rows + 1, dtype=np.int64)
    ptr[1:] = np.cumsum(lens)
    rows = np.repeat(np.arange(n_rows), lens)
    centre = rows * n_cols // n_rows
    idx = np.clip(centre + rng.integers(-6000, 6000, rows.size), 0, n_cols - 1)      # unsorted, with repeats
    data = rng.uniform(-1, 1, rows.size).astype(vdt)
    d, i, p = dev(data), dev(idx.astype(idt)), dev(ptr.astype(pdt))
    assert _is_fused(d, i, p, n_rows, n_cols, FSB_PANEL_NO_CORE="1") == "fused"
    for rounds in (None, 8, 16):
        a, b = _both(d, i, p, n_rows, n_cols, rounds=rounds, FSB_PANEL_NO_CORE="1")
        _assert_same(a, b, f"ragged {vdt.__name__} rounds {rounds}")
    a, _ = _both(d, i, p, n_rows, n_cols, FSB_PANEL_NO_CORE="1")
    x = rng.uniform(-1, 1, n_cols).astype(vdt)
    y = torch.empty(n_rows, dtype=d.dtype, device="cuda:0")
    P.launch_panel(a, dev(x), y, n_rows, n_cols, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert_spmv_ok(y.cpu().numpy(), data, idx.astype(np.int32), ptr, (n_rows, n_cols), x, what="ragged product")


def test_columns_spread_too_widely_fall_back_to_the_host_builder(cuda, fsb_lib):
    lens = [40] * 60000
    data, idx, ptr = handmade_csr(5, lens, 12_000_000, replace=True)   # uniform columns: hundreds of chunks per tile
    d, i, p = dev(data), dev(idx), dev(ptr)
    assert _is_fused(d, i, p, len(lens), 12_000_000) == "host"
    a, b = _both(d, i, p, len(lens), 12_000_000)
    _assert_same(a, b, "wide columns")


def test_tiny_and_degenerate(cuda, fsb_lib):
    data, idx, ptr = handmade_csr(6, [0, 3, 0, 0, 1, 7, 0], 50)
    a, b = _both(dev(data), dev(idx), dev(ptr), 7, 50)
    _assert_same(a, b, "tiny")
    data, idx, ptr = handmade_csr(7, [1], 1)
    a, b = _both(dev(data), dev(idx), dev(ptr), 1, 1)
    _assert_same(a, b, "one entry")
