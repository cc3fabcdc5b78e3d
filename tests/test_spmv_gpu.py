"""CSR SpMV on the GPU against the oracle: golden fixtures, structured edge cases, the benchmark
configurations at reduced and at full size.  Everything goes through the public API and therefore
through the C ABI of libfsb.so."""

import ctypes

import numpy as np
import pytest
import torch

import flagsparse_b200 as fs
from flagsparse_b200 import _lib
from flagsparse_b200 import synthetic as S
from gpu_util import check_spmv_blocks, dev, env, sample_blocks, spmv
from helpers import assert_spmv_ok, golden_files, handmade_csr, load_golden

pytestmark = pytest.mark.gpu

ALGOS = ["vector", "stream"]
# stream tunings: lanes-per-row shift 0..4 (bits 0-7 hold shift+1) x tile size (bits 8-9)
STREAM_TUNINGS = [0, 1, 2, 3, 5, (1 << 8) | 2, (3 << 8) | 3, (3 << 8) | 1]


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("path", golden_files("spmv"), ids=lambda p: p.split("/")[-1])
def test_golden_fixtures(cuda, fsb_lib, path, algo):
    g = load_golden(path)
    args = (g["data"], g["indices"], g["indptr"], g["shape"], g["x"])
    for use_opt in (False, True):
        y = spmv(*args, algo=algo, use_opt=use_opt)
        assert_spmv_ok(y, *args, what=path)
        # and inside the reference's own allclose tolerance of the reference's outputs
        atol, rtol = fs._tolerance_for_dtype(torch.float32 if y.dtype == np.float32 else torch.float64)
        for key in ("y_base", "y_opt"):
            assert np.allclose(y, g[key], atol=atol * 10, rtol=rtol * 10), key
        empty = np.diff(g["indptr"].astype(np.int64)) == 0
        assert np.all(y[empty] == 0)


def _edge_cases():
    T = 2048
    cases = {
        "one_row_one_entry": [1],
        "one_row": [37],
        "rows_31": [5] * 31,
        "rows_32": [5] * 32,
        "rows_33": [5] * 33,
        "all_empty": [0] * 50,
        "empty_then_full": [0] * 40 + [64] * 40 + [0] * 40,
        "ends_on_tile_edge": [T // 2, T // 2, T, 3],
        "straddles_tile_edge": [T - 1, 2, T - 3, 7, 1, 1],
        "one_row_many_tiles": [5 * T + 13],
        "long_row_between_short": [3] * 100 + [3 * T + 5] + [2] * 100,
        "huge_row": [1 << 17],
        "single_entries": [1] * 5000,
        "mixed": [0, 700, 0, 0, 1, 2500, 31, 32, 33, 0, 4097, 1],
        "more_rows_than_offsets_slots": [1] * 4500 + [0] * 3000 + [2] * 600,
    }
    return cases


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("name", sorted(_edge_cases()))
def test_edge_cases(cuda, fsb_lib, name, algo):
    lens = _edge_cases()[name]
    n_cols = max(1 << 17, 4096)
    for vdt, idt, pdt in ((np.float32, np.int32, np.int32), (np.float64, np.int64, np.int64), (np.float32, np.int32, np.int64)):
        data, idx, ptr = handmade_csr(7, lens, n_cols, vdt, idt, pdt)
        x = np.random.default_rng(8).uniform(-1, 1, n_cols).astype(vdt)
        y = spmv(data, idx, ptr, (len(lens), n_cols), x, algo=algo)
        assert_spmv_ok(y, data, idx, ptr, (len(lens), n_cols), x, what=f"{name}/{algo}")
        assert np.all(y[np.asarray(lens) == 0] == 0)


PANEL_CASES = ["one_row_one_entry", "one_row", "rows_31", "rows_32", "rows_33", "all_empty", "empty_then_full",
               "single_entries", "more_rows_than_offsets_slots"]


@pytest.mark.parametrize("name", PANEL_CASES)
def test_panel_kernel_edge_cases(cuda, fsb_lib, name):
    lens = _edge_cases()[name]
    for n_cols in (5001, 1 << 17):  # a ragged last chunk of x, and many chunks
        for vdt in (np.float32, np.float64):
            data, idx, ptr = handmade_csr(17, lens, n_cols, vdt)
            x = np.random.default_rng(18).uniform(-1, 1, n_cols).astype(vdt)
            y = spmv(data, idx, ptr, (len(lens), n_cols), x, algo="panel")
            assert_spmv_ok(y, data, idx, ptr, (len(lens), n_cols), x, what=f"panel/{name}")
            assert np.all(y[np.asarray(lens) == 0] == 0)


@pytest.mark.parametrize("vdt,idt", [("float32", "int32"), ("float64", "int64")])
def test_panel_kernel_on_banded_matrix(cuda, fsb_lib, vdt, idt):
    # 33M nnz in a band of +-65536 columns over 2^20 rows: large enough, and few enough column chunks per row
    # block, for the panel layout to be chosen
    spec = S.config_spec("c2").scaled(1 << 20)
    d, i, p = S.generate_csr(spec, "cuda:0", value_dtype=vdt, index_dtype=idt, indptr_dtype=idt)
    x = S.dense_vector(spec, spec.n_cols, "cuda:0", value_dtype=vdt)
    # float32 picks the panel layout by itself; float64 chunks of x are twice the bytes, which at this size
    # is just over the overhead limit, so ask for it
    with env(FSB_SPMV_ALGO=None if vdt == "float32" else "panel"):
        prep = fs.prepare_spmv_csr(d, i, p, (spec.n_rows, spec.n_cols))
    assert prep.algo == _lib.FSB_SPMV_PANEL and prep.panel is not None
    # columns spread over the whole matrix are not worth regrouping (every unit would load a chunk of x for a few
    # hundred entries): the vector kernel stays
    wide = S.config_spec("c4")
    dw, iw, pw = S.generate_csr(wide, "cuda:0", value_dtype=vdt)
    assert fs.prepare_spmv_csr(dw, iw, pw, (wide.n_rows, wide.n_cols)).algo == _lib.FSB_SPMV_VECTOR
    del dw, iw, pw
    y = fs.flagsparse_spmv_csr(x=x, prepared=prep)
    assert_spmv_ok(y.cpu().numpy(), d.cpu().numpy(), i.cpu().numpy(), p.cpu().numpy(), (spec.n_rows, spec.n_cols),
                   x.cpu().numpy(), what="panel banded")
    assert int(prep.panel.status.item()) == 0
    assert torch.equal(fs.flagsparse_spmv_csr(x=x, prepared=prep), y)          # bit-reproducible
    assert torch.equal(fs.flagsparse_spmv_csr(x=x * 4, prepared=prep), y * 4)  # exact under power-of-two scaling


@pytest.mark.parametrize("tuning", STREAM_TUNINGS)
def test_stream_tunings_stay_in_tolerance(cuda, fsb_lib, tuning):
    spec = S.config_spec("c3").scaled(1 << 15)
    data, idx, ptr = S.generate_csr(spec, None)
    x = S.dense_vector(spec, spec.n_cols)
    y = spmv(data, idx, ptr, (spec.n_rows, spec.n_cols), x, algo="stream", tuning=tuning)
    assert_spmv_ok(y, data, idx, ptr, (spec.n_rows, spec.n_cols), x, what=f"tuning {tuning}")
    lens = _edge_cases()["mixed"]
    data, idx, ptr = handmade_csr(9, lens, 8192)
    x = np.random.default_rng(10).uniform(-1, 1, 8192).astype(np.float32)
    y = spmv(data, idx, ptr, (len(lens), 8192), x, algo="stream", tuning=tuning)
    assert_spmv_ok(y, data, idx, ptr, (len(lens), 8192), x, what=f"mixed tuning {tuning}")


@pytest.mark.parametrize("tuning", STREAM_TUNINGS)
@pytest.mark.parametrize("vdt", [np.float32, np.float64])
def test_stream_rows_across_many_tiles(cuda, fsb_lib, tuning, vdt):
    """Rows that cross hundreds of tiles: their carries are summed by a whole warp of the fix-up kernel, the
    shorter crossings beside them by one thread each."""
    lens = [3, 700_000, 0, 5000, 1, 150_000, 40_000, 2, 300_001, 7]
    n_cols = 1 << 20
    data, idx, ptr = handmade_csr(21, lens, n_cols, value_dtype=vdt)
    x = np.random.default_rng(22).uniform(-1, 1, n_cols).astype(vdt)
    y = spmv(data, idx, ptr, (len(lens), n_cols), x, algo="stream", tuning=tuning)
    assert_spmv_ok(y, data, idx, ptr, (len(lens), n_cols), x, what=f"rows across many tiles, tuning {tuning}")
    y2 = spmv(data, idx, ptr, (len(lens), n_cols), x, algo="stream", tuning=tuning)
    assert np.array_equal(y, y2)


@pytest.mark.parametrize("lanes", [2, 4, 8, 16, 32])
def test_vector_lane_counts(cuda, fsb_lib, lanes):
    spec = S.config_spec("c2").scaled(5000)
    data, idx, ptr = S.generate_csr(spec, None)
    x = S.dense_vector(spec, spec.n_cols)
    y = spmv(data, idx, ptr, (spec.n_rows, spec.n_cols), x, algo="vector", tuning=lanes)
    assert_spmv_ok(y, data, idx, ptr, (spec.n_rows, spec.n_cols), x, what=f"lanes {lanes}")


def test_duplicates_unsorted_and_index_widths(cuda, fsb_lib):
    lens = [9, 0, 300, 5, 2500, 1]
    data, idx, ptr = handmade_csr(3, lens, 64, sort=False, replace=True)  # duplicates, unsorted
    x = np.random.default_rng(4).uniform(-1, 1, 64).astype(np.float32)
    shape = (len(lens), 64)
    for algo in ALGOS:
        y32 = spmv(data, idx, ptr, shape, x, algo=algo)
        assert_spmv_ok(y32, data, idx, ptr, shape, x, what="dups")
        # int64 indices / int64 indptr describe the same matrix: the result must be the same bits
        y64 = spmv(data, idx.astype(np.int64), ptr.astype(np.int64), shape, x, algo=algo)
        assert np.array_equal(y32, y64)
        # any integer indptr dtype is accepted for SpMV, as in the reference
        y16 = spmv(data, idx, ptr.astype(np.int16), shape, x, algo=algo)
        assert np.array_equal(y32, y16)


def test_determinism_and_exact_scaling(cuda, fsb_lib):
    spec = S.config_spec("c3").scaled(1 << 16)
    d, i, p = (t for t in S.generate_csr(spec, "cuda:0"))
    x = S.dense_vector(spec, spec.n_cols, "cuda:0")
    for algo in ALGOS:
        with env(FSB_SPMV_ALGO=algo):
            prep = fs.prepare_spmv_csr(d, i, p, (spec.n_rows, spec.n_cols))
            y1 = fs.flagsparse_spmv_csr(x=x, prepared=prep).clone()
            y2 = fs.flagsparse_spmv_csr(x=x, prepared=prep).clone()
            y4 = fs.flagsparse_spmv_csr(x=x * 4, prepared=prep)
        assert torch.equal(y1, y2)          # no atomics: same bits every time
        assert torch.equal(y4, y1 * 4)      # scaling x by a power of two scales y exactly


def test_out_argument_and_return_time(cuda, fsb_lib):
    g = load_golden(golden_files("spmv")[0])
    d, i, p, x = dev(g["data"]), dev(g["indices"]), dev(g["indptr"]), dev(g["x"])
    n = g["shape"][0]
    out = torch.full((n,), 7.0, dtype=d.dtype, device="cuda:0")
    y = fs.flagsparse_spmv_csr(d, i, p, x, g["shape"], out=out)
    assert y.data_ptr() == out.data_ptr()
    assert_spmv_ok(out.cpu().numpy(), g["data"], g["indices"], g["indptr"], g["shape"], g["x"])
    # non-contiguous out: filled through a copy, still the same object back
    wide = torch.zeros((n, 2), dtype=d.dtype, device="cuda:0")
    y2 = fs.flagsparse_spmv_csr(d, i, p, x, g["shape"], out=wide[:, 0])
    assert y2.data_ptr() == wide.data_ptr() and torch.equal(wide[:, 0], out)
    with pytest.raises(ValueError):
        fs.flagsparse_spmv_csr(d, i, p, x, g["shape"], out=torch.empty(n + 1, dtype=d.dtype, device="cuda:0"))
    with pytest.raises(ValueError):
        fs.flagsparse_spmv_csr(d, i, p, x, g["shape"], out=torch.empty(n, dtype=torch.float64, device="cuda:0"))
    y3, ms = fs.flagsparse_spmv_csr(d, i, p, x, g["shape"], return_time=True)
    assert ms > 0 and torch.equal(y3, out)


def test_c_abi_direct_call_with_unaligned_arrays(cuda, fsb_lib):
    """Straight ctypes calls: element-aligned but not 16-byte aligned data/indices take the scalar-load path."""
    spec = S.config_spec("c2").scaled(4000)
    data, idx, ptr = S.generate_csr(spec, None)
    x = S.dense_vector(spec, spec.n_cols)
    nnz = data.size
    dpad, ipad = dev(np.concatenate([[0], data]).astype(np.float32)), dev(np.concatenate([[0], idx]).astype(np.int32))
    d1, i1 = dpad[1:], ipad[1:]
    assert d1.data_ptr() % 16 == 4
    p, xd = dev(ptr), dev(x)
    y = torch.empty(spec.n_rows, dtype=torch.float32, device="cuda:0")
    T = fsb_lib.fsb_spmv_tile_nnz(_lib.FSB_F32, 0)
    n_tiles = fsb_lib.fsb_csr_num_tiles(nnz, T)
    plan = torch.empty(n_tiles + 1, dtype=torch.int32, device="cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    assert fsb_lib.fsb_csr_tile_plan(_lib.FSB_I32, p.data_ptr(), spec.n_rows, nnz, T, plan.data_ptr(), st) == 0
    nbytes = fsb_lib.fsb_spmv_csr_scratch_bytes(_lib.FSB_F32, nnz, 0)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda:0")
    rc = fsb_lib.fsb_spmv_csr(_lib.FSB_F32, _lib.FSB_I32, _lib.FSB_I32, d1.data_ptr(), i1.data_ptr(), p.data_ptr(),
                              xd.data_ptr(), y.data_ptr(), spec.n_rows, spec.n_cols, nnz, _lib.FSB_SPMV_STREAM, 0,
                              plan.data_ptr(), scratch.data_ptr(), nbytes, st)
    assert rc == 0
    assert_spmv_ok(y.cpu().numpy(), data, idx, ptr, (spec.n_rows, spec.n_cols), x, what="unaligned")
    # the vector kernel on the same unaligned arrays (scalar loads) and on aligned ones (128-bit groups)
    for dd, ii in ((d1, i1), (dev(data), dev(idx))):
        y.fill_(float("nan"))
        rc = fsb_lib.fsb_spmv_csr(_lib.FSB_F32, _lib.FSB_I32, _lib.FSB_I32, dd.data_ptr(), ii.data_ptr(), p.data_ptr(),
                                  xd.data_ptr(), y.data_ptr(), spec.n_rows, spec.n_cols, nnz, _lib.FSB_SPMV_VECTOR, 0,
                                  None, None, 0, st)
        assert rc == 0
        assert_spmv_ok(y.cpu().numpy(), data, idx, ptr, (spec.n_rows, spec.n_cols), x, what="vector direct")
    # too little scratch and a misaligned value pointer are refused, not launched
    assert fsb_lib.fsb_spmv_csr(_lib.FSB_F32, _lib.FSB_I32, _lib.FSB_I32, d1.data_ptr(), i1.data_ptr(), p.data_ptr(),
                                xd.data_ptr(), y.data_ptr(), spec.n_rows, spec.n_cols, nnz, _lib.FSB_SPMV_STREAM, 0,
                                plan.data_ptr(), scratch.data_ptr(), 8, st) == -4
    assert fsb_lib.fsb_spmv_csr(_lib.FSB_F32, _lib.FSB_I32, _lib.FSB_I32, d1.data_ptr() + 2, i1.data_ptr(), p.data_ptr(),
                                xd.data_ptr(), y.data_ptr(), spec.n_rows, spec.n_cols, nnz, _lib.FSB_SPMV_VECTOR, 0,
                                None, None, 0, st) == -3
    # the plan kernel agrees with numpy's searchsorted
    want = np.searchsorted(ptr.astype(np.int64), np.arange(n_tiles + 1) * T, side="right") - 1
    want[0], want[-1] = 0, spec.n_rows
    assert np.array_equal(plan.cpu().numpy(), want)


def test_analysis_statistics(cuda, fsb_lib):
    lens = [0, 700, 0, 0, 1, 2500, 31, 32, 33, 0, 4097, 1]
    data, idx, ptr = handmade_csr(9, lens, 8192)
    prep = fs.prepare_spmv_csr(dev(data), dev(idx), dev(ptr), (len(lens), 8192))
    s = prep.stats
    assert (s.ptr_first, s.ptr_last, s.n_decreasing) == (0, sum(lens), 0)
    assert (s.min_index, s.max_index) == (int(idx.min()), int(idx.max()))
    assert s.max_row_nnz == 4097 and s.n_empty_rows == lens.count(0)
    assert prep.max_row_nnz == 4097 and prep.shape == (len(lens), 8192) and prep.supports_opt
    assert prep.kernel_indices.dtype == torch.int32 and prep.kernel_indptr.dtype == torch.int32
    p64 = fs.prepare_spmv_csr(dev(data), dev(idx.astype(np.int64)), dev(ptr.astype(np.int64)), (len(lens), 8192))
    assert p64.kernel_indices.dtype == torch.int32  # narrowed like the reference does


# ---- the benchmark configurations -----------------------------------------------------------------------
@pytest.mark.parametrize("name,rows", [("c2", 1 << 17), ("c3", 1 << 19), ("c5", 1 << 17), ("c5", 1 << 22)])
def test_configs_reduced_full_oracle(cuda, fsb_lib, name, rows):
    # c5 at 2^22 rows keeps the full band of +-2^20 columns: 256 column chunks per row block, a few thousand entries
    # per unit -- the geometry of the full-size matrix on the panel kernel
    spec = S.config_spec(name).scaled(rows)
    pdt = "int64" if name == "c5" else "int32"
    d, i, p = S.generate_csr(spec, "cuda:0", indptr_dtype=pdt)
    x = S.dense_vector(spec, spec.n_cols, "cuda:0")
    dn, inn, pn, xn = d.cpu().numpy(), i.cpu().numpy(), p.cpu().numpy(), x.cpu().numpy()
    # the panel kernel where the columns are banded (forcing it on uniform columns would build a unit per chunk)
    for algo in ALGOS + (["panel"] if name != "c3" else []):
        with env(FSB_SPMV_ALGO=algo):
            y = fs.flagsparse_spmv_csr(d, i, p, x, (spec.n_rows, spec.n_cols))
        assert_spmv_ok(y.cpu().numpy(), dn, inn, pn, (spec.n_rows, spec.n_cols), xn, what=f"{name}/{algo}")


def test_config_c1_full(cuda, fsb_lib):
    spec = S.config_spec("c1")
    data, idx, ptr = S.generate_csr(spec, None)
    x = S.dense_vector(spec, spec.n_cols)
    for algo in (None, "vector", "stream"):
        y = spmv(data, idx, ptr, (4096, 4096), x, algo=algo)
        assert_spmv_ok(y, data, idx, ptr, (4096, 4096), x, what=f"c1/{algo}")


@pytest.mark.parametrize("vdt,idt", [("float32", "int32"), ("float64", "int64")])
def test_config_c2_full_size(cuda, fsb_lib, vdt, idt):
    spec = S.config_spec("c2")
    d, i, p = S.generate_csr(spec, "cuda:0", value_dtype=vdt, index_dtype=idt, indptr_dtype=idt)
    x = S.dense_vector(spec, spec.n_cols, "cuda:0", value_dtype=vdt)
    prep = fs.prepare_spmv_csr(d, i, p, (spec.n_rows, spec.n_cols))
    assert prep.algo == _lib.FSB_SPMV_PANEL  # uniform row lengths inside a narrow band
    y = fs.flagsparse_spmv_csr(x=x, prepared=prep)
    worst = check_spmv_blocks(spec, y, x.cpu().numpy(), sample_blocks(spec.n_rows, 24, 2048), vdt, idt, idt)
    assert int(prep.panel.status.item()) == 0
    for other in ("stream", "vector"):
        with env(FSB_SPMV_ALGO=other):
            ys = fs.flagsparse_spmv_csr(d, i, p, x, (spec.n_rows, spec.n_cols))
        check_spmv_blocks(spec, ys, x.cpu().numpy(), sample_blocks(spec.n_rows, 8, 2048, seed=1), vdt, idt, idt)
    assert torch.equal(fs.flagsparse_spmv_csr(x=x * 2, prepared=prep), y * 2)
    assert torch.equal(fs.flagsparse_spmv_csr(x=x, prepared=prep), y)
    print(f"c2 {vdt}: nnz {d.numel()}, worst bound ratio {worst:.2e}")


def test_config_c3_full_size(cuda, fsb_lib):
    spec = S.config_spec("c3")
    d, i, p = S.generate_csr(spec, "cuda:0")
    x = S.dense_vector(spec, spec.n_cols, "cuda:0")
    prep = fs.prepare_spmv_csr(d, i, p, (spec.n_rows, spec.n_cols))
    y = fs.flagsparse_spmv_csr(x=x, prepared=prep)
    xn = x.cpu().numpy()
    blocks = sample_blocks(spec.n_rows, 16, 2048)
    # plus the longest rows of the matrix, one by one
    lens = (p[1:] - p[:-1])
    blocks += [(int(r), int(r) + 1) for r in torch.topk(lens, 6).indices.tolist()]
    worst = check_spmv_blocks(spec, y, xn, blocks)
    assert torch.equal(fs.flagsparse_spmv_csr(x=x, prepared=prep), y)
    assert int(lens.max()) > 60000
    print(f"c3: nnz {d.numel()}, longest row {int(lens.max())}, worst bound ratio {worst:.2e}")


def test_config_c5_full_size_on_the_panel_kernel(cuda, fsb_lib):
    """The 2^26-row matrix of the sharded configuration on one GPU, through the kernel the benchmark times on it:
    host-regenerated row blocks (the ends, around the row where the entry count passes 2^31, random ones), the
    wait-status word, bit equality of two calls and exact scaling."""
    if torch.cuda.get_device_properties(0).total_memory < 80 * 2**30:
        pytest.skip("needs about 60 GB of device memory")
    spec = S.config_spec("c5")
    d, i, p = S.generate_csr(spec, "cuda:0", indptr_dtype="int64")
    assert d.numel() > 2**31 - 2**24 and p.dtype == torch.int64
    x = S.dense_vector(spec, spec.n_cols, "cuda:0")
    prep = fs.prepare_spmv_csr(d, i, p, (spec.n_rows, spec.n_cols))
    assert prep.algo == _lib.FSB_SPMV_PANEL and prep.panel is not None
    lay = prep.panel
    assert lay.n_units // lay.n_row_blocks > 200            # every row block spans the whole band of chunks
    y = fs.flagsparse_spmv_csr(x=x, prepared=prep)
    prep.check_status()
    edge = int(torch.searchsorted(p, torch.tensor([2**31 - 1], device=p.device))[0]) if d.numel() >= 2**31 else None
    blocks = sample_blocks(spec.n_rows, 8, 2048)
    if edge is not None:
        blocks.append((max(0, edge - 1024), min(spec.n_rows, edge + 1024)))
    blocks.append((lay.rb_rows - 1024, lay.rb_rows + 1024))  # across the first row-block boundary
    worst = check_spmv_blocks(spec, y, x.cpu().numpy(), blocks, indptr_dtype="int64")
    assert torch.equal(fs.flagsparse_spmv_csr(x=x, prepared=prep), y)
    assert torch.equal(fs.flagsparse_spmv_csr(x=x * 2, prepared=prep), y * 2)
    print(f"c5 panel: nnz {d.numel()}, rounds {lay.rounds}, flags {lay.flags}, longest run {lay.max_run}, "
          f"worst bound ratio {worst:.2e}")


def test_panel_kernel_with_long_runs(cuda, fsb_lib):
    """Rows of 48 consecutive columns (block-structured matrices): runs longer than a lane's rounds, summed through
    the kernel's segmented path; every piece size."""
    n, width, n_cols = 200000, 48, 300000
    rng = np.random.default_rng(3)
    start = np.clip(np.arange(n) * n_cols // n + rng.integers(-2000, 2000, n), 0, n_cols - width)
    idx = (start[:, None] + np.arange(width)[None, :]).reshape(-1).astype(np.int32)
    ptr = (np.arange(n + 1, dtype=np.int64) * width).astype(np.int32)
    data = rng.uniform(-1, 1, idx.size).astype(np.float32)
    x = rng.uniform(-1, 1, n_cols).astype(np.float32)
    from flagsparse_b200 import panel as P

    for rounds in (None, 4, 8, 16):
        with env(FSB_SPMV_ALGO="panel", FSB_PANEL_ROUNDS=rounds):
            prep = fs.prepare_spmv_csr(dev(data), dev(idx), dev(ptr), (n, n_cols))
        assert prep.panel is not None and prep.panel.flags & P.FLAG_LONG_RUNS and prep.panel.max_run == width
        assert prep.panel.rounds == (rounds or 16)
        y = fs.flagsparse_spmv_csr(x=dev(x), prepared=prep)
        assert_spmv_ok(y.cpu().numpy(), data, idx, ptr, (n, n_cols), x, what=f"48-entry runs, rounds {rounds}")
        assert torch.equal(fs.flagsparse_spmv_csr(x=dev(x), prepared=prep), y)
        prep.check_status()


@pytest.mark.parametrize("rounds", [4, 8, 16])
@pytest.mark.parametrize("vdt", ["float32", "float64"])
def test_panel_piece_sizes(cuda, fsb_lib, rounds, vdt):
    spec = S.config_spec("c5").scaled(1 << 20)
    d, i, p = S.generate_csr(spec, "cuda:0", value_dtype=vdt)
    x = S.dense_vector(spec, spec.n_cols, "cuda:0", value_dtype=vdt)
    with env(FSB_SPMV_ALGO="panel", FSB_PANEL_ROUNDS=rounds):
        prep = fs.prepare_spmv_csr(d, i, p, (spec.n_rows, spec.n_cols))
    assert prep.panel.rounds == rounds
    y = fs.flagsparse_spmv_csr(x=x, prepared=prep)
    assert_spmv_ok(y.cpu().numpy(), d.cpu().numpy(), i.cpu().numpy(), p.cpu().numpy(), (spec.n_rows, spec.n_cols),
                   x.cpu().numpy(), what=f"panel rounds {rounds} {vdt}")
    prep.check_status()
    # the same product launched in three slices of row blocks (what the sharded driver does)
    from flagsparse_b200 import panel as P
    from flagsparse_b200._common import _stream_ptr

    y2 = torch.full_like(y, float("nan"))
    nb = prep.panel.n_row_blocks
    for b0, b1 in ((0, nb // 3), (nb // 3, nb // 3), (nb // 3, nb)):
        P.launch_panel(prep.panel, x, y2, spec.n_rows, spec.n_cols, _stream_ptr(x.device), b0, b1)
    assert torch.equal(y2, y)


def test_a_wait_that_runs_out_is_reported_to_the_caller(cuda, fsb_lib):
    """The kernel's bounded wait on a copy of x, made to run out (the kernel is told to expect 16 bytes that never
    arrive and to give up after a short spin): it returns, sets its status word, and the next look at the prepared
    matrix raises instead of handing on an incomplete y.  Nothing faults and nothing hangs; the following product is
    correct again."""
    from flagsparse_b200 import panel as P

    spec = S.config_spec("c2").scaled(1 << 17)
    d, i, p = S.generate_csr(spec, "cuda:0")
    x = S.dense_vector(spec, spec.n_cols, "cuda:0")
    with env(FSB_SPMV_ALGO="panel"):
        prep = fs.prepare_spmv_csr(d, i, p, (spec.n_rows, spec.n_cols))
    good = fs.flagsparse_spmv_csr(x=x, prepared=prep)
    prep.check_status()
    prep.panel.flags |= P.FLAG_DEBUG_TIMEOUT
    fs.flagsparse_spmv_csr(x=x, prepared=prep)
    with pytest.raises(RuntimeError, match="wait ran out"):
        prep.check_status()
    assert int(prep.panel.status.item()) == 0               # the word was reset
    with pytest.raises(RuntimeError, match="wait ran out"):
        fs.flagsparse_spmv_csr(x=x, prepared=prep, return_time=True)
    # the failure is also seen, without any wait, by the next product on the same matrix
    fs.flagsparse_spmv_csr(x=x, prepared=prep)
    torch.cuda.synchronize()
    prep.panel.flags &= ~P.FLAG_DEBUG_TIMEOUT
    with pytest.raises(RuntimeError, match="wait ran out"):
        fs.flagsparse_spmv_csr(x=x, prepared=prep)
    assert torch.equal(fs.flagsparse_spmv_csr(x=x, prepared=prep), good)
    prep.check_status()


def test_more_than_2_31_entries(cuda, fsb_lib):
    """A matrix whose nnz does not fit int32 (2^26 rows, Poisson(34) rows, 2.28e9 entries, int64 indptr): both
    kernels against host-regenerated row blocks, including blocks whose offsets lie beyond 2^31."""
    if torch.cuda.get_device_properties(0).total_memory < 60 * 2**30:
        pytest.skip("needs about 40 GB of device memory")
    spec = S.CsrSpec("c5x", 1 << 26, 1 << 26, ("poisson", 34.0), ("band", 1 << 20), False, 0)
    d, i, p = S.generate_csr(spec, "cuda:0", indptr_dtype="int64")
    nnz = d.numel()
    assert nnz > 2**31 and p.dtype == torch.int64 and int(p[-1]) == nnz
    x = S.dense_vector(spec, spec.n_cols, "cuda:0")
    xn = x.cpu().numpy()
    blocks = sample_blocks(spec.n_rows, 6, 2048) + [(spec.n_rows - 4096, spec.n_rows), (63_500_000, 63_502_048)]
    assert int(p[63_500_000]) > 2**31 - 2**27  # around and past the int32 boundary
    for algo in ("vector", "stream"):
        with env(FSB_SPMV_ALGO=algo):
            prep = fs.prepare_spmv_csr(d, i, p, (spec.n_rows, spec.n_cols))
            assert prep.kernel_indptr.dtype == torch.int64
            y = fs.flagsparse_spmv_csr(x=x, prepared=prep)
        check_spmv_blocks(spec, y, xn, blocks, indptr_dtype="int64")
        del prep, y
