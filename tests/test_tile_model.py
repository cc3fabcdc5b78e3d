"""The tiling scheme of the CUDA kernels, restated in numpy (helpers.tiled_spmv_model): plan ownership,
partial rows, carries and the fix-up give every row exactly one write and the right sum.  CPU only."""

import numpy as np
import pytest

from helpers import handmade_csr, tile_plan_model, tiled_spmv_model
from oracle import csr_oracle as O

CASES = {
    "uniform": [7] * 40,
    "ragged": [0, 0, 3, 0, 1, 300, 0, 0, 64, 65, 0, 33, 32, 31, 1, 1, 0, 700, 0, 0, 2, 0],
    "leading_empty": [0] * 9 + [5, 0, 0, 12],
    "trailing_empty": [16, 16, 0, 0, 0],
    "one_long": [1000],
    "long_between_empty": [0, 0, 513, 0, 0],
    "exact_tiles": [16] * 8,
    "single_entry": [1],
    "all_ones": [1] * 70,
}


@pytest.mark.parametrize("tile", [8, 16, 64, 256])
@pytest.mark.parametrize("name", sorted(CASES))
def test_model_matches_oracle(name, tile):
    lens = CASES[name]
    n_cols = 1024
    data, idx, ptr = handmade_csr(1, lens, n_cols, value_dtype=np.float64)
    x = np.random.default_rng(2).uniform(-1, 1, n_cols)
    y, written = tiled_spmv_model(data, idx, ptr, x, tile)
    ref, mag = O.spmv_f64(data, idx, ptr, (len(lens), n_cols), x)
    assert np.all(written == 1), written
    assert np.allclose(y, ref, rtol=0, atol=1e-12)


def test_plan_properties():
    lens = CASES["ragged"]
    _, _, ptr = handmade_csr(1, lens, 1024)
    for tile in (8, 64, 2048):
        plan = tile_plan_model(ptr, tile)
        assert plan[0] == 0 and plan[-1] == len(lens)
        assert np.all(np.diff(plan) >= 0)
        for t in range(1, len(plan) - 1):
            r = plan[t]
            assert ptr[r] <= t * tile < ptr[r + 1]  # the row that holds nnz number t*tile
