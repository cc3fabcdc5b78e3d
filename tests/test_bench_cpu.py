"""bench.py without a GPU: the CPU arm (`--impl reference`) prints the contract's JSON line, ranks other than 0
stay silent, and the byte / workload bookkeeping agrees with the formulas the roofline figures are built on."""

import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _run(extra_env=None, *args):
    env = dict(os.environ, **(extra_env or {}))
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          env=env, timeout=600, cwd=ROOT)


def test_reference_arm_prints_the_contract_line(fsb_lib):
    out = _run(None, "--impl", "reference", "--steps", "1", "--warmup", "1", "--workload", "c2")
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["value"] > 0
    assert line["config"]["name"] == "c2" and "workload" in line["config"] and line["vs_baseline"] is None
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"] and "rows" in line["cpu_baseline"]["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_defaults_to_the_sharded_workload(fsb_lib):
    # the default workload is the same at every --gpus N (c5); the timed sample is a slice from the middle of the band
    out = _run(None, "--impl", "reference", "--steps", "1", "--warmup", "1", "--cpu-rows-log2", "12")
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["config"]["name"] == "c5" and line["impl"] == "reference" and line["value"] > 0
    assert "rows [33552384, 33556480) of 67108864" in line["cpu_baseline"]["sample"]


def test_reference_arm_runs_on_rank_zero_only():
    out = _run({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}, "--impl", "reference", "--gpus", "2", "--steps", "1",
               "--warmup", "1")
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_byte_formulas():
    import bench

    # A once, indptr once, x once, y once
    assert bench.spmv_bytes(10, 20, 100, 4, 4, 8) == 100 * 8 + 11 * 8 + 20 * 4 + 10 * 4
    assert bench.spmm_bytes(10, 20, 100, 32, 4, 4, 8) == 100 * 8 + 11 * 8 + 20 * 32 * 4 + 10 * 32 * 4
    assert set(bench.NCU_TRAFFIC_BYTES) <= set(bench.SPMV_WORKLOADS) | set(bench.SPMM_WORKLOADS)
    for w in bench.NCU_TRAFFIC_BYTES:   # a capture is reported only for the kernel source it was taken on
        assert bench.measured_traffic(w) in (None, bench.NCU_TRAFFIC_BYTES[w][0])
    assert bench.measured_traffic("c1") is None
    for w in list(bench.SPMV_WORKLOADS) + list(bench.SPMM_WORKLOADS):
        cfg = bench.workload_config(w, 1)
        assert cfg["name"] == w and isinstance(cfg["workload"], str) and "model" not in cfg
    assert "parallelism" in bench.workload_config("c5", 8)
    # blocks of the in-run check: both ends, around every mark, inside the matrix
    blocks = bench.parity_blocks(100000, [50000, 99999, 10], block_rows=2048, extra=2)
    assert blocks[0] == (0, 2048) and blocks[-1] == (100000 - 2048, 100000)
    assert any(a <= 50000 < b for a, b in blocks) and all(0 <= a < b <= 100000 for a, b in blocks)
    assert bench.parity_blocks(100, [], block_rows=2048, extra=1) == [(0, 100)]
    peak, kind = bench.measured_peak()
    assert peak > 1000 and kind in ("measured", "fallback")


def test_bench_needs_a_gpu_for_the_product_arm():
    import torch

    if torch.cuda.is_available():
        pytest.skip("this check is for machines without a GPU")
    out = _run(None, "--steps", "1", "--warmup", "1")
    assert out.returncode != 0 and "CUDA" in (out.stderr + out.stdout)
