"""Row-sharded SpMV and SpMM on GPUs: the single-rank path always, the 2-rank paths (NCCL all-gather, slices
pushed by the copy engines, peer stores fused into the kernel) when the box has two GPUs.  Ranks are child
processes, one per GPU."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flagsparse_b200 import synthetic as S
from flagsparse_b200.sharded import ShardedCsrSpmm, ShardedCsrSpmv, partition_rows_by_nnz

pytestmark = pytest.mark.gpu


def test_single_rank(cuda, fsb_lib):
    from helpers import assert_spmm_ok, assert_spmv_ok

    spec = S.config_spec("c5").scaled(1 << 15)
    d, i, p = S.generate_csr(spec, "cuda:0", indptr_dtype="int64")
    x = S.dense_vector(spec, spec.n_cols, "cuda:0")
    op = ShardedCsrSpmv(d, i, p, 0, (spec.n_rows, spec.n_cols))
    y = op.matvec(x)
    assert op.mode == "nccl" and op.row_ranges == [(0, spec.n_rows)]
    host = (d.cpu().numpy(), i.cpu().numpy(), p.cpu().numpy(), (spec.n_rows, spec.n_cols))
    assert_spmv_ok(y.cpu().numpy(), *host, x.cpu().numpy())
    B = S.dense_vector(spec, spec.n_cols, "cuda:0", n_dense=24)
    mm = ShardedCsrSpmm(d, i, p, 0, (spec.n_rows, spec.n_cols))
    assert mm.mode == "nccl"
    assert_spmm_ok(mm.matmul(B).cpu().numpy(), *host, B.cpu().numpy())


SPMV_CASES = (("nccl", None), ("peer", None), ("fused", None), ("fused", "stream"), ("peer", "panel"),
              ("nccl", "panel"), ("nccl-chunks", "panel"), ("peer", "stream"))


def _worker(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      FSB_SHARD_WAVE_BLOCKS="16")     # the small shard's panel layout spans several "waves"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        device = f"cuda:{rank}"
        spec = S.config_spec("c5").scaled(1 << 18)
        lens = S.row_lengths(spec, S._ops(device), 0, spec.n_rows)
        ptr = torch.zeros(spec.n_rows + 1, dtype=torch.int64, device=device)
        ptr[1:] = torch.cumsum(lens, 0)
        b = partition_rows_by_nnz(ptr, world)
        r0, r1 = b[rank], b[rank + 1]
        d, i, p = S.generate_csr(spec, device, indptr_dtype="int64", row_range=(r0, r1))
        x = S.dense_vector(spec, spec.n_cols, device)
        results = {}
        for mode, algo in SPMV_CASES:
            if algo:
                os.environ["FSB_SPMV_ALGO"] = algo
            if mode == "nccl-chunks":                   # slice j gathered while slice j + 1 is computed
                os.environ["FSB_NCCL_CHUNKS"] = "1"
            try:
                op = ShardedCsrSpmv(d, i, p, r0, (spec.n_rows, spec.n_cols), mode=mode.split("-")[0])
            finally:
                os.environ.pop("FSB_SPMV_ALGO", None)
                os.environ.pop("FSB_NCCL_CHUNKS", None)
            assert (op._nccl_chunks is not None) == (mode == "nccl-chunks")
            if mode == "nccl-chunks":
                assert len(op._nccl_chunks) > 1
            if (mode, algo) == ("peer", "panel"):
                assert len(op._slices) > 1, op._slices       # slices pushed while later ones are computed
            y = None
            for rep in range(3):
                y = op.matvec(x * float(rep + 1))
            torch.cuda.synchronize()
            results[(mode, algo)] = y.clone()
        # one kernel, three ways of assembling y: the same sums, the same bits
        assert torch.equal(results[("nccl", None)], results[("peer", None)])
        assert torch.equal(results[("nccl", None)], results[("fused", None)])
        assert torch.equal(results[("nccl", "panel")], results[("peer", "panel")])
        assert torch.equal(results[("nccl-chunks", "panel")], results[("peer", "panel")])
        assert torch.equal(results[("fused", "stream")], results[("peer", "stream")])
        # other kernels add in another order: held to the oracle bound by the parent, close to each other here
        assert torch.allclose(results[("nccl", None)], results[("fused", "stream")], rtol=1e-4, atol=1e-4)
        assert torch.allclose(results[("nccl", None)], results[("peer", "panel")], rtol=1e-4, atol=1e-4)
        for name, key in (("p", ("peer", "panel")), ("y", ("peer", None)), ("n", ("fused", "stream"))):
            np.save(os.path.join(result_dir, f"{name}{rank}.npy"), results[key].cpu().numpy())
        # SpMM: B replicated, C assembled on every rank
        B = S.dense_vector(spec, spec.n_cols, device, n_dense=40)
        cs = {}
        for mode in ("nccl", "peer"):
            mm = ShardedCsrSpmm(d, i, p, r0, (spec.n_rows, spec.n_cols), mode=mode)
            C = None
            for rep in range(2):
                C = mm.matmul(B * float(rep + 1))
            torch.cuda.synchronize()
            cs[mode] = C.clone()
        assert cs["peer"].shape == (spec.n_rows, 40)
        assert torch.allclose(cs["nccl"], cs["peer"], rtol=1e-4, atol=1e-4)
        np.save(os.path.join(result_dir, f"c{rank}.npy"), cs["peer"].cpu().numpy())
    finally:
        dist.destroy_process_group()


def test_two_ranks(cuda, fsb_lib, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from helpers import assert_spmm_ok, assert_spmv_ok

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    spec = S.config_spec("c5").scaled(1 << 18)
    d, i, p = S.generate_csr(spec, None, indptr_dtype="int64")
    x = S.dense_vector(spec, spec.n_cols) * np.float32(3.0)
    shape = (spec.n_rows, spec.n_cols)
    for name, what in (("y", "vector kernel, pushed"), ("n", "stream kernel, fused peer stores"),
                       ("p", "panel kernel, slices pushed")):
        a, b = np.load(tmp_path / f"{name}0.npy"), np.load(tmp_path / f"{name}1.npy")
        assert np.array_equal(a, b), what             # every rank holds the same assembled vector
        assert_spmv_ok(a, d, i, p, shape, x, what=f"two ranks, {what}")
    c0, c1 = np.load(tmp_path / "c0.npy"), np.load(tmp_path / "c1.npy")
    assert np.array_equal(c0, c1)
    B = S.dense_vector(spec, spec.n_cols, n_dense=40) * np.float32(2.0)
    assert_spmm_ok(c0, d, i, p, shape, B, what="two ranks, SpMM, sub-shards pushed")
