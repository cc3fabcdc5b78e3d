"""Row-sharded SpMV on GPUs: the single-rank path always, the 2-rank NCCL and peer-store paths when the box
has two GPUs.  Ranks are child processes, one per GPU."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flagsparse_b200 import synthetic as S
from flagsparse_b200.sharded import ShardedCsrSpmv, partition_rows_by_nnz

pytestmark = pytest.mark.gpu


def test_single_rank(cuda, fsb_lib):
    from helpers import assert_spmv_ok

    spec = S.config_spec("c5").scaled(1 << 15)
    d, i, p = S.generate_csr(spec, "cuda:0", indptr_dtype="int64")
    x = S.dense_vector(spec, spec.n_cols, "cuda:0")
    op = ShardedCsrSpmv(d, i, p, 0, (spec.n_rows, spec.n_cols))
    y = op.matvec(x)
    assert op.mode == "nccl" and op.row_ranges == [(0, spec.n_rows)]
    assert_spmv_ok(y.cpu().numpy(), d.cpu().numpy(), i.cpu().numpy(), p.cpu().numpy(), (spec.n_rows, spec.n_cols),
                   x.cpu().numpy())


def _worker(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
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
        # the peer-store epilogue exists for the vector kernel (picked for these uniform rows), the stream kernel
        # and the panel kernel
        for mode, algo in (("nccl", None), ("peer", None), ("peer", "stream"), ("peer", "panel"), ("nccl", "panel")):
            if algo:
                os.environ["FSB_SPMV_ALGO"] = algo
            try:
                op = ShardedCsrSpmv(d, i, p, r0, (spec.n_rows, spec.n_cols), mode=mode)
            finally:
                os.environ.pop("FSB_SPMV_ALGO", None)
            y = None
            for rep in range(3):
                y = op.matvec(x * float(rep + 1))
            torch.cuda.synchronize()
            results[(mode, algo)] = y.clone()
        # vector kernel with local stores and with peer stores: the same sums, the same bits
        assert torch.equal(results[("nccl", None)], results[("peer", None)])
        # the stream kernel adds in another order: held to the oracle bound by the parent, close to the others here
        assert torch.allclose(results[("nccl", None)], results[("peer", "stream")], rtol=1e-4, atol=1e-4)
        # the panel kernel with local stores + NCCL and with peer stores: the same sums, the same bits
        assert torch.equal(results[("nccl", "panel")], results[("peer", "panel")])
        assert torch.allclose(results[("nccl", None)], results[("peer", "panel")], rtol=1e-4, atol=1e-4)
        np.save(os.path.join(result_dir, f"p{rank}.npy"), results[("peer", "panel")].cpu().numpy())
        np.save(os.path.join(result_dir, f"y{rank}.npy"), results[("peer", None)].cpu().numpy())
        np.save(os.path.join(result_dir, f"n{rank}.npy"), results[("peer", "stream")].cpu().numpy())
    finally:
        dist.destroy_process_group()


def test_two_ranks_nccl_and_peer(cuda, fsb_lib, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from helpers import assert_spmv_ok

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    y0, y1 = np.load(tmp_path / "y0.npy"), np.load(tmp_path / "y1.npy")
    assert np.array_equal(y0, y1)  # every rank holds the same assembled vector
    n0, n1 = np.load(tmp_path / "n0.npy"), np.load(tmp_path / "n1.npy")
    assert np.array_equal(n0, n1)
    spec = S.config_spec("c5").scaled(1 << 18)
    d, i, p = S.generate_csr(spec, None, indptr_dtype="int64")
    x = S.dense_vector(spec, spec.n_cols) * np.float32(3.0)
    assert_spmv_ok(y0, d, i, p, (spec.n_rows, spec.n_cols), x, what="two ranks, peer stores, vector kernel")
    assert_spmv_ok(n0, d, i, p, (spec.n_rows, spec.n_cols), x, what="two ranks, peer stores, stream kernel")
    p0, p1 = np.load(tmp_path / "p0.npy"), np.load(tmp_path / "p1.npy")
    assert np.array_equal(p0, p1)
    assert_spmv_ok(p0, d, i, p, (spec.n_rows, spec.n_cols), x, what="two ranks, peer stores, panel kernel")
