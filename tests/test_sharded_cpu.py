"""Host logic of the row-sharded driver on CPU ranks (gloo, world size 2 and 3): nnz-balanced partition,
shard bookkeeping, assembly of y on every rank, and what happens when a rank misbehaves.  The local product
is supplied by the test (the oracle), so no GPU is involved."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flagsparse_b200 import synthetic as S
from flagsparse_b200.sharded import ShardedCsrSpmm, ShardedCsrSpmv, partition_rows_by_nnz, slice_plan


def test_partition_is_balanced_and_covers():
    spec = S.config_spec("c3").scaled(1 << 14)
    _, _, ptr = S.generate_csr(spec, None, indptr_dtype="int64")
    nnz = int(ptr[-1])
    for parts in (1, 2, 3, 8):
        b = partition_rows_by_nnz(ptr, parts)
        assert b[0] == 0 and b[-1] == spec.n_rows and len(b) == parts + 1
        assert all(b[i] <= b[i + 1] for i in range(parts))
        sizes = [int(ptr[b[i + 1]] - ptr[b[i]]) for i in range(parts)]
        assert sum(sizes) == nnz
        longest = int(np.diff(ptr).max())
        assert max(sizes) <= nnz // parts + longest + 1  # off by at most one row
        assert b == partition_rows_by_nnz(torch.from_numpy(ptr), parts)
    # degenerate inputs
    assert partition_rows_by_nnz(np.zeros(1, dtype=np.int64), 4) == [0, 0, 0, 0, 0]
    assert partition_rows_by_nnz(np.zeros(6, dtype=np.int64), 2) == [0, 0, 5]
    assert partition_rows_by_nnz(np.array([0, 10]), 4) == [0, 1, 1, 1, 1]
    with pytest.raises(ValueError):
        partition_rows_by_nnz(ptr, 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, scenario, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import csr_oracle as O

        spec = S.config_spec("c2").scaled(3000)
        data, idx, ptr = S.generate_csr(spec, None, indptr_dtype="int64")
        x = S.dense_vector(spec, spec.n_cols)
        bounds = partition_rows_by_nnz(ptr, world)
        r0, r1 = bounds[rank], bounds[rank + 1]
        if scenario == "wrong_cover" and rank == 1:
            r1 -= 1  # this rank claims one row too few
        ld, li, lp = S.generate_csr(spec, None, indptr_dtype="int64", row_range=(r0, r1))

        def local_spmv(xv, out):
            y = O.spmv_base(ld, li, lp, (r1 - r0, spec.n_cols), xv.numpy())
            out.copy_(torch.from_numpy(y))

        try:
            op = ShardedCsrSpmv(torch.from_numpy(ld), torch.from_numpy(li), torch.from_numpy(lp), r0,
                                (spec.n_rows, spec.n_cols), mode="nccl", local_spmv=local_spmv)
        except ValueError as exc:
            np.save(os.path.join(result_dir, f"err{rank}.npy"), np.array([1]))
            assert scenario == "wrong_cover", exc
            return
        assert scenario == "ok"
        assert op.row_ranges == [(bounds[i], bounds[i + 1] - bounds[i]) for i in range(world)]
        for rep in range(2):
            y = op.matvec(torch.from_numpy(x) * (rep + 1))
        full = O.spmv_base(data, idx, ptr, (spec.n_rows, spec.n_cols), x * 2)
        ok = np.array_equal(y.numpy(), full)

        # the same shards as a sharded SpMM: B replicated, C assembled on every rank
        B = S.dense_vector(spec, spec.n_cols, n_dense=5)

        def local_spmm(Bv, out):
            out.copy_(torch.from_numpy(O.spmm_base(ld, li, lp, (r1 - r0, spec.n_cols), Bv.numpy())))

        mm = ShardedCsrSpmm(torch.from_numpy(ld), torch.from_numpy(li), torch.from_numpy(lp), r0,
                            (spec.n_rows, spec.n_cols), mode="nccl", local_spmm=local_spmm)
        C = mm.matmul(torch.from_numpy(B))
        ok = ok and C.shape == (spec.n_rows, 5) and np.array_equal(
            C.numpy(), O.spmm_base(data, idx, ptr, (spec.n_rows, spec.n_cols), B))
        np.save(os.path.join(result_dir, f"ok{rank}.npy"), np.array([int(ok)]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_assembly_on_gloo(world, tmp_path):
    mp.spawn(_worker, args=(world, _free_port(), "ok", str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert np.load(tmp_path / f"ok{r}.npy")[0] == 1  # every rank holds the full, correct y


def test_inconsistent_shards_are_rejected_on_every_rank(tmp_path):
    mp.spawn(_worker, args=(2, _free_port(), "wrong_cover", str(tmp_path)), nprocs=2, join=True)
    assert all((tmp_path / f"err{r}.npy").exists() for r in range(2))


def test_slice_plan():
    # whole waves, later slices never larger, everything covered once
    assert slice_plan(296, 148, 4) == [(0, 148), (148, 296)]
    assert slice_plan(888, 148, 4) == [(0, 296), (296, 592), (592, 740), (740, 888)]
    assert slice_plan(444, 148, 4) == [(0, 148), (148, 296), (296, 444)]
    assert slice_plan(100, 148, 4) == [(0, 100)]
    assert slice_plan(150, 148, 4) == [(0, 148), (148, 150)]
    assert slice_plan(0, 148, 4) == []
    for n in (1, 147, 149, 1000, 1776):
        for k in (1, 2, 4):
            plan = slice_plan(n, 148, k)
            assert plan[0][0] == 0 and plan[-1][1] == n and len(plan) <= k
            assert all(a[1] == b[0] for a, b in zip(plan, plan[1:]))
            sizes = [e - b for b, e in plan]
            assert sizes == sorted(sizes, reverse=True)
