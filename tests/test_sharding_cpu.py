"""CPU: the multi-GPU host logic (row/batch partition, shard views, all-gather) on two gloo ranks.

The local product is a stand-in (the CPU oracle) -- the point here is the partitioning and the
collective, which are the same code the GPU ranks run."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from fastnn_b200 import sharding

NN, NT, TN = 0, 1, 2


def test_row_partition_covers_everything_once():
    for total in (0, 1, 7, 8, 8192, 8193):
        for world in (1, 2, 3, 8):
            spans = [sharding.row_partition(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0 and a0 <= a1
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.row_partition(4, 2, 2)


def test_shard_views_are_views():
    a = torch.arange(24, dtype=torch.float32).reshape(4, 6)
    s = sharding.shard_left_operand(TN, a, 2, 1)          # columns 3..5 of the stored [k, m]
    assert s.shape == (4, 3) and s.data_ptr() == a.data_ptr() + 3 * 4 and s.stride(0) == 6
    s = sharding.shard_left_operand(NN, a, 2, 0)
    assert s.shape == (2, 6) and s.data_ptr() == a.data_ptr()
    b3 = torch.zeros(5, 2, 3)
    assert sharding.shard_left_operand(NT, b3, 2, 0).shape[0] == 3


def _oracle_local(layout, a, b):
    fn = [oracle.matmul, oracle.matmul_nt, oracle.matmul_tn][layout]
    return torch.from_numpy(fn(a.contiguous().numpy(), b.contiguous().numpy()))


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(123)                   # same operands on every rank
        ok = True
        for layout, (m, n, k) in ((NN, (10, 6, 5)), (NT, (9, 4, 7)), (TN, (11, 5, 3)), (NN, (8, 3, 2))):
            sa = (k, m) if layout == TN else (m, k)
            sb = (n, k) if layout == NT else (k, n)
            a = torch.from_numpy(rng.standard_normal(sa, dtype=np.float32))
            b = torch.from_numpy(rng.standard_normal(sb, dtype=np.float32))
            shard = sharding.shard_left_operand(layout, a, world, rank)
            c_local = sharding.sharded_matmul(layout, shard, b, local_matmul=_oracle_local)
            full = sharding.all_gather_rows(c_local, m)
            want = _oracle_local(layout, a, b)
            ok = ok and torch.equal(full, want)
        # batched: partition the batch, nothing replicated
        q = torch.from_numpy(rng.standard_normal((5, 4, 3), dtype=np.float32))
        kk = torch.from_numpy(rng.standard_normal((5, 6, 3), dtype=np.float32))
        r0, r1 = sharding.row_partition(5, world, rank)
        s_local = sharding.sharded_matmul(NT, q[r0:r1], kk[r0:r1], local_matmul=_oracle_local)
        full = sharding.all_gather_rows(s_local, 5)
        ok = ok and torch.equal(full, _oracle_local(NT, q, kk))
        # K-sharded weight gradient (plain form: local product + all_reduce, then this rank's rows)
        x = torch.from_numpy(rng.standard_normal((12, 7), dtype=np.float32))     # [k, m]
        dy = torch.from_numpy(rng.standard_normal((12, 5), dtype=np.float32))    # [k, n]
        k0, k1 = sharding.row_partition(12, world, rank)
        mine = sharding.k_sharded_matmul_tn(x[k0:k1].contiguous(), dy[k0:k1].contiguous(), fused=False,
                                            local_matmul=_oracle_local)
        m0, m1 = sharding.row_partition(7, world, rank)
        ok = ok and tuple(mine.shape) == (m1 - m0, 5)
        ok = ok and torch.allclose(mine, _oracle_local(TN, x, dy)[m0:m1], atol=1e-5)
        flag = torch.tensor([1 if ok else 0])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            results.put(int(flag.item()))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.timeout(120)
def test_two_rank_sharded_matmul_and_gather_gloo():
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(100)
        assert p.exitcode == 0
    assert results.get(timeout=5) == 1


def test_gather_plan_places_every_shard_once():
    """The fused-gather arguments of all ranks tile the full C without gaps or overlap, and a TN
    shard (a column slice of the stored [k, m]) keeps the full row stride."""
    for world in (1, 2, 3, 8):
        for layout, (m, n, k) in ((NN, (8192, 512, 64)), (NT, (1001, 36, 20)), (TN, (250, 72, 64))):
            covered = np.zeros(m * n, dtype=np.int32)
            for rank in range(world):
                r0, r1 = sharding.row_partition(m, world, rank)
                a_shape = (k, r1 - r0) if layout == TN else (r1 - r0, k)
                b_shape = (n, k) if layout == NT else (k, n)
                plan = sharding.gather_plan(layout, a_shape, m if layout == TN else k, b_shape, m, world, rank)
                assert (plan["m"], plan["n"], plan["k"], plan["batch"]) == (r1 - r0, n, k, 1)
                assert plan["lda"] == (m if layout == TN else k) and plan["ldc"] == n
                covered[plan["offset"]: plan["offset"] + plan["m"] * n] += 1
            assert (covered == 1).all()
    # batched: batches are partitioned, strides are dense
    plan = sharding.gather_plan(NT, (3, 128, 32), 32, (3, 128, 32), 6, 2, 1)
    assert plan == dict(m=128, n=128, k=32, batch=3, lda=32, ldb=32, ldc=128, sa=4096, sb=4096,
                        sc=128 * 128, offset=3 * 128 * 128)
    with pytest.raises(ValueError):
        sharding.gather_plan(NN, (5, 4), 4, (4, 3), 8, 2, 0)          # 5 rows is not this rank's share
    with pytest.raises(ValueError):
        sharding.gather_plan(NN, (4, 4), 4, (5, 3), 8, 2, 0)          # inner dimensions differ


def _gather_worker(rank, world, port, results):
    """Two gloo ranks play the fused gather with host memory standing in for peer-mapped C: each
    rank computes its shard with the oracle and 'stores' it at gather_plan's offset into every
    rank's buffer (an all_gather of (offset, values) pairs); all buffers must equal the product."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(321)
        ok = True
        for layout, (m, n, k) in ((NN, (11, 6, 5)), (NT, (9, 4, 7)), (TN, (10, 5, 3))):
            sa = (k, m) if layout == TN else (m, k)
            sb = (n, k) if layout == NT else (k, n)
            a = torch.from_numpy(rng.standard_normal(sa, dtype=np.float32))
            b = torch.from_numpy(rng.standard_normal(sb, dtype=np.float32))
            shard = sharding.shard_left_operand(layout, a, world, rank)
            plan = sharding.gather_plan(layout, tuple(shard.shape), shard.stride(0), tuple(b.shape), m,
                                        world, rank)
            mine = _oracle_local(layout, shard, b).reshape(-1)
            pieces = [None] * world
            dist.all_gather_object(pieces, (plan["offset"], mine.numpy()))
            full = np.full(m * n, np.nan, dtype=np.float32)
            for off, vals in pieces:
                full[off: off + vals.size] = vals
            want = [oracle.matmul, oracle.matmul_nt, oracle.matmul_tn][layout](a.numpy(), b.numpy())
            ok = ok and np.array_equal(full.reshape(m, n), want)
        results.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_fused_gather_layout():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    procs = [ctx.Process(target=_gather_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(results.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert got == [(0, True), (1, True)]
