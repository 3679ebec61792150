"""GPU (needs two devices): rows of C / batches partitioned over two ranks with the real kernels,
NCCL all-gather of the shards, result checked against the CPU oracle.  Skipped on one GPU."""
import os
import socket

import numpy as np
import pytest

import oracle
from helpers import check_tf32_parity

pytestmark = pytest.mark.gpu

NN, NT, TN = 0, 1, 2


def _worker(rank, world, port, queue):
    import torch
    import torch.distributed as dist
    import fastnn_b200 as f
    from fastnn_b200 import sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    f.cuda_init(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        _work(rank, world, queue, torch, dist, f, sharding)
    except BaseException as exc:                 # the parent must not wait for results that never come
        import traceback
        queue.put(("error", rank, "".join(traceback.format_exception(exc))))
        raise
    finally:
        dist.destroy_process_group()


def _work(rank, world, queue, torch, dist, f, sharding):
    if True:
        rng = np.random.default_rng(7)                      # same operands on every rank
        out = {}
        for layout, (m, n, k) in ((NN, (520, 264, 132)), (NT, (512, 256, 128)), (TN, (768, 136, 260)),
                                  (TN, (250, 72, 64))):
            sa = (k, m) if layout == TN else (m, k)
            sb = (n, k) if layout == NT else (k, n)
            a = rng.standard_normal(sa, dtype=np.float32)
            b = rng.standard_normal(sb, dtype=np.float32)
            da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
            shard = sharding.shard_left_operand(layout, da, world, rank)   # a view; TN: column slice
            c_local = sharding.sharded_matmul(layout, shard, db)
            full = sharding.all_gather_rows(c_local, m)
            out[(layout, m, n, k)] = (full.cpu().numpy(), a, b)
        q = rng.standard_normal((6, 128, 32), dtype=np.float32)
        kk = rng.standard_normal((6, 128, 32), dtype=np.float32)
        r0, r1 = sharding.row_partition(6, world, rank)
        s_local = sharding.sharded_matmul(NT, torch.from_numpy(q[r0:r1]).cuda(), torch.from_numpy(kk[r0:r1]).cuda())
        s_full = sharding.all_gather_rows(s_local, 6).cpu().numpy()
        # K-sharded weight gradient, fused form: partial tiles go straight into the owner's
        # symmetric-memory slots from the GEMM epilogue; twice per shape (slots are reused)
        grads = {}
        for (m, n, k) in ((512, 256, 1024), (251, 72, 96)):
            x = rng.standard_normal((k, m), dtype=np.float32)
            dy = rng.standard_normal((k, n), dtype=np.float32)
            k0, k1 = sharding.row_partition(k, world, rank)
            xl, dyl = torch.from_numpy(x[k0:k1].copy()).cuda(), torch.from_numpy(dy[k0:k1].copy()).cuda()
            ws = sharding.KShardedGradWorkspace(m, n)
            mine = None
            for _ in range(2):
                mine = sharding.k_sharded_matmul_tn(xl, dyl, workspace=ws, fused=True)
            plain = sharding.k_sharded_matmul_tn(xl, dyl, fused=False)
            full = sharding.all_gather_rows(mine, m).cpu().numpy()
            full_plain = sharding.all_gather_rows(plain, m).cpu().numpy()
            grads[(m, n, k)] = (full, full_plain, x, dy)
        # all of C on every rank with the all-gather fused into the GEMM epilogue (peer stores
        # into symmetric memory), twice per shape (the buffer is reused), incl. a batched product
        gathered = {}
        for layout, (m, n, k) in ((NN, (520, 264, 132)), (NT, (512, 256, 128)), (TN, (768, 136, 260)),
                                  (TN, (251, 72, 64))):
            sa = (k, m) if layout == TN else (m, k)
            sb = (n, k) if layout == NT else (k, n)
            a = rng.standard_normal(sa, dtype=np.float32)
            b = rng.standard_normal(sb, dtype=np.float32)
            da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
            shard = sharding.shard_left_operand(layout, da, world, rank)
            full = sharding.GatheredOutput((m, n))
            # unicast stores twice (the buffer is reused), then -- where the fabric offers a multicast
            # address and the shape allows 16-byte stores -- once through the switch
            modes = [False, False] + ([True] if full.mc_ptr != 0 and n % 4 == 0 and shard.stride(0) % 4 == 0 else [])
            for mc in modes:
                full.tensor.fill_(float("nan"))
                full.barrier()
                sharding.sharded_matmul_gathered(layout, shard, db, full, multicast=mc)
                full.barrier()
                torch.cuda.synchronize()
                assert not torch.isnan(full.tensor).any(), f"multicast={mc}: rows missing on rank {rank}"
            gathered[(layout, m, n, k)] = (full.tensor.cpu().numpy(), a, b)
        gb = sharding.GatheredOutput((6, 128, 128))
        gb.tensor.fill_(float("nan"))
        gb.barrier()
        sharding.sharded_matmul_gathered(NT, torch.from_numpy(q[r0:r1]).cuda(), torch.from_numpy(kk[r0:r1]).cuda(), gb)
        gb.barrier()
        gathered_batched = gb.tensor.cpu().numpy()
        status = f.device_status()
        queue.put((rank, gathered, gathered_batched))
        if rank == 0:
            queue.put((out, s_full, q, kk, status, grads))
        dist.barrier()


def test_two_gpu_sharded_matmul_nccl(built_library):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = [ctx.Process(target=_worker, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    items = []
    while len(items) < 3:
        item = queue.get(timeout=300)
        if item[0] == "error":
            for p in procs:
                p.join(30)
                if p.is_alive():
                    p.kill()
            pytest.fail(f"rank {item[1]} failed:\n{item[2]}")
        items.append(item)
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    out, s_full, q, kk, status, grads = [it for it in items if len(it) == 6][0]
    assert status == 0
    per_rank = sorted((it for it in items if len(it) == 3), key=lambda it: it[0])
    assert [it[0] for it in per_rank] == [0, 1]
    for rank, gathered, gathered_batched in per_rank:          # EVERY rank holds all of C
        for (layout, m, n, k), (got, a, b) in gathered.items():
            want = [oracle.matmul, oracle.matmul_nt, oracle.matmul_tn][layout](a, b)
            check_tf32_parity(got, want, k, a, b, what=f"fused gather rank {rank} L{layout} {m}x{n}x{k}")
        check_tf32_parity(gathered_batched, oracle.matmul_nt(q, kk), 32, q, kk,
                          what=f"fused gather batched rank {rank}")
    assert np.array_equal(per_rank[0][2], per_rank[1][2])
    for (layout, m, n, k), (got, a, b) in out.items():
        want = [oracle.matmul, oracle.matmul_nt, oracle.matmul_tn][layout](a, b)
        check_tf32_parity(got, want, k, a, b, what=f"2-GPU L{layout} {m}x{n}x{k}")
    check_tf32_parity(s_full, oracle.matmul_nt(q, kk), 32, q, kk, what="2-GPU batched")
    for (m, n, k), (fused, plain, x, dy) in grads.items():
        want = oracle.matmul_tn(x, dy)
        check_tf32_parity(fused, want, k, x, dy, what=f"K-sharded dW fused {m}x{n}x{k}")
        check_tf32_parity(plain, want, k, x, dy, what=f"K-sharded dW all_reduce {m}x{n}x{k}")
