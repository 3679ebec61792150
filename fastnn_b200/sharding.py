"""Multi-GPU form of the matmul path: partition the OUTPUT rows (or the batch) over ranks.

One process per GPU.  The compute needs no exchange: rank r owns rows [r0, r1) of C (or batches
[r0, r1) of a batched product), reads the matching rows of the left operand and the whole right
operand, and calls the single-GPU entry point on its shard.  Only a caller that wants all of C on
every device pays for a collective (``all_gather_rows``, NCCL all-gather over NVLink).

For ``matmul_tn`` the left operand is stored [k, m]; the row shard of C corresponds to a COLUMN
slice of that storage, which is passed to the kernel by pointer offset and leading dimension
(no copy).

``local_matmul`` arguments exist so that the host-side logic can be exercised on CPU ranks
(gloo) with a stand-in; the default is the CUDA path of this package.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from . import cuda_backend as cb

NN, NT, TN = cb.NN, cb.NT, cb.TN


def row_partition(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced split of ``total`` rows (or batches): the first ``total % world``
    ranks get one extra.  Returns [r0, r1)."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad world/rank")
    base, extra = divmod(total, world)
    r0 = rank * base + min(rank, extra)
    return r0, r0 + base + (1 if rank < extra else 0)


def shard_left_operand(layout: int, a_full: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """The part of the left operand rank ``rank`` needs for its rows of C (a view, no copy):
    rows of A for NN/NT, columns of the stored [k, m] matrix for TN, batches for 3-D operands."""
    if a_full.dim() == 3:
        r0, r1 = row_partition(a_full.shape[0], world, rank)
        return a_full[r0:r1]
    if layout == TN:
        r0, r1 = row_partition(a_full.shape[1], world, rank)
        return a_full[:, r0:r1]
    r0, r1 = row_partition(a_full.shape[0], world, rank)
    return a_full[r0:r1]


def _cuda_local(layout: int, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Single-GPU product of a (possibly strided) left shard with the replicated right operand."""
    if a.dim() == 3:
        return [cb.matmul, cb.matmul_nt, cb.matmul_tn][layout](a.contiguous(), b)
    if layout == TN and not a.is_contiguous():
        # column slice of the stored [k, m_total] matrix: same row stride, shifted base
        k, m = a.shape
        n = b.shape[1]
        c = torch.empty((m, n), dtype=torch.float32, device=a.device)
        cb._ensure_ctx(b)
        cb.gemm_ex(TN, a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, 1,
                   a.stride(0), b.stride(0), n, 0, 0, 0)
        return c
    return [cb.matmul, cb.matmul_nt, cb.matmul_tn][layout](a, b)


def sharded_matmul(layout: int, a_shard: torch.Tensor, b: torch.Tensor,
                   local_matmul: Optional[Callable] = None) -> torch.Tensor:
    """This rank's rows (or batches) of C.  ``b`` is replicated for 2-D products; for batched
    products ``b`` is this rank's batches as well."""
    fn = local_matmul or _cuda_local
    return fn(layout, a_shard, b)


def all_gather_rows(c_local: torch.Tensor, total_rows: int, group=None) -> torch.Tensor:
    """All of C on every rank.  Equal shards use one all_gather_into_tensor; ragged shards
    (total_rows not divisible by the world size) gather padded shards and trim."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    r0, r1 = row_partition(total_rows, world, rank)
    if c_local.shape[0] != r1 - r0:
        raise ValueError("c_local does not hold this rank's rows")
    rest = tuple(c_local.shape[1:])
    if total_rows % world == 0:
        out = torch.empty((total_rows,) + rest, dtype=c_local.dtype, device=c_local.device)
        dist.all_gather_into_tensor(out, c_local.contiguous(), group=group)
        return out
    most = -(-total_rows // world)
    padded = torch.zeros((most,) + rest, dtype=c_local.dtype, device=c_local.device)
    padded[: r1 - r0] = c_local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    pieces = []
    for r in range(world):
        q0, q1 = row_partition(total_rows, world, r)
        pieces.append(parts[r][: q1 - q0])
    return torch.cat(pieces, dim=0)
