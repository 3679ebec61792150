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
                   a.stride(0), b.stride(0), n, 0, 0, 0, stream=cb.current_stream_ptr())
        return c
    return [cb.matmul, cb.matmul_nt, cb.matmul_tn][layout](a, b)


# ------------------------------------------------------------------------------------------
# All of C on every rank, with the all-gather fused into the GEMM: rank r computes its rows (or
# batches) of C and its GEMM's epilogue stores every finished tile into the same rows of EVERY
# rank's full-size C (TMA stores to peer-mapped symmetric memory over NVLink), while the tensor
# core works on the next tile.  No collective follows; the ranks meet at one barrier before any
# of them reads rows it did not compute.  Nothing is ever loaded from a peer.
# ------------------------------------------------------------------------------------------

def gather_plan(layout: int, a_shape, a_row_stride: int, b_shape, total: int, world: int, rank: int):
    """Arguments of the fused-gather GEMM of rank ``rank``, as plain integers (no device needed):
    the GEMM's m, n, k, batch, leading dimensions and batch strides in elements, and ``offset``,
    the element offset of this rank's part inside the full C (``total`` rows, or batches).
    ``a_shape`` is the shape of this rank's shard of the left operand, ``a_row_stride`` its row
    stride in elements (a TN shard is a column slice: the stride is the full row)."""
    r0, r1 = row_partition(total, world, rank)
    if len(a_shape) == 3:
        batch = int(a_shape[0])
        if batch != r1 - r0:
            raise ValueError("a_shard does not hold this rank's batches")
        m = int(a_shape[2] if layout == TN else a_shape[1])
        k = int(a_shape[1] if layout == TN else a_shape[2])
        n = int(b_shape[1] if layout == NT else b_shape[2])
        if int(b_shape[0]) != batch or int(b_shape[2] if layout == NT else b_shape[1]) != k:
            raise ValueError("operand shapes do not match")
        return dict(m=m, n=n, k=k, batch=batch, lda=int(a_shape[2]), ldb=int(b_shape[2]), ldc=n,
                    sa=int(a_shape[1] * a_shape[2]), sb=int(b_shape[1] * b_shape[2]), sc=m * n,
                    offset=r0 * m * n)
    m = int(a_shape[1] if layout == TN else a_shape[0])
    k = int(a_shape[0] if layout == TN else a_shape[1])
    if m != r1 - r0:
        raise ValueError("a_shard does not hold this rank's rows")
    n = int(b_shape[0] if layout == NT else b_shape[1])
    if int(b_shape[1] if layout == NT else b_shape[0]) != k:
        raise ValueError("operand shapes do not match")
    return dict(m=m, n=n, k=k, batch=1, lda=int(a_row_stride), ldb=int(b_shape[1]), ldc=n,
                sa=0, sb=0, sc=0, offset=r0 * n)


class GatheredOutput:
    """The full C of a sharded product in symmetric memory: the same ``shape`` on every rank, each
    rank's buffer mapped into every other rank's address space."""

    def __init__(self, shape, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world - 1 > 7:
            raise ValueError("the fused gather stores to at most seven peers")
        self.tensor = symm_mem.empty(tuple(shape), dtype=torch.float32,
                                     device=torch.device("cuda", torch.cuda.current_device()))
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        self.base_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        # NVLink multicast address of the buffer (0 when the fabric or the driver offers none)
        self.mc_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)

    def barrier(self, channel: int = 0) -> None:
        """Every rank's GEMMs enqueued before this point are complete on every rank afterwards
        (runs on torch's current stream; no host synchronisation)."""
        self.handle.barrier(channel=channel)


def sharded_matmul_gathered(layout: int, a_shard: torch.Tensor, b: torch.Tensor, out: GatheredOutput,
                            bias: Optional[torch.Tensor] = None, act: int = cb.ACT_NONE,
                            stream: Optional[int] = None, multicast: Optional[bool] = None) -> torch.Tensor:
    """This rank's rows (or batches) of C = act(op(A).op(B) + bias), written by the GEMM itself
    into ``out`` on EVERY rank.  Returns this rank's full-size buffer; rows computed by other ranks
    are valid after ``out.barrier()``.

    ``multicast``: False (the default) stores every tile to each peer in turn (TMA stores); True
    sends it once through the NVSwitch (multimem.st to the buffer's multicast address), which cuts
    what a rank sends to 1/(N-1) but makes every rank take in its own rows as well.  Measured on
    four GPUs the two take the same time (0.61-0.66 ms per 8192-row GEMM: the receiving side, not
    the sending side, is the limit), so the form that needs no multicast object is the default.

    (A second form -- the shard in row panels, each finished panel copied to the peers with
    cudaMemcpyAsync on side streams while the next panel is computed -- was built and measured:
    the copies of peer-mapped memory did not overlap the persistent GEMM and moved no more bytes per
    second than the epilogue's own stores, 0.61 ms against 0.61-0.62 ms per 8192-row GEMM on four
    GPUs and 1.05 against 0.79 ms on two, so it was taken out again.)"""
    cb._ensure_ctx(b)
    total = int(out.tensor.shape[0])
    if a_shard.dim() == 3:
        a_shard = a_shard.contiguous()
    elif a_shard.stride(1) != 1:
        raise ValueError("a_shard must have contiguous rows")
    plan = gather_plan(layout, tuple(a_shard.shape), a_shard.stride(-2), tuple(b.shape), total,
                       out.world, out.rank)
    if plan["m"] == 0 or plan["batch"] == 0:
        return out.tensor
    off = 4 * plan["offset"]
    cur = cb.current_stream_ptr() if stream is None else stream
    mc_ok = out.mc_ptr != 0 and plan["n"] % 4 == 0 and a_shard.data_ptr() % 16 == 0 and plan["lda"] % 4 == 0
    if multicast:
        if not mc_ok:
            raise ValueError("no multicast address for this buffer, or a shape multimem.st cannot serve")
        cb.gemm_gather_mc_ex(layout, a_shard.data_ptr(), b.data_ptr(), out.base_ptrs[out.rank] + off,
                             plan["m"], plan["n"], plan["k"], plan["batch"], plan["lda"], plan["ldb"],
                             plan["ldc"], plan["sa"], plan["sb"], plan["sc"], out.mc_ptr + off,
                             bias_ptr=bias.data_ptr() if bias is not None else 0, act=act, stream=cur)
        return out.tensor
    # destinations start at the next rank, so that the ranks do not all write one GPU at a time
    peers = [out.base_ptrs[(out.rank + 1 + i) % out.world] + off for i in range(out.world - 1)]
    cb.gemm_gather_ex(layout, a_shard.data_ptr(), b.data_ptr(), out.base_ptrs[out.rank] + off,
                      plan["m"], plan["n"], plan["k"], plan["batch"], plan["lda"], plan["ldb"], plan["ldc"],
                      plan["sa"], plan["sb"], plan["sc"], peers,
                      bias_ptr=bias.data_ptr() if bias is not None else 0, act=act, stream=cur)
    return out.tensor


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


# ------------------------------------------------------------------------------------------
# K-sharded weight gradient:  dW[m,n] = X^T . dY  with the CONTRACTION dimension split over ranks
# (each rank holds its own rows of X[k,m] and dY[k,n] -- the data-parallel case of FastNN's
# MatmulBackward, src/autograd/backward_ops.rs:93).  Every rank's product is a partial sum of the
# whole dW, so an exchange is unavoidable; the result is reduce-scattered: rank r ends with rows
# row_partition(m, world, r) of dW.
#
# Fused form (CUDA): this is split-K across GPUs.  Rank r runs one GEMM per destination rank o
# over the column slice of X that produces o's rows, and the GEMM's own epilogue (TMA stores)
# writes the partial tile straight into slot r of o's symmetric-memory workspace over NVLink --
# the transfer of tile i overlaps the math of tile i+1, no staging copy, no separate collective.
# After one symmetric-memory barrier each rank adds its `world` slots in ascending rank order
# (deterministic) with the split-K reduce kernel.
# Plain form: local GEMM + all_reduce, then slice (what "call NCCL after the GEMM" costs; also the
# path CPU ranks can run).
# ------------------------------------------------------------------------------------------

class KShardedGradWorkspace:
    """Symmetric-memory slots for one (m, n): on every rank [world][rows_max][n] floats."""

    def __init__(self, m: int, n: int, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.m, self.n = m, n
        self.rows_max = -(-m // self.world)
        self.slots = symm_mem.empty((self.world, self.rows_max, n), dtype=torch.float32,
                                    device=torch.device("cuda", torch.cuda.current_device()))
        self.handle = symm_mem.rendezvous(self.slots, self.group)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]

    def slot_ptr(self, owner: int, writer: int) -> int:
        return self.peer_ptrs[owner] + 4 * writer * self.rows_max * self.n


def k_sharded_matmul_tn(x_local: torch.Tensor, dy_local: torch.Tensor, group=None,
                        workspace: Optional[KShardedGradWorkspace] = None, fused: bool = True,
                        local_matmul: Optional[Callable] = None) -> torch.Tensor:
    """This rank's rows of dW = sum over ranks of X_r^T . dY_r.  x_local [k_r, m], dy_local [k_r, n]."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    k_r, m = x_local.shape
    n = dy_local.shape[1]
    if dy_local.shape[0] != k_r:
        raise ValueError("x_local and dy_local must have the same number of rows")
    r0, r1 = row_partition(m, world, rank)
    if not fused or not x_local.is_cuda:
        fn = local_matmul or _cuda_local
        partial = fn(TN, x_local, dy_local)                  # full [m, n] partial sum
        dist.all_reduce(partial, group=group)
        return partial[r0:r1].contiguous()
    ws = workspace or KShardedGradWorkspace(m, n, group)
    if (ws.m, ws.n, ws.world) != (m, n, world):
        raise ValueError("workspace was built for another problem")
    cb._check(x_local, "x_local"); cb._check(dy_local, "dy_local")
    cb._ensure_ctx(x_local)
    # everything on torch's current stream: the symmetric-memory barriers run there too
    stream = cb.current_stream_ptr()
    ws.handle.barrier(channel=0)                             # previous use of the slots is over
    for step in range(world):                                # start at the neighbour: spread traffic
        owner = (rank + 1 + step) % world
        o0, o1 = row_partition(m, world, owner)
        if o1 == o0:
            continue
        cb.gemm_ex(TN, x_local.data_ptr() + 4 * o0, dy_local.data_ptr(), ws.slot_ptr(owner, rank),
                   o1 - o0, n, k_r, 1, m, n, n, 0, 0, 0, stream=stream)
    ws.handle.barrier(channel=1)                             # every partial has landed
    out = torch.empty((r1 - r0, n), dtype=torch.float32, device=x_local.device)
    if r1 > r0:
        # slots are [world][rows_max][n]; a partial occupies the first r1-r0 rows of its slot, so
        # the reduce walks slots with a stride of rows_max*n by treating them as rows_max-row blocks
        if r1 - r0 == ws.rows_max:
            cb.reduce_partials(ws.slots.data_ptr(), out.data_ptr(), r1 - r0, n, world, stream=stream)
        else:
            packed = ws.slots[:, : r1 - r0].contiguous()
            cb.reduce_partials(packed.data_ptr(), out.data_ptr(), r1 - r0, n, world, stream=stream)
    return out
