"""Column-block sharding of one large GEMM over the GPUs of a box (one process per GPU).

    D[:, J_r] = A * B[:, J_r]        rank r owns the column block J_r of B and of D

The blocks are independent; the only exchange is A, sent once from the root into every rank's own
memory with a `torch.distributed` broadcast (NCCL over NVLink on GPUs).  Kernels then read local
memory only: no peer loads, no multicast, no collective inside a step.  The reference has no
multi-GPU path; this is the partitioning named for the 16384^3 BFloat16 configuration.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ColumnShard:
    rank: int
    world: int
    n_total: int
    start: int       # first column of this rank's block
    count: int       # columns in the block

    @property
    def stop(self) -> int:
        return self.start + self.count


def column_shard(n_total: int, world: int, rank: int, multiple: int = 1) -> ColumnShard:
    """Contiguous column block of `rank`: blocks differ by at most `multiple` columns, every block
    but possibly the last is a multiple of `multiple` (use the tile width so no rank gets a ragged
    tile it could have avoided), blocks cover [0, n_total) exactly, empty blocks are allowed."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if n_total < 0 or multiple < 1:
        raise ValueError("n_total must be >= 0 and multiple >= 1")
    units = -(-n_total // multiple)                 # ceil
    base, extra = divmod(units, world)
    u0 = rank * base + min(rank, extra)
    u1 = u0 + base + (1 if rank < extra else 0)
    start, stop = min(u0 * multiple, n_total), min(u1 * multiple, n_total)
    return ColumnShard(rank, world, n_total, start, stop - start)


def broadcast_a(a_storage, src: int = 0, group=None):
    """Sends A from `src` to every rank, in place.  `a_storage` must be the contiguous storage of A
    (for a column-major device array `a` that is `a.T`).  Returns the tensor."""
    import torch.distributed as dist
    if not a_storage.is_contiguous():
        raise ValueError("broadcast_a needs the contiguous storage view of A (a.T for a column-major array)")
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.broadcast(a_storage, src=src, group=group)
    return a_storage


def colshard_matmul(local_product, a_storage, b_block, d_block, *, src: int = 0, group=None, a_is_resident=False):
    """One sharded product on this rank: broadcast A (unless it is already resident from an earlier
    call) and run `local_product(a_storage, b_block, d_block)` on the rank's own column block.
    `local_product` is the single-GPU GEMM (e.g. a closure over `GemmKernels.matmul`)."""
    if not a_is_resident:
        broadcast_a(a_storage, src, group)
    local_product(a_storage, b_block, d_block)
    return d_block


def colshard_matmul_host(conf, a_host, a_dev, b_host_block, d_host_block, *, src: int = 0, group=None, device_index=None):
    """The sharded product with operands and result in host memory.  Rank `src` uploads A (its
    `a_host`; other ranks pass None) into its `a_dev`, A goes to every rank over NVLink (NCCL
    broadcast into each rank's `a_dev`), and every rank runs the host-path GEMM on its own column
    block of B and D with A used in place — so A crosses PCIe once per job instead of once per rank."""
    import torch
    from .matmul import matmul_host
    import torch.distributed as dist
    if a_host is not None:
        a_dev.copy_(a_host, non_blocking=True)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        broadcast_a(a_dev.T, src, group)            # a_dev.T is the contiguous storage of the column-major array
    matmul_host(conf, a_dev, b_host_block, None, d_host_block, device_index=device_index, a_on_device=True)
    return d_host_block


def gather_columns(d_block, shard: ColumnShard, group=None):
    """Assembles the full D on every rank from the column blocks (outside any timed region; used by
    tests and by callers that want D in one place).  `d_block` is the contiguous storage of the
    rank's block, shape (count, M) for column-major data.  Returns a (n_total, M) tensor."""
    import torch
    import torch.distributed as dist
    world = shard.world
    if world == 1 or not (dist.is_available() and dist.is_initialized()):
        return d_block
    m = d_block.shape[1]
    # blocks may differ in size: exchange through padded buffers of the largest block
    sizes = [None] * world
    dist.all_gather_object(sizes, int(d_block.shape[0]), group=group)
    biggest = max(sizes)
    padded = torch.zeros(biggest, m, dtype=d_block.dtype, device=d_block.device)
    padded[: d_block.shape[0]] = d_block
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:s] for p, s in zip(parts, sizes)], dim=0)
