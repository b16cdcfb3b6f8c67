"""Batch data-parallelism: each rank runs whole images through a replica of the model."""
from __future__ import annotations

import torch


def shard_batch(batch: int, rank: int, world: int) -> slice:
    """The images rank `rank` owns out of `batch` (contiguous, remainder to the low ranks)."""
    base, extra = divmod(batch, world)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))


def gather_outputs(local: torch.Tensor, group=None) -> torch.Tensor:
    """All ranks' outputs concatenated along the batch dim (equal shards).  Only for
    collecting results; the forward path itself needs no communication."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    out = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(out, local.contiguous(), group=group)
    return torch.cat(out, dim=0)
