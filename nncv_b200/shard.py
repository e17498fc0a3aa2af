"""Batch sharding of the forward across the GPUs of one box (one process per GPU).

Images are independent, weights are replicated, and the only exchange is the gather of the
logits to rank 0.  nncv itself has no multi-device code (its platform probe warns when the GPU
count is not 1, include/nncv/compiler/Utils/PlatformCtx.hpp:140-144); this is the data-parallel
extension of its forward.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous slice [lo, hi) of a batch of n images owned by `rank`; the first n % world
    ranks get one extra image, and a rank may own nothing when n < world."""
    if world <= 0 or not (0 <= rank < world) or n < 0:
        raise ValueError("bad shard arguments")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def gather_logits(local: torch.Tensor, n: int, group=None) -> Optional[torch.Tensor]:
    """Gather the per-rank logits [n_r, 1000] to rank 0 as [n, 1000] (None on the other ranks).

    Ragged shards are padded to the largest shard so that one fixed-size gather serves every rank.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if world == 1:
        return local
    sizes = [shard_range(n, r, world) for r in range(world)]
    cap = max(hi - lo for lo, hi in sizes)
    buf = local
    if local.shape[0] != cap:
        buf = local.new_zeros((cap,) + tuple(local.shape[1:]))
        buf[: local.shape[0]] = local
    outs: Optional[List[torch.Tensor]] = None
    if rank == 0:
        outs = [torch.empty_like(buf) for _ in range(world)]
    dist.gather(buf, outs, dst=0, group=group)
    if rank != 0:
        return None
    return torch.cat([o[: hi - lo] for o, (lo, hi) in zip(outs, sizes)], dim=0)
