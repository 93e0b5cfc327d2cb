"""Batch x head partitioning of the CASTLE hot path over the GPUs of one box.

Every (batch, head) pair is independent in the forward, the backward and the
decode step (the reference's launch grid is (query blocks, batch*heads):
lookahead_keys_attention/lookahead_keys_attention_triton.py:463-466), so ranks
own disjoint rectangles of the (batch, head) grid and no collective is needed
inside the path; only the final outputs are gathered.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Shard:
    b0: int
    b1: int
    h0: int
    h1: int

    @property
    def pairs(self) -> int:
        return (self.b1 - self.b0) * (self.h1 - self.h0)


def partition(batch: int, heads: int, world: int, rank: int) -> Shard:
    """Rectangle of (batch, head) pairs owned by `rank`.

    When world <= batch the batch is split (weights replicated, nothing to reduce);
    otherwise each batch element is shared by world // batch ranks that split its heads.
    `world` must divide batch, or batch must divide world with world // batch dividing heads.
    """
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    if batch % world == 0:
        per = batch // world
        return Shard(rank * per, (rank + 1) * per, 0, heads)
    if world % batch == 0 and heads % (world // batch) == 0:
        groups = world // batch
        hp = heads // groups
        b, g = divmod(rank, groups)
        return Shard(b, b + 1, g * hp, (g + 1) * hp)
    raise ValueError(f"cannot split batch {batch} x heads {heads} evenly over {world} ranks")


def gather_heads(local, shard: Shard, batch: int, heads: int, group=None, dst: int = 0):
    """Gather per-rank (b, h, n, d) outputs into the full (batch, heads, n, d) tensor on `dst`.
    Uses torch.distributed (NCCL on GPUs, gloo on CPU); returns None on other ranks."""
    import torch
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    bufs = [torch.empty_like(local) for _ in range(world)] if rank == dst else None
    dist.gather(local.contiguous(), bufs, dst=dst, group=group)
    if rank != dst:
        return None
    full = local.new_empty(batch, heads, *local.shape[2:])
    for r, buf in enumerate(bufs):
        s = partition(batch, heads, world, r)
        full[s.b0:s.b1, s.h0:s.h1] = buf
    return full
