"""Batch x head partitioning of the CASTLE hot path over the GPUs of one box.

Every (batch, head) pair is independent in the forward, the backward and the
decode step (the reference's launch grid is (query blocks, batch*heads):
lookahead_keys_attention/lookahead_keys_attention_triton.py:463-466), so ranks
own disjoint rectangles of the (batch, head) grid and no collective is needed
inside the path; only the final outputs are gathered.

When there are more ranks than batch rows, the ranks that share a batch row split its HEADS for
the attention core.  The two projections around the core are then split by ROWS (positions)
instead, with the full weights on every rank, and the tensors change hands twice per pass with
an all-to-all inside the row's group (`rows_to_heads`, `heads_to_rows`): each rank uploads,
projects and downloads only its own positions, and nothing is ever summed across ranks.
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


def _all_to_all(t, group):
    """all_to_all_single over dim 0 (one equal slice per rank of `group`), differentiable: the
    gradient of an exchange is the reverse exchange."""
    import torch
    import torch.distributed as dist

    class _Exchange(torch.autograd.Function):
        @staticmethod
        def forward(ctx, inp):
            inp = inp.contiguous()                      # the collective cuts dim 0 in memory order
            out = torch.empty_like(inp)
            dist.all_to_all_single(out, inp, group=group)
            return out

        @staticmethod
        def backward(ctx, g):
            g = g.contiguous()                          # autograd may hand over a permuted gradient
            back = torch.empty_like(g)
            dist.all_to_all_single(back, g, group=group)
            return back

    return _Exchange.apply(t)


def rows_to_heads(packed_rows, group=None):
    """(B, n_local, 6, H, d) - this rank's positions, every head - becomes (B, n_local * G, 6, H / G, d):
    every position of the row's group, this rank's heads (rank r owns positions [r*n_local, (r+1)*n_local)
    and heads [r*H/G, (r+1)*H/G)).  One all-to-all inside `group` (G ranks)."""
    import torch.distributed as dist
    G = dist.get_world_size(group)
    B, n, six, H, d = packed_rows.shape
    assert H % G == 0
    # destination rank first: (G, B, n, 6, H/G, d)
    send = packed_rows.view(B, n, six, G, H // G, d).permute(3, 0, 1, 2, 4, 5).contiguous()
    recv = _all_to_all(send, group)                      # source rank first = position chunks in order
    return recv.permute(1, 0, 2, 3, 4, 5).reshape(B, G * n, six, H // G, d)


def heads_to_rows(out_heads, group=None):
    """The way back for the core's output: (B, H / G, N, d) - this rank's heads, every position - becomes
    (B, N / G, H * d): this rank's positions with the heads of all ranks merged, ready for `combine_heads`."""
    import torch.distributed as dist
    G = dist.get_world_size(group)
    B, h, N, d = out_heads.shape
    assert N % G == 0
    n = N // G
    # destination rank (position chunk) first: (G, B, n, h, d)
    send = out_heads.permute(0, 2, 1, 3).reshape(B, G, n, h, d).permute(1, 0, 2, 3, 4).contiguous()
    recv = _all_to_all(send, group)                      # source rank first = head chunks in order
    return recv.permute(1, 2, 0, 3, 4).reshape(B, n, G * h * d)
