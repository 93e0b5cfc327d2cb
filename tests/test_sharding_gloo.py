"""CPU, world_size 2, gloo: the (batch, head) shards of the parallel pass, computed
independently per rank (by the oracle standing in for the kernels), gather to exactly
the unsharded result - the N>1 path has no other communication."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, batch, heads, q):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lookahead_keys_attention_b200.sharding import gather_heads, partition
    from oracle import castle_oracle as O
    torch.manual_seed(0)
    t = [torch.randn(batch, heads, 24, 16) for _ in range(6)]
    s = partition(batch, heads, world, rank)
    local = O.castle_parallel(*[x[s.b0:s.b1, s.h0:s.h1] for x in t], 0.25)
    full = gather_heads(local, s, batch, heads)
    if rank == 0:
        q.put(float((full - O.castle_parallel(*t, 0.25)).abs().max()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("batch,heads", [(2, 4), (1, 4)])
def test_two_rank_shards_gather_to_full(batch, heads):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29611 + batch
    procs = [ctx.Process(target=_worker, args=(r, 2, port, batch, heads, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert q.get(timeout=10) < 1e-6
