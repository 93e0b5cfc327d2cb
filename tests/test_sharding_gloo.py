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


def _exchange_worker(rank, world, port, q):
    """Heads split inside a batch row: rows -> heads -> (oracle core) -> rows, forward and backward, against
    the unsharded module arithmetic."""
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lookahead_keys_attention_b200.sharding import heads_to_rows, rows_to_heads
    from oracle import castle_oracle as O
    torch.manual_seed(0)
    B, N, H, d, dim = 1, 12, 4, 8, 16
    w1, w2 = torch.randn(6 * H * d, dim) * 0.2, torch.randn(dim, H * d) * 0.2
    x, g = torch.randn(B, N, dim), torch.randn(B, N, dim)
    n = N // world
    xr = x[:, rank * n:(rank + 1) * n].clone().requires_grad_()
    w1r, w2r = w1.clone().requires_grad_(), w2.clone().requires_grad_()
    packed = rows_to_heads((xr @ w1r.T).view(B, n, 6, H, d))                 # every position, my heads
    assert packed.shape == (B, N, 6, H // world, d)
    qu, ku, vu, qc, kc, vc = (packed[:, :, i].permute(0, 2, 1, 3) for i in range(6))
    core = O.castle_parallel(qc, kc, vc, qu, ku, vu, d ** -0.5)              # (B, H/G, N, d)
    out = heads_to_rows(core) @ w2r.T                                         # my positions
    out.backward(g[:, rank * n:(rank + 1) * n])
    xf = x.clone().requires_grad_()
    ref = O.castle_module_forward(xf, w1, w2, H, d)
    ref.backward(g)
    err = max(float((out - ref[:, rank * n:(rank + 1) * n]).abs().max()),
              float((xr.grad - xf.grad[:, rank * n:(rank + 1) * n]).abs().max()))
    q.put(err)
    dist.barrier()
    dist.destroy_process_group()


def test_row_head_exchange_matches_unsharded_module():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_exchange_worker, args=(r, 2, 29631, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert max(q.get(timeout=10), q.get(timeout=10)) < 1e-5
