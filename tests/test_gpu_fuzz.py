"""GPU: seeded random shapes (ragged lengths around the 128-row tile, every supported head size, both
16-bit dtypes) through the parallel pass and the decode step, against the oracle."""
import random

import pytest
import torch

from oracle import castle_oracle as O

pytestmark = pytest.mark.gpu

_rng = random.Random(0)
PAR_CASES = [(_rng.choice([1, 1, 2, 3]), _rng.choice([1, 2, 3, 5]),
              _rng.choice([1, 2, 3, 7, 31, 64, 127, 128, 129, 200, 255, 256, 257, 383, 385, 511, 513, 700]),
              _rng.choice([16, 24, 32, 64, 64, 96, 128, 128]), _rng.choice(["bfloat16", "bfloat16", "float16"]))
             for _ in range(24)]
DEC_CASES = [(_rng.choice([1, 2, 5]), _rng.choice([1, 2, 3]), _rng.choice([16, 32, 64, 128]),
              _rng.choice([0, 1, 5, 100, 255, 256, 300, 1000, 2047, 3000]),
              _rng.choice(["bfloat16", "float16", "float32"])) for _ in range(16)]


@pytest.mark.parametrize("case", range(len(PAR_CASES)))
def test_parallel_random_shape(case):
    from lookahead_keys_attention_b200 import castle_attention_packed, check_status
    B, H, N, d, dt = PAR_CASES[case]
    dtype = getattr(torch, dt)
    torch.manual_seed(case)
    packed = (torch.randn(B, N, 6, H, d) * 3 ** -0.5).to(dtype)
    gout = torch.randn(B, H, N, d).to(dtype)
    p = packed.cuda().requires_grad_()
    out, U = castle_attention_packed(p, d ** -0.5, True)
    out.backward(gout.cuda())
    torch.cuda.synchronize()
    check_status()
    v = [packed[:, :, i].permute(0, 2, 1, 3).float() for i in range(6)]  # qu,ku,vu,qc,kc,vc
    ro = O.castle_parallel(v[3], v[4], v[5], v[0], v[1], v[2], d ** -0.5)
    rg = O.castle_parallel_bwd(v[3], v[4], v[5], v[0], v[1], v[2], d ** -0.5, gout.float())
    atol, rtol = (2e-2, 1e-2) if dtype == torch.bfloat16 else (5e-3, 5e-3)
    g = p.grad.float().cpu()
    pairs = [("out", out.float().cpu(), ro)] + [(n, g[:, :, s].permute(0, 2, 1, 3), r) for n, s, r in
                                                 zip(("dqc", "dkc", "dvc", "dqu", "dku", "dvu"), (3, 4, 5, 0, 1, 2), rg)]
    for name, a, b in pairs:
        excess = ((a - b).abs() - atol - rtol * b.abs()).max().item()
        assert excess <= 0, f"{PAR_CASES[case]} {name}: excess {excess:.3e}"


@pytest.mark.parametrize("case", range(len(DEC_CASES)))
def test_decode_random_shape(case):
    from lookahead_keys_attention_b200 import castle_decode_step, check_status
    B, H, d, t0, dt = DEC_CASES[case]
    dtype = getattr(torch, dt)
    torch.manual_seed(100 + case)
    mk = lambda *s: torch.randn(*s).to(dtype)
    cache = O.Cache(mk(B, H, t0, d) * 0.5, mk(B, H, t0, d), mk(B, H, t0, d), mk(B, H, t0, d))
    bufs = []
    for c in cache:
        b = torch.zeros(B, H, t0 + 3, d, dtype=dtype, device="cuda")
        b[:, :, :t0] = c.cuda()
        bufs.append(b)
    new = [mk(B, H, 1, d) for _ in range(6)]
    out = castle_decode_step(*[n.cuda() for n in new], *bufs, t0, d ** -0.5)
    ro, rc = O.castle_decode_step(*[n.float() for n in new], O.Cache(*(c.float() for c in cache)), d ** -0.5)
    torch.cuda.synchronize()
    check_status()
    atol = {torch.float32: 1e-4, torch.bfloat16: 2e-2, torch.float16: 3e-3}[dtype]
    assert (out.float().cpu() - ro).abs().max().item() <= 2 * atol
    assert (bufs[0][:, :, :t0 + 1].float().cpu() - rc.U).abs().max().item() <= 4 * atol
