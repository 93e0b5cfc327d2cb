"""GPU: the cached single-token step against the CPU oracle, through the C ABI."""
import pytest
import torch

from oracle import castle_oracle as O

pytestmark = pytest.mark.gpu

TOL = {torch.float32: (1e-4, 1e-4), torch.bfloat16: (2e-2, 1e-2), torch.float16: (3e-3, 3e-3)}


def _run_steps(B, H, d, t0, steps, dtype, cap=None):
    from lookahead_keys_attention_b200 import castle_decode_step, check_status
    torch.manual_seed(1234 + d + t0)
    scale = d ** -0.5
    cap = cap or (t0 + steps + 3)
    mk = lambda *s: torch.randn(*s).to(dtype)
    cache = O.Cache(mk(B, H, t0, d) * 0.5, mk(B, H, t0, d), mk(B, H, t0, d), mk(B, H, t0, d))
    bufs = []
    for c in cache:
        buf = torch.zeros(B, H, cap, d, dtype=dtype, device="cuda")
        buf[:, :, :t0] = c.cuda()
        bufs.append(buf)
    ref_cache = O.Cache(*(c.float() for c in cache))
    atol, rtol = TOL[dtype]
    for s in range(steps):
        new = [mk(B, H, 1, d) for _ in range(6)]  # qc,kc,vc,qu,ku,vu
        out = castle_decode_step(*[n.cuda() for n in new], *bufs, t0 + s, scale)
        ref_out, ref_cache = O.castle_decode_step(*[n.float() for n in new], ref_cache, scale)
        torch.cuda.synchronize()
        check_status()
        assert torch.allclose(out.float().cpu(), ref_out, atol=atol, rtol=rtol), \
            f"step {s}: {(out.float().cpu() - ref_out).abs().max()}"
        t = t0 + s + 1
        for buf, rc, nm in zip(bufs, ref_cache, ref_cache._fields):
            assert torch.allclose(buf[:, :, :t].float().cpu(), rc, atol=atol * 4, rtol=rtol * 2), f"step {s}: cache {nm}"
        if dtype != torch.float32:  # keep the oracle on the values the device actually stored
            ref_cache = O.Cache(*(buf[:, :, :t].float().cpu() for buf in bufs))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", [16, 32, 64, 128])
def test_decode_small(d, dtype):
    _run_steps(2, 2, d, 5, 4, dtype)


@pytest.mark.parametrize("t0", [0, 1, 255, 256, 257, 1000])
def test_decode_lengths(t0):
    _run_steps(1, 3, 64, t0, 2, torch.bfloat16)


def test_decode_split_rows():
    # few (batch, head) pairs and a long cache: rows are split over several CTAs and merged
    _run_steps(1, 2, 128, 5000, 2, torch.bfloat16)
    _run_steps(2, 1, 64, 3000, 2, torch.float32)


def test_decode_rejects_full_cache():
    from lookahead_keys_attention_b200 import castle_decode_step
    z = lambda n: torch.zeros(1, 1, n, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="capacity"):
        castle_decode_step(*[z(1) for _ in range(6)], *[z(4) for _ in range(4)], 4, 0.125)
