"""GPU: the benchmark configurations at their full sizes.

The dense oracle cannot hold a whole configuration (it materialises N x N tensors per head), so
at full size the kernels are checked (a) against the oracle on a sampled (batch, head) pair -
the pairs are independent, so one pair's result does not depend on the others being there -
and (b) through size-independent properties: prefix invariance of the forward, linearity of
the backward in the upstream gradient, and parallel == prefill + cached decode."""
import pytest
import torch

from oracle import castle_oracle as O

pytestmark = pytest.mark.gpu

PROJ_STD = 3 ** -0.5
TOL = (2e-2, 1e-2)  # |a-b| <= 2e-2 + 1e-2 |b|


def _close(a, b, what, tol=TOL):
    err = (a - b).abs()
    bound = tol[0] + tol[1] * b.abs()
    assert bool((err <= bound).all()), f"{what}: max err {err.max().item():.3e}, worst excess {(err - bound).max().item():.3e}"


def _packed(B, N, H, d, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(B, N, 6, H, d, device="cuda", generator=g) * PROJ_STD).bfloat16()


def _oracle_pair(ins, gout, d):
    """fp32 oracle for one (N, d) head: the dense form while its N x N tensors are small, the blockwise
    recurrence (same algebra, checked against the dense form on the CPU) beyond that."""
    qu, ku, vu, qc, kc, vc = ins
    n = qc.shape[0]
    if n <= 4096:
        ro, rU = O.castle_parallel(qc, kc, vc, qu, ku, vu, d ** -0.5, return_U=True)
        return ro, rU, O.castle_parallel_bwd(qc, kc, vc, qu, ku, vu, d ** -0.5, gout)
    ro, rU, lse = O.castle_parallel_blockwise(qc, kc, vc, qu, ku, vu, d ** -0.5, block=128)
    return ro, rU, O.castle_parallel_bwd_blockwise(qc, kc, vc, qu, ku, vu, d ** -0.5, ro, lse, rU, gout, block=128)


@pytest.mark.parametrize("B,N,H,d,pair", [(4, 4096, 16, 64, (2, 11)), (1, 8192, 4, 128, (0, 3)), (1, 8192, 3, 64, (0, 1)),
                                          (1, 16384, 2, 128, (0, 1))])
def test_sampled_pair_matches_oracle_at_full_size(B, N, H, d, pair):
    """Config 2 (B=4 N=4096 H=16 d=64) in full, and long sequences up to the long-context configuration's
    N = 16384 at d = 128: forward, U and ALL six gradients of one (batch, head) pair inside
    |a-b| <= 2e-2 + 1e-2|b| of the fp32 oracle on the same bf16 inputs - no weaker bar for any of them."""
    from lookahead_keys_attention_b200 import castle_attention_packed, check_status
    packed = _packed(B, N, H, d, seed=N + d).requires_grad_()
    g = torch.Generator(device="cuda").manual_seed(1)
    gout = torch.randn(B, H, N, d, device="cuda", generator=g).bfloat16()
    out, U = castle_attention_packed(packed, d ** -0.5, True)
    out.backward(gout)
    torch.cuda.synchronize()
    check_status()
    b, h = pair
    ins = [packed.detach()[b, :, i, h].float().cpu() for i in range(6)]  # qu,ku,vu,qc,kc,vc  (N, d)
    ro, rU, rg = _oracle_pair(ins, gout[b, h].float().cpu(), d)          # rg: dqc,dkc,dvc,dqu,dku,dvu
    _close(out[b, h].float().cpu(), ro, "out")
    ulp = 2.0 ** -8
    _close(U[b, h].float().cpu(), rU, "U", (TOL[0] + 2 * ulp * rU.abs().max().item(), TOL[1]))
    got = packed.grad[b, :, :, h].float().cpu()  # (N, 6, d)
    worst = {}
    for name, slot, ref in [("dqc", 3, rg[0]), ("dkc", 4, rg[1]), ("dvc", 5, rg[2]), ("dqu", 0, rg[3]), ("dku", 1, rg[4]), ("dvu", 2, rg[5])]:
        err = (got[:, slot] - ref).abs()
        worst[name] = (round(err.max().item(), 4), round((err - TOL[0] - TOL[1] * ref.abs()).max().item(), 4))
    print(f"N={N} d={d}: max error / worst excess over the rule per gradient: {worst}")
    bad = {k: v for k, v in worst.items() if v[1] > 0}
    assert not bad, f"outside |a-b| <= 2e-2 + 1e-2|b|: {bad} (all: {worst})"


def test_upstream_gradient_rescaling_is_exact():
    """Where bf16 callers run on fp16 operands (long sequences) the upstream gradient is rescaled by a power
    of two: gradients of a tiny and of a large upstream gradient are the same up to that factor."""
    from lookahead_keys_attention_b200 import castle_attention_packed, ops
    N = ops.LONG_SEQ_FP16
    packed = _packed(1, N, 1, 64, seed=5)
    gen = torch.Generator(device="cuda").manual_seed(7)
    gout = torch.randn(1, 1, N, 64, device="cuda", generator=gen).bfloat16()

    def grads(scale):
        p = packed.clone().requires_grad_()
        castle_attention_packed(p, 0.125, False).backward((gout.float() * scale).bfloat16())
        return p.grad.float()

    base = grads(1.0)
    for k in (-20, 12):   # 1e-6 x and 4096 x the gradient: both out of fp16's comfortable range without the rescaling
        got = grads(2.0 ** k) * 2.0 ** -k
        for slot in (0, 4, 5):   # dqu, dkc, dvc are written by their owner: bit for bit
            assert torch.equal(got[:, :, slot], base[:, :, slot])
        assert torch.allclose(got, base, atol=3e-2, rtol=3e-2)   # the other three are fp32 sums in arrival order


def test_prefix_invariance_and_backward_linearity_config2():
    from lookahead_keys_attention_b200 import castle_attention_packed
    B, N, H, d = 4, 4096, 16, 64
    packed = _packed(B, N, H, d, seed=9)
    full = castle_attention_packed(packed, 0.125, False)
    half = castle_attention_packed(packed[:, :2048].contiguous(), 0.125, False)
    assert torch.allclose(full[:, :, :2048].float(), half.float(), atol=1e-3)   # causality

    def grads(gout):
        p = packed.clone().requires_grad_()
        castle_attention_packed(p, 0.125, False).backward(gout)
        return p.grad.float()

    gen = torch.Generator(device="cuda").manual_seed(3)
    g1 = torch.randn(B, H, N, d, device="cuda", generator=gen).bfloat16()
    g2 = torch.randn(B, H, N, d, device="cuda", generator=gen).bfloat16()
    mix = (0.5 * g1.float() - 0.25 * g2.float()).bfloat16()
    lin = 0.5 * grads(g1) - 0.25 * grads(g2)
    got = grads(mix)
    # bf16 rounding of the mixed upstream gradient and of the results bounds the mismatch
    rel = ((got - lin).norm() / lin.norm()).item()
    assert rel < 1e-2, rel


@torch.no_grad()
def test_prefill_then_decode_equals_parallel_d128():
    """Config-5 geometry on a slice: Castle(2048, 16 heads of 128), prefix 2048, then 16 cached steps."""
    from lookahead_keys_attention_b200 import Castle, check_status
    torch.manual_seed(0)
    m = Castle(2048, heads=16, dim_head=128).cuda().bfloat16()
    x = torch.randn(2, 2064, 2048, device="cuda").bfloat16()
    ref = m(x)
    out, cache = m(x[:, :2048], return_next_cache=True)
    outs = [out]
    for t in range(2048, 2064):
        o, cache = m(x[:, t:t + 1], cache=cache)
        outs.append(o)
    check_status()
    _close(torch.cat(outs, 1).float().cpu(), ref.float().cpu(), "prefill + decode vs parallel")


def test_repeatability_config2():
    """Nothing in the forward, and nothing in dkc / dvc / dqu, is reduced atomically: two runs on the same
    inputs must agree bit for bit at full size (a race in a shared-memory or TMEM hand-off would show here)."""
    from lookahead_keys_attention_b200 import castle_attention_packed, check_status
    packed = _packed(4, 4096, 16, 64, seed=21)
    gen = torch.Generator(device="cuda").manual_seed(5)
    gout = torch.randn(4, 16, 4096, 64, device="cuda", generator=gen).bfloat16()
    res = []
    for _ in range(3):
        p = packed.clone().requires_grad_()
        out, U = castle_attention_packed(p, 0.125, True)
        out.backward(gout)
        res.append((out.detach().clone(), U.clone(), p.grad.clone()))
    torch.cuda.synchronize()
    check_status()
    for out, U, g in res[1:]:
        assert torch.equal(out, res[0][0]) and torch.equal(U, res[0][1])
        for slot in (0, 4, 5):  # dqu, dkc, dvc
            assert torch.equal(g[:, :, slot], res[0][2][:, :, slot])
        # dqc, dku, dvu are fp32 sums in arrival order: equal up to a few bf16 ulps of the result
        assert torch.allclose(g.float(), res[0][2].float(), atol=3e-2, rtol=3e-2)


def test_repeatability_d128():
    """Same at dim_head 128 (its kernels hand tiles over in tensor memory, refill shared-memory panels lane by
    lane, and the two backward kernels pass three tiles per step through global memory): out, U, dqu, dkc and
    dvc bit for bit; dqc, dku, dvu are fp32 sums in arrival order."""
    from lookahead_keys_attention_b200 import castle_attention_packed, check_status
    packed = _packed(1, 4096, 8, 128, seed=22)
    gen = torch.Generator(device="cuda").manual_seed(6)
    gout = torch.randn(1, 8, 4096, 128, device="cuda", generator=gen).bfloat16()
    res = []
    for _ in range(4):
        p = packed.clone().requires_grad_()
        out, U = castle_attention_packed(p, 128 ** -0.5, True)
        out.backward(gout)
        res.append((out.detach().clone(), U.clone(), p.grad.clone()))
    torch.cuda.synchronize()
    check_status()
    for out, U, g in res[1:]:
        assert torch.equal(out, res[0][0]) and torch.equal(U, res[0][1])
        for slot in (0, 4, 5):  # dqu, dkc, dvc
            assert torch.equal(g[:, :, slot], res[0][2][:, :, slot])
        assert torch.allclose(g.float(), res[0][2].float(), atol=3e-2, rtol=3e-2)
