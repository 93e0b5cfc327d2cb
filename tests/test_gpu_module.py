"""GPU: the `Castle` module against the golden vectors recorded from the reference module and
against the oracle - the five properties the reference's own tests check
(tests/test_lookahead.py in the reference: parallel == sequential :10-64, kernel == PyTorch path
forward and all gradients :67-143, causality :145-222, prefill-with-U then decode :225-282)."""
import pytest
import torch

from conftest import load_golden, rebuild_module_case
from oracle import castle_oracle as O

pytestmark = pytest.mark.gpu

MODULE_CASES = ["module_d16", "module_d16_prenorm", "module_d32", "module_d64_n256", "module_readme"]


def _build(cfg, w1, w2, nw, dtype=torch.float32):
    from lookahead_keys_attention_b200 import Castle
    m = Castle(cfg["dim"], heads=cfg["heads"], dim_head=cfg["dim_head"], prenorm=cfg["prenorm"]).cuda()
    sd = {"to_all_qkv.weight": w1, "combine_heads.weight": w2}
    if nw is not None:
        sd["norm.weight"] = nw
    m.load_state_dict(sd)  # same keys as the reference module
    return m.to(dtype)


@pytest.mark.parametrize("name", MODULE_CASES)
def test_module_fp32_forward_and_grads_vs_reference(name):
    """fp32 module: forward atol 1e-3, input and parameter gradients atol 2e-2
    (the reference's tolerances, tests/test_lookahead.py:114,135,143)."""
    g = load_golden(name)
    cfg, w1, w2, nw, x, gout = rebuild_module_case(g)
    st = cfg["stride"]
    m = _build(cfg, w1, w2, nw)
    xg = x.cuda().requires_grad_()
    out = m(xg)
    out.backward(gout.cuda())
    assert torch.allclose(out.detach().cpu()[:, ::st], torch.from_numpy(g["out"]), atol=1e-3)
    assert torch.allclose(xg.grad.cpu()[:, ::st], torch.from_numpy(g["dx"]), atol=2e-2)
    assert torch.allclose(m.to_all_qkv.weight.grad.cpu()[::37, ::11], torch.from_numpy(g["dw_qkv_sample"]), atol=2e-2)
    assert torch.allclose(m.combine_heads.weight.grad.cpu()[::11, ::13], torch.from_numpy(g["dw_out_sample"]), atol=2e-2)


@pytest.mark.parametrize("name", MODULE_CASES)
@torch.no_grad()
def test_module_prefill_then_decode_vs_reference(name):
    """Prefill (kernel emits U) + cached single-token steps == the reference's sequential outputs, atol 1e-3."""
    from lookahead_keys_attention_b200 import check_status
    g = load_golden(name)
    cfg, w1, w2, nw, x, _ = rebuild_module_case(g)
    st, split, n = cfg["stride"], cfg["split"], cfg["n"]
    m = _build(cfg, w1, w2, nw)
    xc = x.cuda()
    pre, cache = m(xc[:, :split], return_next_cache=True)
    assert cache.U.shape == (cfg["b"], cfg["heads"], split, cfg["dim_head"])
    gU = torch.from_numpy(g["prefill_U"])
    assert torch.allclose(cache.U.cpu(), gU, atol=1e-3 + 2 * 2.0 ** -11 * gU.abs().max().item())
    outs = [pre]
    for t in range(split, n):
        o, cache = m(xc[:, t:t + 1], cache=cache)  # return_next_cache defaults to True for one token
        assert cache.kc_cache.shape[-2] == t + 1
        outs.append(o)
    seq = torch.cat(outs, 1).cpu()
    check_status()
    assert torch.allclose(seq[:, ::st], torch.from_numpy(g["seq_out"]), atol=1e-3)
    assert torch.allclose(cache.qu_cache.cpu()[:, :, ::st], torch.from_numpy(g["final_qu"]), atol=1e-3)
    # parallel == sequential (README contract, atol 1e-3)
    assert torch.allclose(seq, m(xc).cpu(), atol=1e-3)


@torch.no_grad()
def test_module_decode_from_empty_cache_and_functional_mode():
    from lookahead_keys_attention_b200 import Castle
    torch.manual_seed(0)
    m = Castle(64, heads=2, dim_head=32, inplace_cache=False).cuda()
    x = torch.randn(2, 6, 64, device="cuda")
    cache, outs, caches = None, [], []
    for t in range(6):
        o, cache = m(x[:, t:t + 1], cache=cache)
        outs.append(o)
        caches.append(cache)
    assert torch.allclose(torch.cat(outs, 1), m(x), atol=1e-3)
    # functional mode: an old cache is still what it was, and stepping from it again gives the same answer
    o_again, _ = m(x[:, 3:4], cache=caches[2])
    assert torch.allclose(o_again, outs[3], atol=1e-6)


@torch.no_grad()
def test_module_causality_bf16():
    from lookahead_keys_attention_b200 import Castle
    torch.manual_seed(1)
    m = Castle(128, heads=2, dim_head=64, prenorm=True).cuda().bfloat16()
    x = torch.randn(2, 64, 128, device="cuda").bfloat16()
    assert torch.allclose(m(x)[:, :32].float(), m(x[:, :32]).float(), atol=1e-3)


def test_module_bf16_vs_fp32_oracle():
    """bf16 module at a few hundred tokens: |a-b| <= 2e-2 + 1e-2|b| against the fp32 oracle on the
    same bf16-rounded weights and inputs, for the output, dx and both weight gradients."""
    from lookahead_keys_attention_b200 import Castle
    torch.manual_seed(2)
    m = Castle(256, heads=4, dim_head=64).cuda().bfloat16()
    x = torch.randn(2, 512, 256).bfloat16()
    gout = torch.randn(2, 512, 256).bfloat16()
    xg = x.cuda().requires_grad_()
    out = m(xg)
    out.backward(gout.cuda())
    w1 = m.to_all_qkv.weight.detach().float().cpu().requires_grad_()
    w2 = m.combine_heads.weight.detach().float().cpu().requires_grad_()
    xr = x.float().requires_grad_()
    ref = O.castle_module_forward(xr, w1, w2, 4, 64)
    ref.backward(gout.float())
    for what, a, b in [("out", out, ref.detach()), ("dx", xg.grad, xr.grad)]:
        err = (a.float().cpu() - b).abs()
        assert bool((err <= 2e-2 + 1e-2 * b.abs()).all()), f"{what}: {err.max().item():.3e}"
    # weight gradients sum over 1024 tokens: compare relative to their scale (rel-Frobenius 1e-2)
    for what, a, b in [("dW_qkv", m.to_all_qkv.weight.grad, w1.grad), ("dW_out", m.combine_heads.weight.grad, w2.grad)]:
        rel = ((a.float().cpu() - b).norm() / b.norm()).item()
        assert rel < 1e-2, f"{what}: rel-F {rel:.3e}"


@torch.no_grad()
@pytest.mark.parametrize("prenorm", [False, True])
def test_module_rotary_parallel_equals_sequential_and_is_causal(prenorm):
    """With rotary_emb=True (this package's own rotary embedding; the reference's third-party one is not
    available to compare values against) the reference's two self-consistency properties still hold:
    parallel == prefill + cached steps (tests/test_lookahead.py:10-64 there) and prefix invariance (:145-182)."""
    from lookahead_keys_attention_b200 import Castle
    torch.manual_seed(4)
    m = Castle(64, heads=2, dim_head=32, rotary_emb=True, prenorm=prenorm).cuda()
    x = torch.randn(2, 40, 64, device="cuda")
    full = m(x)
    out, cache = m(x[:, :24], return_next_cache=True)
    outs = [out]
    for t in range(24, 40):
        o, cache = m(x[:, t:t + 1], cache=cache)
        outs.append(o)
    assert torch.allclose(torch.cat(outs, 1), full, atol=1e-3)
    assert torch.allclose(full[:, :20], m(x[:, :20]), atol=1e-3)


@torch.no_grad()
def test_module_cache_regrows_when_capacity_runs_out():
    from lookahead_keys_attention_b200 import Castle
    torch.manual_seed(5)
    m = Castle(64, heads=2, dim_head=32, cache_headroom=2).cuda()
    x = torch.randn(1, 20, 64, device="cuda")
    out, cache = m(x[:, :3], return_next_cache=True)
    outs, ptrs = [out], set()
    for t in range(3, 20):
        o, cache = m(x[:, t:t + 1], cache=cache)
        outs.append(o)
        ptrs.add(cache.U.data_ptr())
        assert cache.U.shape[-2] == t + 1
    assert len(ptrs) > 1  # the buffers were re-allocated at least once on the way
    assert torch.allclose(torch.cat(outs, 1), m(x), atol=1e-3)


def test_forward_chunking_of_scratch(monkeypatch):
    """The forward's partial-soft-max scratch is bounded by cutting the (batch, head) grid into
    launches: whole batch rows when they fit, head ranges of one batch row when they do not."""
    from lookahead_keys_attention_b200 import castle_attention_packed, ops
    torch.manual_seed(6)
    packed = (torch.randn(3, 300, 6, 4, 64, device="cuda") * 0.5).bfloat16().requires_grad_()
    g = torch.randn(3, 4, 300, 64, device="cuda").bfloat16()
    ref, ref_u = castle_attention_packed(packed, 0.125, True)
    ref.backward(g)
    ref_grad, packed.grad = packed.grad, None
    per_pair = 6 * 128 * (8 + 2 * 64)          # 3 query blocks -> 6 tiles of (max, sum) + a 16-bit row
    for limit in (4 * per_pair, 3 * per_pair, per_pair):   # one batch row; 3 + 1 heads; one pair per launch
        monkeypatch.setattr(ops, "MAX_WORKSPACE_BYTES", limit)
        out, u = castle_attention_packed(packed, 0.125, True)
        assert torch.equal(out, ref) and torch.equal(u, ref_u)
        out.backward(g)   # the saved per-pair state of a head-chunked forward feeds the backward as usual
        assert torch.allclose(packed.grad.float(), ref_grad.float(), atol=3e-2, rtol=3e-2)
        packed.grad = None
    monkeypatch.setattr(ops, "MAX_WORKSPACE_BYTES", per_pair - 1)
    with pytest.raises(RuntimeError, match="more than"):
        castle_attention_packed(packed, 0.125, True)


@torch.no_grad()
@pytest.mark.parametrize("d,rotary,N", [(64, False, 333), (128, False, 333), (64, True, 333), (64, False, 1333)])
def test_prefill_kernels_write_the_decode_caches(d, rotary, N, monkeypatch):
    """Prefill hand-off (reference: lookahead_keys_attention.py:161-164): for 16-bit modules the forward
    kernels fill all four caches themselves - U from the final lookahead state, qu/kc/vc from the tiles
    in shared memory - straight into the capacity buffers; the module makes no copy pass."""
    from lookahead_keys_attention_b200 import Castle, ModuleCache
    torch.manual_seed(7)
    H = 3              # N = 333: the last key block is ragged, rows beyond N must stay untouched;
    #                    N = 1333 at dim_head 64: few pairs and 11 key blocks, so the walks run as segments
    m = Castle(96, heads=H, dim_head=d, rotary_emb=rotary).cuda().bfloat16()
    x = torch.randn(2, N, 96, device="cuda").bfloat16()
    copies = []
    real_copy = torch.Tensor.copy_
    monkeypatch.setattr(torch.Tensor, "copy_", lambda self, *a, **k: (copies.append(self.shape), real_copy(self, *a, **k))[1])
    out, cache = m(x, return_next_cache=True)
    monkeypatch.setattr(torch.Tensor, "copy_", real_copy)
    assert not copies, f"prefill made copy passes: {copies}"
    assert isinstance(cache, ModuleCache) and cache.is_current()
    bufs = cache._state.bufs
    for c, b in zip(cache, bufs):
        assert c.data_ptr() == b.data_ptr() and c.shape == (2, H, N, d) and b.shape[2] > N
    qu, ku, vu, qc, kc, vc = m._split(m.to_all_qkv(x))
    if rotary:
        qc, kc, qu, ku, vu = (m.rotary_emb.rotate(t, 0) for t in (qc, kc, qu, ku, vu))
    assert torch.equal(cache.qu_cache, qu) and torch.equal(cache.kc_cache, kc) and torch.equal(cache.vc_cache, vc)
    ref_u = O.castle_parallel(*[t.float().cpu() for t in (qc, kc, vc, qu, ku, vu)], m.scale, return_U=True)[1]
    err = (cache.U.float().cpu() - ref_u).abs()
    # U is an un-normalised sum of up to N rows: a few bf16 ulps of its largest entry on top of the rule
    assert bool((err <= 2e-2 + 2 * 2.0 ** -8 * ref_u.abs().max() + 1e-2 * ref_u.abs()).all()), err.max().item()
    # and the hand-off works: cached steps continue the sequence
    x2 = torch.randn(2, 3, 96, device="cuda").bfloat16()
    full = m(torch.cat((x, x2), 1))
    for t in range(3):
        o, cache = m(x2[:, t:t + 1], cache=cache)
        assert torch.allclose(o.float(), full[:, N + t:N + t + 1].float(), atol=2e-2, rtol=2e-2)


@torch.no_grad()
def test_decode_never_writes_a_callers_tensor():
    """A cache made of the caller's own tensors (here: prefix slices of larger tensors, which look just
    like capacity buffers) is copied before the in-place step; the caller's memory stays as it was, and
    decoding twice from it gives the same answer."""
    from lookahead_keys_attention_b200 import Cache, Castle
    torch.manual_seed(8)
    m = Castle(64, heads=2, dim_head=64).cuda().bfloat16()
    big = [torch.randn(2, 2, 10, 64, device="cuda").bfloat16() for _ in range(4)]
    keep = [b.clone() for b in big]
    foreign = Cache(*(b[:, :, :4] for b in big))
    x = torch.randn(2, 1, 64, device="cuda").bfloat16()
    o1, c1 = m(x, cache=foreign)
    o2, c2 = m(x, cache=foreign)
    torch.cuda.synchronize()
    assert all(torch.equal(b, k) for b, k in zip(big, keep))
    assert torch.equal(o1, o2) and c1.U.data_ptr() != c2.U.data_ptr() and c1.U.data_ptr() != big[0].data_ptr()
    # a stale module cache is refused rather than silently decoded from rewritten rows
    _, c3 = m(x, cache=c1)
    with pytest.raises(RuntimeError, match="advanced in place"):
        m(x, cache=c1)
    assert c3.is_current()
