"""GPU: the parallel CASTLE pass (forward, backward) against the CPU oracle and the
golden vectors recorded from the reference, through the operator / C ABI."""
import pytest
import torch

from conftest import load_golden, rebuild_core_case
from oracle import castle_oracle as O

pytestmark = pytest.mark.gpu


def _inputs(B, H, N, d, dtype, seed=0):
    torch.manual_seed(seed)
    # qu,ku,vu,qc,kc,vc as views of one packed projection output, like the module produces them
    packed = torch.randn(B, N, 6, H, d).to(dtype)
    return packed


def _views(packed):
    return [packed[:, :, i].permute(0, 2, 1, 3) for i in range(6)]  # qu,ku,vu,qc,kc,vc


def _close(a, b, atol, rtol, what):
    err = (a - b).abs()
    bound = atol + rtol * b.abs()
    assert bool((err <= bound).all()), f"{what}: max err {err.max().item():.3e}, worst excess {(err - bound).max().item():.3e}"


# tolerance the task states for 16-bit runs: |a-b| <= 2e-2 + 1e-2*|b| against the fp32
# oracle evaluated on the same (already rounded) inputs
BF16_TOL = (2e-2, 1e-2)


@pytest.mark.parametrize("B,H,N,d", [(1, 1, 128, 64), (2, 2, 256, 64), (1, 2, 200, 64), (1, 1, 1, 64), (1, 1, 129, 64),
                                     (1, 1, 130, 128), (2, 1, 384, 128), (1, 2, 40, 16), (1, 1, 77, 32)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_forward_matches_oracle(B, H, N, d, dtype):
    from lookahead_keys_attention_b200 import castle_attention, check_status
    packed = _inputs(B, H, N, d, dtype, seed=N + d)
    qu, ku, vu, qc, kc, vc = _views(packed.cuda())
    scale = d ** -0.5
    out, U = castle_attention(qc, kc, vc, qu, ku, vu, scale, True)
    torch.cuda.synchronize()
    check_status()
    rqu, rku, rvu, rqc, rkc, rvc = [t.float() for t in _views(packed)]
    ro, rU = O.castle_parallel(rqc, rkc, rvc, rqu, rku, rvu, scale, return_U=True)
    atol, rtol = BF16_TOL if dtype == torch.bfloat16 else (3e-3, 3e-3)
    _close(out.float().cpu(), ro, atol, rtol, "out")
    # U is an un-normalised sum of up to N gate-weighted rows, so its rounding error scales with
    # its magnitude: allow a few 16-bit ulps of the largest entry on top of the element-wise rule
    ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    _close(U.float().cpu(), rU, atol + 2 * ulp * rU.abs().max().item(), rtol, "U")
    out2 = castle_attention(qc, kc, vc, qu, ku, vu, scale, False)
    assert torch.equal(out2, out)


@pytest.mark.parametrize("B,H,N", [(1, 2, 1100), (2, 1, 2048), (1, 1, 3000)])
def test_forward_walk_segments_match_oracle(B, H, N):
    """Few (batch, head) pairs and many key blocks: the dim_head-64 forward cuts each long walk into
    segments, and a segment that starts mid-walk rebuilds its lookahead state with a state-only pre-loop.
    Output, U (written by the last segment only) and the saved state (through the backward) must match."""
    from lookahead_keys_attention_b200 import castle_attention, check_status
    d, scale = 64, 0.125
    packed = (_inputs(B, H, N, d, torch.float32, seed=N) * 3 ** -0.5).bfloat16()
    views = [t.cuda().requires_grad_() for t in _views(packed)]
    qu, ku, vu, qc, kc, vc = views
    out, U = castle_attention(qc, kc, vc, qu, ku, vu, scale, True)
    gout = torch.randn(B, H, N, d, generator=torch.Generator().manual_seed(1)).bfloat16()
    out.backward(gout.cuda())
    torch.cuda.synchronize()
    check_status()
    r = [t.float() for t in _views(packed)]
    ro, rU = O.castle_parallel(r[3], r[4], r[5], r[0], r[1], r[2], scale, return_U=True)
    _close(out.float().cpu(), ro, *BF16_TOL, "out")
    _close(U.float().cpu(), rU, BF16_TOL[0] + 2 * 2.0 ** -8 * rU.abs().max().item(), BF16_TOL[1], "U")
    rg = O.castle_parallel_bwd(r[3], r[4], r[5], r[0], r[1], r[2], scale, gout.float())   # dqc,dkc,dvc,dqu,dku,dvu
    for name, t, ref in zip(("dqc", "dkc", "dvc", "dqu", "dku", "dvu"), (qc, kc, vc, qu, ku, vu), rg):
        _close(t.grad.float().cpu(), ref, *BF16_TOL, name)


@pytest.mark.parametrize("name", ["core_n40_d16", "core_n200_d64", "core_n130_d128"])
def test_forward_matches_reference_golden(name):
    from lookahead_keys_attention_b200 import castle_attention
    g = load_golden(name)
    (b, h, n, d), packed, gout = rebuild_core_case(g)
    p16 = packed.float().half()  # fp32 callers run with fp16 operands
    qu, ku, vu, qc, kc, vc = [t.cuda() for t in O.split_heads(p16, h)]
    out, U = castle_attention(qc, kc, vc, qu, ku, vu, d ** -0.5, True)
    merged = out.permute(0, 2, 1, 3).reshape(b, n, h * d).float().cpu()
    _close(merged, torch.from_numpy(g["out"]), 3e-3, 3e-3, "out vs reference")
    gU = torch.from_numpy(g["U"])
    _close(U.float().cpu(), gU, 3e-3 + 2 * 2.0 ** -11 * gU.abs().max().item(), 3e-3, "U vs reference")


@pytest.mark.parametrize("B,H,N,d", [(2, 8, 128, 64), (1, 2, 300, 64), (1, 2, 300, 128)])
def test_forward_fp32_caller_atol_1e3(B, H, N, d):
    """fp32 caller (first case: the README shape's head geometry): atol 1e-3 against the fp32 oracle, for both
    forward kernels and more than one key block."""
    from lookahead_keys_attention_b200 import castle_attention
    packed = _inputs(B, H, N, d, torch.float32, seed=7) * 0.5
    qu, ku, vu, qc, kc, vc = _views(packed.cuda())
    out = castle_attention(qc, kc, vc, qu, ku, vu, d ** -0.5, False)
    assert out.dtype == torch.float32
    rqu, rku, rvu, rqc, rkc, rvc = _views(packed)
    ro = O.castle_parallel(rqc, rkc, rvc, rqu, rku, rvu, d ** -0.5)
    _close(out.cpu(), ro, 1e-3, 0.0, "out")


def test_forward_causality():
    from lookahead_keys_attention_b200 import castle_attention
    packed = _inputs(1, 2, 300, 64, torch.bfloat16, seed=3).cuda()
    qu, ku, vu, qc, kc, vc = _views(packed)
    full = castle_attention(qc, kc, vc, qu, ku, vu, 0.125, False)
    half = castle_attention(*[t[:, :, :150] for t in (qc, kc, vc, qu, ku, vu)], 0.125, False)
    _close(full[:, :, :150].float(), half.float(), 1e-3, 0.0, "prefix invariance")


# q/k/v of a default-initialised projection of x ~ N(0,1) have std 1/sqrt(3): nn.Linear draws
# its weights uniformly in +-1/sqrt(fan_in).  The tolerance tests use inputs of that scale.
PROJ_STD = 3 ** -0.5


def _grads(B, H, N, d, dtype, seed, std=PROJ_STD, want_ref16=False):
    from lookahead_keys_attention_b200 import castle_attention, check_status
    packed = (_inputs(B, H, N, d, torch.float32, seed=seed) * std).to(dtype)
    torch.manual_seed(seed + 1)
    gout = torch.randn(B, H, N, d).to(dtype)
    pk = packed.cuda().requires_grad_()
    qu, ku, vu, qc, kc, vc = _views(pk)
    scale = d ** -0.5
    out = castle_attention(qc, kc, vc, qu, ku, vu, scale, False)
    out.backward(gout.cuda())
    torch.cuda.synchronize()
    check_status()
    rqu, rku, rvu, rqc, rkc, rvc = [t.float() for t in _views(packed)]
    ref = O.castle_parallel_bwd(rqc, rkc, rvc, rqu, rku, rvu, scale, gout.float())  # dqc,dkc,dvc,dqu,dku,dvu
    got = pk.grad.float().cpu()
    gqu, gku, gvu, gqc, gkc, gvc = _views(got)
    if want_ref16:  # the reference's own arithmetic in the 16-bit dtype, on the CPU
        r16 = _views(packed)
        ref16 = O.castle_parallel_bwd(r16[3], r16[4], r16[5], r16[0], r16[1], r16[2], scale, gout)
        return [(g, r, r16_.float()) for g, r, r16_ in zip((gqc, gkc, gvc, gqu, gku, gvu), ref, ref16)]
    return dict(dqc=(gqc, ref[0]), dkc=(gkc, ref[1]), dvc=(gvc, ref[2]), dqu=(gqu, ref[3]), dku=(gku, ref[4]), dvu=(gvu, ref[5]))


@pytest.mark.parametrize("B,H,N,d", [(1, 1, 128, 64), (1, 1, 256, 64), (2, 2, 384, 64), (1, 2, 200, 64), (1, 1, 1, 64),
                                     (1, 1, 129, 64), (1, 2, 40, 16), (1, 1, 77, 32), (1, 1, 1024, 64),
                                     (1, 1, 128, 128), (1, 1, 130, 128), (1, 2, 384, 128), (2, 1, 300, 128),
                                     (1, 1, 1, 128), (1, 1, 72, 96), (1, 1, 640, 128)])
def test_backward_matches_oracle_bf16(B, H, N, d):
    res = _grads(B, H, N, d, torch.bfloat16, seed=N + d)
    for name, (g, r) in res.items():
        _close(g, r, *BF16_TOL, name)


def test_backward_d128_pairs_in_chunks(monkeypatch):
    """dim_head 128: with a workspace that holds the tile hand-over scratch of two (batch, head) pairs only, the
    five pairs run as three launch pairs (2 + 2 + 1) and the gradients are the same as in one chunk: the
    owner-written ones bit for bit, the reduced ones to a few ulps; with an even smaller bound one pair runs at a time.
    (That the library itself refuses a workspace that holds no pair is checked on the CPU in test_host.py.)"""
    from lookahead_keys_attention_b200 import ops
    B, H, N, d = 1, 5, 640, 128
    whole = _grads(B, H, N, d, torch.bfloat16, seed=77)
    nblk = (N + 127) // 128
    pair = nblk * (nblk + 1) // 2 * 3 * 32768
    acc = (B * H * N * (3 * d + 1) * 4 + 1023) // 1024 * 1024
    monkeypatch.setattr(ops, "MAX_WORKSPACE_BYTES", acc + 2 * pair + 512)
    ops.release_workspaces()
    chunked = _grads(B, H, N, d, torch.bfloat16, seed=77)
    for name, (g, r) in chunked.items():
        _close(g, r, *BF16_TOL, name)
        if name in ("dkc", "dvc", "dqu"):
            assert torch.equal(g, whole[name][0]), name
        else:
            assert torch.allclose(g, whole[name][0], atol=3e-2, rtol=3e-2), name
    # below one pair's worth the operator still passes the least the library accepts: one pair per chunk
    monkeypatch.setattr(ops, "MAX_WORKSPACE_BYTES", 1 << 20)
    ops.release_workspaces()
    single = _grads(B, H, N, d, torch.bfloat16, seed=77)
    for name in ("dkc", "dvc", "dqu"):
        assert torch.equal(single[name][0], whole[name][0]), name
    ops.release_workspaces()


@pytest.mark.parametrize("B,H,N,d", [(1, 2, 256, 64), (1, 1, 200, 32), (1, 1, 260, 128)])
def test_backward_matches_oracle_fp16(B, H, N, d):
    res = _grads(B, H, N, d, torch.float16, seed=N + d)
    for name, (g, r) in res.items():
        _close(g, r, 5e-3, 5e-3, name)


@pytest.mark.parametrize("name", ["core_n200_d64", "core_n130_d128", "core_n40_d16"])
def test_backward_matches_reference_golden(name):
    """Gradients of the reference's own autograd (fp64, recorded) vs the kernels run with fp16 operands."""
    from lookahead_keys_attention_b200 import castle_attention
    g = load_golden(name)
    (b, h, n, d), packed, gout = rebuild_core_case(g)
    pk = packed.float().cuda().requires_grad_()
    qu, ku, vu, qc, kc, vc = O.split_heads(pk, h)
    out = castle_attention(qc, kc, vc, qu, ku, vu, d ** -0.5, False)
    out.backward(gout.float().view(b, n, h, d).permute(0, 2, 1, 3).cuda())
    _close(pk.grad.cpu(), torch.from_numpy(g["dpacked"]), 2e-2, 0.0, "packed grads vs reference (atol 2e-2)")


@pytest.mark.parametrize("N", [256, 1024])
def test_backward_unit_variance_inputs_no_worse_than_16bit_reference(N):
    """With N(0,1) q/k/v the lookahead state reaches tens and 16-bit rounding alone breaks the
    element-wise rule - for the reference's own bf16 run too.  There the bar is the reference's
    error: the kernel's max error stays within 1.5x of the CPU bf16 run's."""
    names = ("dqc", "dkc", "dvc", "dqu", "dku", "dvu")
    for name, (g, r, r16) in zip(names, _grads(1, 1, N, 64, torch.bfloat16, seed=N, std=1.0, want_ref16=True)):
        e, e16 = (g - r).abs().max().item(), (r16 - r).abs().max().item()
        assert e <= 1.5 * e16 + 2e-3, f"{name}: kernel {e:.3e} vs reference-bf16 {e16:.3e}"


def test_backward_deterministic_forward_state():
    """Two identical calls give identical key-block gradients (dkc, dvc, dqu are not reduced atomically)."""
    a = _grads(1, 2, 300, 64, torch.bfloat16, seed=11)
    b = _grads(1, 2, 300, 64, torch.bfloat16, seed=11)
    for name in ("dkc", "dvc", "dqu"):
        assert torch.equal(a[name][0], b[name][0]), name


def test_packed_operator_equals_six_view_operator():
    from lookahead_keys_attention_b200 import castle_attention, castle_attention_packed
    packed = (_inputs(2, 2, 300, 64, torch.float32, seed=5) * PROJ_STD).bfloat16().cuda()
    g = torch.randn(2, 2, 300, 64, device="cuda").bfloat16()
    a = packed.clone().requires_grad_()
    qu, ku, vu, qc, kc, vc = _views(a)
    oa, Ua = castle_attention(qc, kc, vc, qu, ku, vu, 0.125, True)
    oa.backward(g)
    b = packed.clone().requires_grad_()
    ob, Ub = castle_attention_packed(b, 0.125, True)
    ob.backward(g)
    assert torch.equal(oa, ob) and torch.equal(Ua, Ub)
    # dkc, dvc, dqu are bit-reproducible; dqc, dvu, dku are summed with fp32 atomics
    assert torch.allclose(a.grad.float(), b.grad.float(), atol=1e-2, rtol=1e-2)
    for i in (0, 4, 5):  # qu, kc, vc slots
        assert torch.equal(a.grad[:, :, i], b.grad[:, :, i])
