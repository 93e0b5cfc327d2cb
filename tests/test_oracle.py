"""The CPU oracle against the golden vectors recorded from the real reference
(tests/golden/make_golden.py), plus the reference's own self-consistency
properties (tests/test_lookahead.py:10-64 and :145-182 in the reference)."""
import pytest
import torch

from conftest import load_golden, rebuild_core_case, rebuild_module_case
from oracle import castle_oracle as O

MODULE_CASES = ["module_d16", "module_d16_prenorm", "module_d32", "module_d64_n256", "module_readme"]
CORE_CASES = ["core_n40_d16", "core_n200_d64", "core_n130_d128"]


def _module_fwd(cfg, w1, w2, nw, x, **kw):
    return O.castle_module_forward(x, w1, w2, cfg["heads"], cfg["dim_head"], norm_weight=nw, **kw)


@pytest.mark.parametrize("name", MODULE_CASES)
def test_oracle_module_matches_reference(name):
    g = load_golden(name)
    cfg, w1, w2, nw, x, gout = rebuild_module_case(g)
    st = cfg["stride"]
    w1r, w2r, xr = w1.clone().requires_grad_(), w2.clone().requires_grad_(), x.clone().requires_grad_()
    out = _module_fwd(cfg, w1r, w2r, nw, xr)
    out.backward(gout)
    assert torch.allclose(out.detach()[:, ::st], torch.from_numpy(g["out"]), atol=1e-6)
    assert torch.allclose(xr.grad[:, ::st], torch.from_numpy(g["dx"]), atol=1e-5)
    assert torch.allclose(w1r.grad[::37, ::11], torch.from_numpy(g["dw_qkv_sample"]), atol=1e-4, rtol=1e-4)
    assert torch.allclose(w2r.grad[::11, ::13], torch.from_numpy(g["dw_out_sample"]), atol=1e-4, rtol=1e-4)
    assert abs(w1r.grad.abs().sum().item() - float(g["dw_qkv_sum_abs"])) <= 1e-4 * float(g["dw_qkv_sum_abs"])


@pytest.mark.parametrize("name", MODULE_CASES)
def test_oracle_sequential_matches_reference(name):
    g = load_golden(name)
    cfg, w1, w2, nw, x, _ = rebuild_module_case(g)
    st, split, n = cfg["stride"], cfg["split"], cfg["n"]
    with torch.no_grad():
        pre, cache = _module_fwd(cfg, w1, w2, nw, x[:, :split], return_next_cache=True)
        assert torch.allclose(cache.U, torch.from_numpy(g["prefill_U"]), atol=1e-5)
        outs = [pre]
        for t in range(split, n):
            o, cache = _module_fwd(cfg, w1, w2, nw, x[:, t:t + 1], cache=cache)
            outs.append(o)
        seq = torch.cat(outs, dim=1)
        assert torch.allclose(seq[:, ::st], torch.from_numpy(g["seq_out"]), atol=1e-6)
        assert torch.allclose(cache.U[:, :, ::st], torch.from_numpy(g["final_U"]), atol=1e-5)
        assert torch.allclose(cache.qu_cache[:, :, ::st], torch.from_numpy(g["final_qu"]), atol=1e-6)
        # reference property: sequential == parallel
        assert torch.allclose(seq, _module_fwd(cfg, w1, w2, nw, x), atol=1e-5)


def _unpack(packed, h, d):
    return [t.contiguous() for t in O.split_heads(packed, h)]  # qu,ku,vu,qc,kc,vc


@pytest.mark.parametrize("name", CORE_CASES)
def test_oracle_core_matches_reference(name):
    g = load_golden(name)
    (b, h, n, d), packed, gout = rebuild_core_case(g)
    qu, ku, vu, qc, kc, vc = _unpack(packed, h, d)
    scale = d ** -0.5
    out, U = O.castle_parallel(qc, kc, vc, qu, ku, vu, scale, return_U=True)
    merged = out.permute(0, 2, 1, 3).reshape(b, n, h * d)
    assert torch.allclose(merged.float(), torch.from_numpy(g["out"]), atol=1e-6)
    assert torch.allclose(U.float(), torch.from_numpy(g["U"]), atol=2e-6, rtol=1e-6)
    do = gout.view(b, n, h, d).permute(0, 2, 1, 3)
    dqc, dkc, dvc, dqu, dku, dvu = O.castle_parallel_bwd(qc, kc, vc, qu, ku, vu, scale, do)
    dp = torch.stack([dqu, dku, dvu, dqc, dkc, dvc], 0).permute(1, 3, 0, 2, 4).reshape(b, n, 6 * h * d)
    assert torch.allclose(dp.float(), torch.from_numpy(g["dpacked"]), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("name", CORE_CASES)
@pytest.mark.parametrize("block", [16, 128])
def test_blockwise_recurrence_matches_dense(name, block):
    """The O(N^2 d) key-stationary recurrence the kernels evaluate, fwd and bwd."""
    g = load_golden(name)
    (b, h, n, d), packed, gout = rebuild_core_case(g)
    qu, ku, vu, qc, kc, vc = [t[0, 0] for t in _unpack(packed, h, d)]
    scale = d ** -0.5
    do = gout.view(b, n, h, d)[0, :, 0]
    out, U, lse = O.castle_parallel(qc, kc, vc, qu, ku, vu, scale, return_U=True, return_lse=True)
    ob, Ub, lb = O.castle_parallel_blockwise(qc, kc, vc, qu, ku, vu, scale, block=block)
    assert torch.allclose(ob, out, atol=1e-12) and torch.allclose(Ub, U, atol=1e-12)
    assert torch.allclose(lb.float(), lse, atol=1e-5)
    gd = O.castle_parallel_bwd(qc, kc, vc, qu, ku, vu, scale, do)
    gb = O.castle_parallel_bwd_blockwise(qc, kc, vc, qu, ku, vu, scale, out, lb, U, do, block=block)
    for a, b_ in zip(gb, gd):
        assert torch.allclose(a, b_, atol=1e-10)


def test_oracle_causality():
    """Prefix invariance (reference tests/test_lookahead.py:145-182)."""
    torch.manual_seed(0)
    w1 = torch.randn(6 * 64, 64) * 0.1
    w2 = torch.randn(64, 64) * 0.1
    x = torch.randn(2, 32, 64)
    full = O.castle_module_forward(x, w1, w2, 2, 32)
    half = O.castle_module_forward(x[:, :16], w1, w2, 2, 32)
    assert torch.allclose(full[:, :16], half, atol=1e-6)


def test_oracle_single_token_without_cache_and_assert():
    torch.manual_seed(0)
    w1 = torch.randn(6 * 32, 32) * 0.1
    w2 = torch.randn(32, 32) * 0.1
    x = torch.randn(2, 4, 32)
    out, cache = O.castle_module_forward(x[:, :1], w1, w2, 2, 16)
    assert cache.U.shape == (2, 2, 1, 16) and float(cache.U.abs().max()) == 0.0
    with pytest.raises(AssertionError):
        O.castle_module_forward(x, w1, w2, 2, 16, cache=cache)
