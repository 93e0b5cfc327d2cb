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


def test_forward_fp32_caller_atol_1e3():
    """fp32 caller (the README shape's head geometry): atol 1e-3 against the fp32 oracle."""
    from lookahead_keys_attention_b200 import castle_attention
    packed = _inputs(2, 8, 128, 64, torch.float32, seed=7) * 0.5
    qu, ku, vu, qc, kc, vc = _views(packed.cuda())
    out = castle_attention(qc, kc, vc, qu, ku, vu, 0.125, False)
    assert out.dtype == torch.float32
    rqu, rku, rvu, rqc, rkc, rvc = _views(packed)
    ro = O.castle_parallel(rqc, rkc, rvc, rqu, rku, rvu, 0.125)
    _close(out.cpu(), ro, 1e-3, 0.0, "out")


def test_forward_causality():
    from lookahead_keys_attention_b200 import castle_attention
    packed = _inputs(1, 2, 300, 64, torch.bfloat16, seed=3).cuda()
    qu, ku, vu, qc, kc, vc = _views(packed)
    full = castle_attention(qc, kc, vc, qu, ku, vu, 0.125, False)
    half = castle_attention(*[t[:, :, :150] for t in (qc, kc, vc, qu, ku, vu)], 0.125, False)
    _close(full[:, :, :150].float(), half.float(), 1e-3, 0.0, "prefix invariance")
