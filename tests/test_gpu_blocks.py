"""GPU: tensor-core building blocks of the library (through the C ABI)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", range(11))
def test_selftest_mma(mode):
    from lookahead_keys_attention_b200 import _lib
    lib = _lib.load()
    torch.manual_seed(mode)
    x = torch.randn(128, 128, device="cuda").bfloat16()
    y = torch.randn(128, 128, device="cuda").bfloat16()
    d = torch.zeros(128, 128, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.castle_selftest_mma(mode, x.data_ptr(), y.data_ptr(), d.data_ptr(), st.data_ptr(), None)
    _lib.check(rc, "castle_selftest_mma")
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    xf, yf = x.float(), y.float()
    if mode >= 9:   # first operand read from tensor memory
        ref = xf @ yf.T if mode == 9 else xf @ yf
    else:
        op = mode - 5 if mode >= 5 else mode
        ref = [xf @ yf.T, xf @ yf, xf.T @ yf, xf.T @ yf.T, 1.0 - xf @ yf.T][op]
    err = (d - ref).abs().max().item()
    assert err < 1e-3, f"mode {mode}: max err {err}"


@pytest.mark.parametrize("form", range(4))
@pytest.mark.parametrize("n", [64, 128, 256])
def test_mma_rate_runs_and_is_sane(form, n):
    """The rate micro-benchmark finishes with a clean status and a plausible cost per instruction
    (a 128 x n x 16 product cannot beat n/2 cycles on this part, and 4x that would mean a broken loop)."""
    from lookahead_keys_attention_b200 import _lib
    lib = _lib.load()

    def measure(lib, form, n, reps, cyc, st):
        _lib.check(lib.castle_selftest_mma_rate(form, n, reps, cyc.data_ptr(), st.data_ptr(), None), "mma_rate")
        torch.cuda.synchronize()
        assert int(st.item()) == 0
        return cyc.cpu().tolist()
    cyc = torch.zeros(2, dtype=torch.int64, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    _, t1 = measure(lib, form, n, 32, cyc, st)
    _, t2 = measure(lib, form, n, 160, cyc, st)
    per = (t2 - t1) / 128
    assert 0.9 * n / 2 <= per <= 2 * n, per


def test_mma_rate_rejects_bad_arguments():
    from lookahead_keys_attention_b200 import _lib
    lib = _lib.load()
    cyc = torch.zeros(2, dtype=torch.int64, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.castle_selftest_mma_rate(4, 128, 8, cyc.data_ptr(), st.data_ptr(), None) < 0
    assert lib.castle_selftest_mma_rate(0, 96, 8, cyc.data_ptr(), st.data_ptr(), None) < 0
    assert lib.castle_selftest_mma_rate(0, 128, 0, cyc.data_ptr(), st.data_ptr(), None) < 0
    assert lib.castle_selftest_mma_rate(0, 128, 8, None, st.data_ptr(), None) < 0


def test_convert_16bit_saturates_and_scales():
    """bf16 -> fp16 saturates at the fp16 range instead of overflowing; both directions apply the device-resident factor."""
    from lookahead_keys_attention_b200 import _lib
    lib = _lib.load()
    x = torch.tensor([1.0, -2.5, 7e4, -3e38, 6e-5, 0.0, 123.0, -0.375] * 4, device="cuda").bfloat16()
    y = torch.empty_like(x, dtype=torch.float16)
    _lib.check(lib.castle_convert_16bit(_lib.BF16, x.data_ptr(), y.data_ptr(), x.numel(), None, None), "convert")
    assert torch.equal(y.float(), x.float().clamp(-65504.0, 65504.0).half().float())
    mul = torch.tensor([0.25], device="cuda")
    _lib.check(lib.castle_convert_16bit(_lib.BF16, x.data_ptr(), y.data_ptr(), x.numel(), mul.data_ptr(), None), "convert")
    assert torch.equal(y.float(), (x.float() * 0.25).clamp(-65504.0, 65504.0).half().float())
    h = torch.randn(64, device="cuda").half()
    b = torch.empty_like(h, dtype=torch.bfloat16)
    mul.fill_(8.0)
    _lib.check(lib.castle_convert_16bit(_lib.F16, h.data_ptr(), b.data_ptr(), h.numel(), mul.data_ptr(), None), "convert")
    torch.cuda.synchronize()
    assert torch.equal(b.float(), (h.float() * 8.0).bfloat16().float())
