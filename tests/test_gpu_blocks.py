"""GPU: tensor-core building blocks of the library (through the C ABI)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", range(9))
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
    op = mode - 5 if mode >= 5 else mode
    ref = [xf @ yf.T, xf @ yf, xf.T @ yf, xf.T @ yf.T, 1.0 - xf @ yf.T][op]
    err = (d - ref).abs().max().item()
    assert err < 1e-3, f"mode {mode}: max err {err}"
