"""GPU: no entry point writes outside the rows it owns.  Every output buffer of the forward, the
backward and the decode step is over-allocated, pre-filled with a sentinel, and the guard rows are
checked after the call (ragged N, so the last 128-row tile is mostly out of range)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

SENT = 123.0


def _guarded(shape, dtype, guard_rows, dim):
    """Tensor of `shape` with `guard_rows` extra sentinel rows after it along `dim`; returns (view, full)."""
    full_shape = list(shape)
    full_shape[dim] += guard_rows
    full = torch.full(full_shape, SENT, dtype=dtype, device="cuda")
    return full.narrow(dim, 0, shape[dim]), full


def _guard_ok(full, n, dim):
    g = full.narrow(dim, n, full.shape[dim] - n).float()
    return bool((g == SENT).all())


@pytest.mark.parametrize("N,d", [(130, 64), (200, 128), (1, 64)])
def test_forward_backward_stay_inside_their_rows(N, d):
    from lookahead_keys_attention_b200 import _lib as L, check_status
    from lookahead_keys_attention_b200.ops import _desc, status_word
    lib = L.load()
    B, H = 2, 2
    torch.manual_seed(N)
    packed = (torch.randn(B, N, 6, H, d, device="cuda") * 0.5).bfloat16()
    qu, ku, vu, qc, kc, vc = (packed[:, :, i].permute(0, 2, 1, 3) for i in range(6))
    G = 130  # guard rows: more than one tile
    out, out_f = _guarded((B, H, N, d), torch.bfloat16, G, 2)
    U, U_f = _guarded((B, H, N, d), torch.bfloat16, G, 2)
    lse_f = torch.full((B * H * N + G,), SENT, device="cuda")
    wst_f = torch.full((B * H * N * d + G * d,), SENT, device="cuda")
    prob = L.CastleProblem(B, H, N, d, L.BF16, d ** -0.5)
    ws = torch.empty(int(lib.castle_fwd_workspace_bytes(ctypes.byref(prob))) + 16, dtype=torch.uint8, device="cuda")
    st = status_word("cuda")
    ins = [_desc(t) for t in (qc, kc, vc, qu, ku, vu)]
    do_, du_ = _desc(out), _desc(U)
    rc = lib.castle_fwd(ctypes.byref(prob), *[ctypes.byref(x) for x in ins], ctypes.byref(do_), lse_f.data_ptr(),
                        ctypes.byref(du_), L.BF16, wst_f.data_ptr(), ws.data_ptr(), ws.numel(), st.data_ptr(), None)
    L.check(rc, "castle_fwd")
    torch.cuda.synchronize()
    check_status()
    assert _guard_ok(out_f, N, 2) and _guard_ok(U_f, N, 2)
    assert bool((lse_f[B * H * N:] == SENT).all()) and bool((wst_f[B * H * N * d:] == SENT).all())
    assert bool(torch.isfinite(out.float()).all())

    # backward: six gradient tensors with guard rows
    dout = (torch.randn(B, H, N, d, device="cuda")).bfloat16()
    grads, fulls = zip(*[_guarded((B, H, N, d), torch.bfloat16, G, 2) for _ in range(6)])
    need = int(lib.castle_bwd_workspace_bytes(ctypes.byref(prob)))
    wsb_f = torch.full((need // 4 + 64,), SENT, device="cuda")
    a = [_desc(t) for t in (qc, kc, vc, qu, ku, vu, out, dout)]
    g = [_desc(t) for t in grads]
    rc = lib.castle_bwd(ctypes.byref(prob), *[ctypes.byref(x) for x in a], lse_f.data_ptr(), wst_f.data_ptr(),
                        *[ctypes.byref(x) for x in g], wsb_f.data_ptr(), need, st.data_ptr(), None)
    L.check(rc, "castle_bwd")
    torch.cuda.synchronize()
    check_status()
    for f in fulls:
        assert _guard_ok(f, N, 2)
    assert bool((wsb_f[need // 4:] == SENT).all())   # nothing written past the stated workspace size
    for t in grads:
        assert bool(torch.isfinite(t.float()).all())


def test_decode_stays_inside_capacity():
    from lookahead_keys_attention_b200 import castle_decode_step, check_status
    B, H, d, t0, cap = 2, 3, 128, 700, 702
    bufs, fulls = zip(*[_guarded((B, H, cap, d), torch.bfloat16, 4, 2) for _ in range(4)])
    for b in bufs:
        b[:, :, :t0] = torch.randn(B, H, t0, d, device="cuda").bfloat16()
    # the guarded views are not adjacent-row buffers of stride d*cap..., so this exercises the strided kernel too
    news = [torch.randn(B, H, 1, d, device="cuda").bfloat16() for _ in range(6)]
    castle_decode_step(*news, *bufs, t0, d ** -0.5)
    torch.cuda.synchronize()
    check_status()
    for f in fulls:
        assert _guard_ok(f, cap, 2)
    for b in bufs[1:]:
        assert bool((b[:, :, t0 + 1:].float() == SENT).all())   # rows after the appended one are untouched
