"""GPU: `castle_decode_step_static`, the decode entry point for hosts that cannot allocate.

A serving engine that gave all device memory to its own arena, or a small host that binds only
the C ABI, has no scratch buffer to pass.  This entry point keeps the split partials in an array
inside the library instead.  The test drives it through the C ABI next to the ordinary
`castle_decode_step` on identical copies of the caches, for two tokens in a row, and expects the
same outputs and the same caches; it also checks that a problem larger than the built-in array is
refused with a message.  (Collected last on purpose: a failure here must not hide other results.)
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, L, name, prob, t, cap, news, bufs, out, ws=None):
    from lookahead_keys_attention_b200.ops import _desc, status_word
    descs = [_desc(x) for x in (*news, *bufs, out)]
    refs = [ctypes.byref(d) for d in descs]
    st = status_word(out.device).data_ptr()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    if name == "static":
        return lib.castle_decode_step_static(ctypes.byref(prob), t, cap, *refs, st, stream)
    return lib.castle_decode_step(ctypes.byref(prob), t, cap, *refs, ws.data_ptr(), ws.numel(), st, stream)


@pytest.mark.parametrize("B,H,d,t0,dtype", [(1, 2, 128, 5000, torch.bfloat16), (2, 3, 64, 700, torch.float32)])
def test_static_scratch_matches_workspace_entry_two_calls(B, H, d, t0, dtype):
    from lookahead_keys_attention_b200 import _lib as L, check_status
    lib = L.load()
    torch.manual_seed(d + t0)
    cap = t0 + 4
    prob = L.CastleProblem(B, H, 1, d, {torch.bfloat16: L.BF16, torch.float32: L.F32}[dtype], d ** -0.5)
    assert lib.castle_decode_workspace_bytes(ctypes.byref(prob), t0) > (2 + d) * 4 * B * H  # rows really are split
    base = [torch.randn(B, H, cap, d, device="cuda").to(dtype) * (0.5 if i == 0 else 1.0) for i in range(4)]
    bufs_a = [b.clone() for b in base]
    bufs_b = [b.clone() for b in base]
    ws = torch.empty(int(lib.castle_decode_workspace_bytes(ctypes.byref(prob), t0 + 1)), dtype=torch.uint8, device="cuda")
    atol = 1e-5 if dtype == torch.float32 else 2e-2
    from oracle import castle_oracle as O
    ocache = tuple(b[:, :, :t0].float().cpu() for b in base)   # the CPU oracle walks the same two tokens
    for step in range(2):
        news = [torch.randn(B, H, 1, d, device="cuda").to(dtype) for _ in range(6)]
        out_a = torch.empty(B, H, 1, d, device="cuda", dtype=dtype)
        out_b = torch.empty_like(out_a)
        assert _call(lib, L, "workspace", prob, t0 + step, cap, news, bufs_a, out_a, ws) == 0, L.last_error()
        assert _call(lib, L, "static", prob, t0 + step, cap, news, bufs_b, out_b) == 0, L.last_error()
        torch.cuda.synchronize()
        check_status()
        assert torch.allclose(out_a.float(), out_b.float(), atol=atol, rtol=1e-2), f"step {step}: outputs differ"
        # and directly against the oracle (fp32 arithmetic on the same rounded inputs)
        ref, ocache = O.castle_decode_step(*[x.float().cpu() for x in news], ocache, d ** -0.5)
        otol = 1e-4 if dtype == torch.float32 else 2e-2
        err = (out_b.float().cpu() - ref).abs()
        assert bool((err <= otol + 1e-2 * ref.abs()).all()), f"step {step}: static entry vs oracle {err.max().item():.3e}"
        if dtype != torch.float32:   # the kernel keeps U in the cache dtype: re-round the oracle's copy as it does
            ocache = (ocache[0].to(dtype).float(), *ocache[1:])
        n = t0 + step + 1
        for a, b, nm in zip(bufs_a, bufs_b, ("U", "qu_cache", "kc_cache", "vc_cache")):
            assert torch.allclose(a[:, :, :n].float(), b[:, :, :n].float(), atol=atol, rtol=1e-2), f"step {step}: {nm}"


def test_static_scratch_refuses_oversize_problem():
    from lookahead_keys_attention_b200 import _lib as L
    lib = L.load()
    B, H, d, t0 = 65, 8, 16, 600  # 520 (batch, head) pairs x 2 row-splits = 1040 partials > 1024
    prob = L.CastleProblem(B, H, 1, d, L.BF16, 0.25)
    z = lambda n: torch.zeros(B, H, n, d, device="cuda", dtype=torch.bfloat16)
    news, bufs, out = [z(1) for _ in range(6)], [z(t0 + 2) for _ in range(4)], z(1)
    rc = _call(lib, L, "static", prob, t0, t0 + 2, news, bufs, out)
    assert rc < 0 and "1024" in L.last_error() and "castle_decode_step" in L.last_error()
