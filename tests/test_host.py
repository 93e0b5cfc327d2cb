"""CPU: host-side logic - the library's exports, argument checks that need no GPU,
the (batch, head) partition, and the module's cache bookkeeping."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def _lib():
    from lookahead_keys_attention_b200 import _lib
    _lib.build()
    return _lib


def test_library_exports_every_declared_symbol():
    L = _lib()
    lib = L.load()
    names = set()
    for header in sorted((ROOT / "include").glob("*.h")):
        code = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)  # declarations only, not the comments
        found = set(re.findall(r"\b(castle_[a-z0-9_]+)\s*\(", code))
        for n in found:
            assert hasattr(lib, n), f"{n} declared in include/{header.name} but not exported"
        names |= found
    assert {"castle_fwd", "castle_bwd", "castle_decode_step", "castle_abi_version",
            "castle_selftest_wait_timeout"} <= names
    assert lib.castle_abi_version() == 1


def test_argument_rejection_without_gpu():
    L = _lib()
    lib = L.load()
    prob = L.CastleProblem(1, 1, 128, 48, L.BF16, 0.125)
    t = L.CastleTensor(16, 0, 0, 64)
    args = [ctypes.byref(t)] * 7
    rc = lib.castle_fwd(ctypes.byref(prob), *args, None, None, 0, None, None, 0, None, None)
    assert rc < 0 and "dim_head" in L.last_error()
    prob = L.CastleProblem(1, 1, 128, 64, L.F32, 0.125)
    rc = lib.castle_fwd(ctypes.byref(prob), *args, None, None, 0, None, None, 0, None, None)
    assert rc < 0 and "dtype" in L.last_error()
    prob = L.CastleProblem(1, 1, 1, 64, L.BF16, 0.125)
    rc = lib.castle_decode_step(ctypes.byref(prob), 4, 4, *([ctypes.byref(t)] * 11), None, 0, None, None)
    assert rc < 0 and "capacity" in L.last_error()
    t_bad = L.CastleTensor(8, 0, 0, 64)
    prob = L.CastleProblem(1, 1, 128, 64, L.BF16, 0.125)
    rc = lib.castle_fwd(ctypes.byref(prob), ctypes.byref(t_bad), *args[1:], None, None, 0, None, None, 0, None, None)
    assert rc < 0 and "aligned" in L.last_error()
    assert lib.castle_fwd_workspace_bytes(ctypes.byref(prob)) == 128 * (8 + 64 * 2)
    assert lib.castle_bwd_workspace_bytes(ctypes.byref(prob)) == 128 * (3 * 64 + 1) * 4


def test_backward_workspace_at_dim_head_128():
    """Accumulators (rounded up to 1 KB) plus the tile hand-over scratch: 96 KB per (query block, key block) step
    and (batch, head) pair, for as many pairs as stay under 8 GiB; a workspace below one pair's worth is refused
    with the least size in the message."""
    L = _lib()
    lib = L.load()
    def acc(B, H, N):
        return (B * H * N * (3 * 128 + 1) * 4 + 1023) // 1024 * 1024
    def pair(N):
        nblk = (N + 127) // 128
        return nblk * (nblk + 1) // 2 * 3 * 32768
    for B, H, N in [(1, 1, 1), (1, 5, 640), (2, 3, 1333), (1, 8, 8192)]:
        prob = L.CastleProblem(B, H, N, 128, L.BF16, 128 ** -0.5)
        assert lib.castle_bwd_workspace_bytes(ctypes.byref(prob)) == acc(B, H, N) + B * H * pair(N)
    # config 4's slice: 792 MB per pair, so 10 of the 32 pairs per chunk
    prob = L.CastleProblem(1, 32, 16384, 128, L.BF16, 128 ** -0.5)
    assert pair(16384) == 8256 * 98304
    assert lib.castle_bwd_workspace_bytes(ctypes.byref(prob)) == acc(1, 32, 16384) + 10 * pair(16384)
    # beyond 8 GiB for a single pair: one pair per chunk
    prob = L.CastleProblem(1, 4, 65536, 128, L.BF16, 128 ** -0.5)
    assert lib.castle_bwd_workspace_bytes(ctypes.byref(prob)) == acc(1, 4, 65536) + pair(65536)
    # refusal (host-side check, before anything touches the device)
    prob = L.CastleProblem(1, 5, 640, 128, L.BF16, 128 ** -0.5)
    t = L.CastleTensor(16, 5 * 640 * 128, 640 * 128, 128)
    r = ctypes.byref(t)
    least = acc(1, 5, 640) + pair(640)
    rc = lib.castle_bwd(ctypes.byref(prob), *([r] * 8), 16, 16, *([r] * 6), 1024, least - 1, 16, None)
    assert rc < 0 and "workspace too small" in L.last_error() and str(least) in L.last_error()


def test_new_entry_points_reject_bad_arguments_without_gpu():
    L = _lib()
    lib = L.load()
    prob = L.CastleProblem(1, 1, 128, 64, L.BF16, 0.125)
    t = L.CastleTensor(16, 0, 0, 64)
    r = ctypes.byref(t)
    # prefill: the four caches are mandatory
    rc = lib.castle_fwd_prefill(ctypes.byref(prob), *([r] * 7), None, None, r, r, r, None, None, 0, None, None)
    assert rc < 0 and "cache" in L.last_error()
    # conversion: only 16-bit sources, counts in multiples of 8, aligned pointers
    assert lib.castle_convert_16bit(L.F32, 16, 32, 64, None, None) < 0 and "bf16 or fp16" in L.last_error()
    assert lib.castle_convert_16bit(L.BF16, 16, 32, 12, None, None) < 0 and "multiple of 8" in L.last_error()
    assert lib.castle_convert_16bit(L.BF16, 8, 32, 64, None, None) < 0
    assert lib.castle_convert_16bit(L.BF16, None, 32, 64, None, None) < 0


def test_ops_refuse_cpu_tensors():
    from lookahead_keys_attention_b200 import castle_attention
    z = torch.zeros(1, 1, 8, 64)
    with pytest.raises(RuntimeError, match="no CPU path"):
        castle_attention(z, z, z, z, z, z, 0.125)


def test_partition_covers_grid_once():
    from lookahead_keys_attention_b200.sharding import partition
    for batch, heads in [(4, 16), (8, 32), (64, 16)]:
        for world in (1, 2, 4, 8):
            seen = torch.zeros(batch, heads, dtype=torch.int32)
            sizes = set()
            for r in range(world):
                s = partition(batch, heads, world, r)
                seen[s.b0:s.b1, s.h0:s.h1] += 1
                sizes.add(s.pairs)
            assert bool((seen == 1).all()) and len(sizes) == 1
    with pytest.raises(ValueError):
        partition(3, 5, 2, 0)


def test_cache_ownership_is_explicit():
    """Only caches the module made (or was handed through cache_from_buffers) are updated in place;
    tensors of the caller are copied, never written; a stale cache is refused."""
    from lookahead_keys_attention_b200 import Cache, Castle, ModuleCache, cache_from_buffers
    m = Castle(32, heads=3, dim_head=8, cache_headroom=4)
    like = torch.zeros(2, 3, 1, 8)
    # (1) a prefix slice of a caller tensor looks like a buffer with spare rows - it must be copied
    big = [torch.arange(2 * 3 * 10 * 8, dtype=torch.float32).view(2, 3, 10, 8) + i for i in range(4)]
    keep = [b.clone() for b in big]
    foreign = Cache(*(b[:, :, :4] for b in big))
    st = m._buffers_for_step(foreign, 4, like)
    assert all(buf.data_ptr() != b.data_ptr() for buf, b in zip(st.bufs, big))
    assert all(torch.equal(buf[:, :, :4], b[:, :, :4]) for buf, b in zip(st.bufs, big))
    for buf in st.bufs:
        buf.fill_(-1.0)                      # whatever the step writes ...
    assert all(torch.equal(b, k) for b, k in zip(big, keep))   # ... the caller's memory is untouched
    # (2) a cache of the module: in place while it is the latest one
    own = ModuleCache(st, 4)
    assert isinstance(own, Cache) and own.U.shape == (2, 3, 4, 8) and own.is_current()
    st.length = 4
    assert m._buffers_for_step(own, 4, like) is st
    st.length = 5                            # a later step advanced the buffers
    newer = ModuleCache(st, 5)
    assert not own.is_current() and newer.is_current()
    with pytest.raises(RuntimeError, match="advanced in place"):
        m._buffers_for_step(own, 4, like)
    # (3) functional semantics on request: every step gets fresh buffers, old caches stay valid
    mf = Castle(32, heads=3, dim_head=8, inplace_cache=False)
    st2 = mf._buffers_for_step(newer, 5, like)
    assert st2 is not st and st2.length == 5 and torch.equal(st2.bufs[1][:, :, :5], st.bufs[1][:, :, :5])
    # (4) a full buffer grows by copy
    full = cache_from_buffers(*[torch.zeros(2, 3, 6, 8) for _ in range(4)], length=6)
    st3 = m._buffers_for_step(full, 6, like)
    assert st3 is not full._state and st3.capacity >= 7
    # (5) explicit hand-over of caller buffers: used as they are
    mine = [torch.zeros(2, 3, 9, 8) for _ in range(4)]
    c = cache_from_buffers(*mine, length=3)
    assert c.kc_cache.shape == (2, 3, 3, 8) and m._buffers_for_step(c, 3, like).bufs[2] is mine[2]
    with pytest.raises(ValueError):
        cache_from_buffers(*mine, length=10)


def test_forward_chunks_bound_the_scratch():
    from lookahead_keys_attention_b200.ops import forward_chunks
    for B, H, per, limit in [(4, 16, 10, 1000), (4, 16, 10, 100), (8, 32, 7, 50), (1, 32, 9, 9), (3, 5, 4, 9)]:
        seen = torch.zeros(B, H, dtype=torch.int32)
        for b0, b1, h0, h1 in forward_chunks(B, H, per, limit):
            assert (b1 - b0) * (h1 - h0) * per <= limit
            assert b1 - b0 == 1 or (h0, h1) == (0, H)     # several batch rows only with all heads
            seen[b0:b1, h0:h1] += 1
        assert bool((seen == 1).all())
    with pytest.raises(RuntimeError, match="more than"):
        forward_chunks(1, 1, 11, 10)


def test_module_signature_and_state_dict():
    from lookahead_keys_attention_b200 import Cache, Castle
    m = Castle(32, heads=2, dim_head=16, prenorm=True)
    assert set(m.state_dict()) == {"norm.weight", "to_all_qkv.weight", "combine_heads.weight"}
    assert m.to_all_qkv.weight.shape == (6 * 32, 32) and m.combine_heads.weight.shape == (32, 32)
    assert (m.dim, m.heads, m.dim_head, m.scale) == (32, 2, 16, 0.25)
    assert Cache._fields == ("U", "qu_cache", "kc_cache", "vc_cache")
    with pytest.raises(AssertionError):
        m(torch.zeros(1, 4, 32), cache=Cache(*([torch.zeros(1, 2, 3, 16)] * 4)))


def test_rotary_offset_and_norm():
    """This package's own rotary embedding: a rotation (norm preserving) whose `offset` shifts positions,
    which is what makes a cached single-token step agree with the parallel pass."""
    from lookahead_keys_attention_b200.castle import _Rotary
    torch.manual_seed(0)
    r = _Rotary(16)
    t = torch.randn(2, 3, 10, 16)
    full = r.rotate(t)
    assert torch.allclose(full.norm(dim=-1), t.norm(dim=-1), atol=1e-5)
    assert torch.allclose(r.rotate(t[:, :, 4:7], offset=4), full[:, :, 4:7], atol=1e-6)
    assert torch.allclose(r.rotate(t[:, :, :1]), t[:, :, :1], atol=1e-6)  # position 0 is the identity
