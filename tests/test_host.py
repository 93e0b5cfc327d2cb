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
    header = (ROOT / "include" / "castle_b200.h").read_text()
    code = re.sub(r"/\*.*?\*/", "", header, flags=re.S)  # declarations only, not the comments
    names = set(re.findall(r"\b(castle_[a-z0-9_]+)\s*\(", code))
    assert {"castle_fwd", "castle_bwd", "castle_decode_step", "castle_abi_version"} <= names
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/castle_b200.h but not exported"
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


def test_capacity_view_roundtrip():
    from lookahead_keys_attention_b200.castle import _capacity_view
    for B, H in [(2, 3), (1, 3), (2, 1), (1, 1)]:
        buf = torch.arange(B * H * 10 * 8, dtype=torch.float32).view(B, H, 10, 8)
        v = _capacity_view(buf[:, :, :4])
        assert v is not None and v.shape == (B, H, 10, 8) and v.data_ptr() == buf.data_ptr()
        assert torch.equal(v, buf)
    assert _capacity_view(torch.zeros(2, 3, 4, 8)) is None           # no spare rows
    assert _capacity_view(torch.zeros(2, 3, 0, 8)) is None           # empty cache
    assert _capacity_view(torch.zeros(2, 4, 3, 8).transpose(1, 2)) is None


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
