"""`Castle` - drop-in for the reference module of the same name
(lookahead_keys_attention/lookahead_keys_attention.py:41-214): same constructor
arguments, state-dict keys (`to_all_qkv.weight`, `combine_heads.weight`,
`norm.weight`), `forward(x, cache=None, return_next_cache=None)` conventions
and `Cache` tuple.  The attention cores run as sm_100a kernels through the
C-ABI library; the two projections and the optional RMSNorm stay torch ops.

Difference from the reference, by design: the decode step appends to
pre-allocated cache buffers and rewrites the lookahead keys `U` IN PLACE
instead of concatenating new tensors every token (:185-203), so a cache
returned by step t shares memory with the cache returned by step t-1, and
only the LATEST cache of a chain may be decoded from (an older one raises).
Pass `inplace_cache=False` to get the reference's functional behaviour (each
step then copies the caches first, and any cache can be decoded from again).
Only caches this module returned (or took over through `cache_from_buffers`)
are ever written; a cache made of the caller's own tensors is copied first.
"""
from __future__ import annotations

from collections import namedtuple

import torch
from torch import nn

from .ops import castle_attention, castle_attention_packed, castle_decode_step, prefill_writes_caches

Cache = namedtuple("Cache", ("U", "qu_cache", "kc_cache", "vc_cache"))


class _CacheBuffers:
    """Four (B, H, capacity, d) buffers the module allocated, and how many of their rows are valid
    NOW.  Decode steps append to them and rewrite U in place, so only the cache returned by the
    latest step still describes their contents."""

    __slots__ = ("bufs", "length")

    def __init__(self, bufs, length):
        self.bufs, self.length = list(bufs), int(length)

    @property
    def capacity(self):
        return self.bufs[0].shape[2]

    def views(self, n):
        return [b[:, :, :n] for b in self.bufs]


class ModuleCache(Cache):
    """The `Cache` tuple as this module returns it: the same four fields, each a `[:, :, :t]` view,
    plus a record of the capacity buffers behind them.  Ownership is explicit: the in-place decode
    path is taken only for a `ModuleCache` that is the latest one of its buffers.  Any other cache
    (a plain tuple of the caller's tensors, slices, a re-wrapped copy) is treated as read-only
    input and copied into fresh buffers first, so the caller's memory is never written."""

    def __new__(cls, state: _CacheBuffers, length: int):
        self = super().__new__(cls, *state.views(length))
        self._state, self._length = state, int(length)
        return self

    def is_current(self) -> bool:
        return self._state.length == self._length


def cache_from_buffers(U, qu_cache, kc_cache, vc_cache, length: int) -> ModuleCache:
    """Hand four caller-allocated (B, H, capacity, d) buffers with `length` valid rows over to the
    module: from now on decode steps append to them and rewrite U IN PLACE (no copy is made)."""
    bufs = [U, qu_cache, kc_cache, vc_cache]
    shape = tuple(U.shape)
    for b in bufs:
        if b.dim() != 4 or tuple(b.shape) != shape or b.dtype != U.dtype or not b.is_contiguous():
            raise ValueError("cache_from_buffers: four contiguous (B, H, capacity, d) buffers of one dtype expected")
    if not 0 <= length <= shape[2]:
        raise ValueError("cache_from_buffers: length out of range")
    return ModuleCache(_CacheBuffers(bufs, length), length)


class _Rotary(nn.Module):
    """This package's own rotary embedding (pairs of adjacent channels rotated by
    position * theta^(-2i/d)).  The reference delegates to the third-party
    `rotary_embedding_torch` package, which is not available to compare against;
    numerical agreement with that package is not claimed."""

    def __init__(self, dim, theta=10000.0):
        super().__init__()
        self.register_buffer("freqs", theta ** (-torch.arange(0, dim, 2).float() / dim), persistent=False)

    def rotate(self, t, offset=0):
        n = t.shape[-2]
        ang = (torch.arange(n, device=t.device, dtype=torch.float32) + offset)[:, None] * self.freqs.to(t.device)
        cos, sin = ang.cos().to(t.dtype), ang.sin().to(t.dtype)
        a, b = t[..., 0::2], t[..., 1::2]
        return torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1).flatten(-2)


class Castle(nn.Module):
    def __init__(self, dim, heads=8, dim_head=64, use_triton=None, rotary_emb=False, prenorm=False,
                 inplace_cache=True, cache_headroom=256):
        super().__init__()
        dim_inner = dim_head * heads
        self.dim, self.dim_head, self.heads = dim, dim_head, heads
        # Attribute kept for callers that read it; the value follows the reference's default rule
        # (lookahead_keys_attention.py:58, "CUDA available and the kernel backend importable") with this
        # package's kernels in the place of Triton.  It selects nothing: there is one code path.
        self.use_triton = bool(use_triton) if use_triton is not None else torch.cuda.is_available()
        self.scale = dim_head ** -0.5
        self.norm = nn.RMSNorm(dim) if prenorm else nn.Identity()
        self.rotary_emb = _Rotary(dim_head) if rotary_emb else None
        self.to_all_qkv = nn.Linear(dim, dim_inner * 6, bias=False)
        self.combine_heads = nn.Linear(dim_inner, dim, bias=False)
        self.inplace_cache = inplace_cache
        self.cache_headroom = cache_headroom

    def _split(self, qkvs):
        b, n, _ = qkvs.shape
        # 'b n (qkv h d) -> qkv b h n d', order qu, ku, vu, qc, kc, vc (reference :77,104); views, no copies
        return qkvs.view(b, n, 6, self.heads, self.dim_head).permute(2, 0, 3, 1, 4).unbind(0)

    def _new_buffers(self, b, h, d, rows, dtype, device) -> _CacheBuffers:
        cap = rows + max(self.cache_headroom, rows // 4)
        return _CacheBuffers([torch.empty(b, h, cap, d, dtype=dtype, device=device) for _ in range(4)], 0)

    def _buffers_for_step(self, cache, t, like) -> _CacheBuffers:
        """Capacity buffers holding rows [0, t) of `cache` with room for row t."""
        b, h, _, d = like.shape
        state = getattr(cache, "_state", None) if isinstance(cache, ModuleCache) else None
        if state is not None and cache._length == t:
            if not cache.is_current() and self.inplace_cache:
                raise RuntimeError(
                    "this cache was advanced in place by a later decode step and no longer holds its rows; "
                    "construct Castle(..., inplace_cache=False) to decode from one cache more than once")
            if self.inplace_cache and t < state.capacity:
                return state
        # a foreign cache, a full buffer, or functional semantics asked for: copy into fresh buffers
        fresh = self._new_buffers(b, h, d, t + 1, like.dtype, like.device)
        if t > 0:
            for buf, src in zip(fresh.bufs, cache):
                buf[:, :, :t].copy_(src)
        fresh.length = t
        return fresh

    def forward(self, x, cache: Cache | None = None, return_next_cache=None):
        seq_len = x.shape[1]
        is_inference = seq_len == 1
        if return_next_cache is None:
            return_next_cache = is_inference
        x = self.norm(x)
        qkvs = self.to_all_qkv(x)
        qu, ku, vu, qc, kc, vc = self._split(qkvs)
        if self.rotary_emb is not None:
            offset = cache.kc_cache.shape[-2] if cache is not None else 0
            qc, kc, qu, ku, vu = (self.rotary_emb.rotate(t, offset) for t in (qc, kc, qu, ku, vu))

        if not is_inference:
            assert cache is None, "must be inferencing single tokens if receiving cache"
            packed = None
            if self.rotary_emb is None:  # the kernels read the projection output in place
                packed = qkvs.view(x.shape[0], seq_len, 6, self.heads, self.dim_head)
            if return_next_cache:
                # the cache lives in buffers with spare rows so that decode steps can append in place
                b, h, _, d = qu.shape
                state = self._new_buffers(b, h, d, seq_len, qu.dtype, qu.device)
                # 16-bit modules: the forward kernels write all four caches themselves (U from the final
                # lookahead state, qu/kc/vc from the tiles they hold in shared memory)
                fill = prefill_writes_caches(qu.dtype, d, seq_len)
                cache_out = tuple(state.views(seq_len)) if fill else None
                if packed is not None:
                    out, U = castle_attention_packed(packed, self.scale, True, cache_out)
                else:
                    out, U = castle_attention(qc, kc, vc, qu, ku, vu, self.scale, True, cache_out)
                if not fill:   # fp32 modules (the kernels run on fp16 copies) and odd head widths
                    with torch.no_grad():
                        for buf, src in zip(state.bufs, (U, qu, kc, vc)):
                            buf[:, :, :seq_len].copy_(src)
                state.length = seq_len
                next_cache = ModuleCache(state, seq_len)
            elif packed is not None:
                out = castle_attention_packed(packed, self.scale, False)
            else:
                out = castle_attention(qc, kc, vc, qu, ku, vu, self.scale, False)
        else:
            t = 0 if cache is None else cache[0].shape[-2]
            with torch.no_grad():
                state = self._buffers_for_step(cache, t, qu)
                out = castle_decode_step(qc, kc, vc, qu, ku, vu, *state.bufs, t, self.scale)
            state.length = t + 1
            next_cache = ModuleCache(state, t + 1)

        b, h, n, d = out.shape
        out = out.permute(0, 2, 1, 3).reshape(b, n, h * d)  # 'b h n d -> b n (h d)'
        out = self.combine_heads(out)
        if not return_next_cache:
            return out
        return out, next_cache
