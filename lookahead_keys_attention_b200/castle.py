"""`Castle` - drop-in for the reference module of the same name
(lookahead_keys_attention/lookahead_keys_attention.py:41-214): same constructor
arguments, state-dict keys (`to_all_qkv.weight`, `combine_heads.weight`,
`norm.weight`), `forward(x, cache=None, return_next_cache=None)` conventions
and `Cache` tuple.  The attention cores run as sm_100a kernels through the
C-ABI library; the two projections and the optional RMSNorm stay torch ops.

Difference from the reference, by design: the decode step appends to
pre-allocated cache buffers and rewrites the lookahead keys `U` IN PLACE
instead of concatenating new tensors every token (:185-203), so a cache
returned by step t shares memory with the cache returned by step t-1.  Pass
`inplace_cache=False` to get the reference's functional behaviour (each step
then copies the caches first).
"""
from __future__ import annotations

from collections import namedtuple

import torch
from torch import nn

from .ops import castle_attention, castle_attention_packed, castle_decode_step

Cache = namedtuple("Cache", ("U", "qu_cache", "kc_cache", "vc_cache"))


def _capacity_view(t: torch.Tensor):
    """If `t` (B, H, n, d) is the leading rows of a (B, H, cap, d) buffer with cap > n,
    return that full buffer as a view, else None."""
    B, H, n, d = t.shape
    if n == 0 or t.stride(3) != 1 or (n > 1 and t.stride(2) != d):
        return None
    avail = t.untyped_storage().nbytes() // t.element_size() - t.storage_offset()
    if H > 1:
        cap = t.stride(1) // d
        if t.stride(1) != cap * d:
            return None
    elif B > 1:
        cap = t.stride(0) // d
    else:
        cap = avail // d
    if cap <= n or (B > 1 and t.stride(0) != H * cap * d) or avail < B * H * cap * d:
        return None
    return t.as_strided((B, H, cap, d), (H * cap * d, cap * d, d, 1), t.storage_offset())


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
        # kept for signature compatibility only: there is one code path (the CUDA kernels)
        self.use_triton = bool(use_triton) if use_triton is not None else False
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

    def _new_buffers(self, like, rows):
        b, h, _, d = like.shape
        cap = rows + max(self.cache_headroom, rows // 4)
        return [torch.empty(b, h, cap, d, dtype=like.dtype, device=like.device) for _ in range(4)]

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
                if packed is not None:
                    out, U = castle_attention_packed(packed, self.scale, True)
                else:
                    out, U = castle_attention(qc, kc, vc, qu, ku, vu, self.scale, True)
                # the cache lives in buffers with spare rows so that decode steps can append in place
                bufs = self._new_buffers(U, seq_len)
                with torch.no_grad():
                    for buf, src in zip(bufs, (U, qu, kc, vc)):
                        buf[:, :, :seq_len].copy_(src)
                next_cache = Cache(*(buf[:, :, :seq_len] for buf in bufs))
            elif packed is not None:
                out = castle_attention_packed(packed, self.scale, False)
            else:
                out = castle_attention(qc, kc, vc, qu, ku, vu, self.scale, False)
        else:
            t = 0 if cache is None else cache[0].shape[-2]
            bufs = None
            if cache is not None and t > 0:
                views = [_capacity_view(c) for c in cache]
                if all(v is not None for v in views):
                    bufs = views if self.inplace_cache else [v.clone() for v in views]
            if bufs is None:
                bufs = self._new_buffers(qu, t + 1)
                if t > 0:
                    for buf, src in zip(bufs, cache):
                        buf[:, :, :t].copy_(src)
            with torch.no_grad():
                out = castle_decode_step(qc, kc, vc, qu, ku, vu, *bufs, t, self.scale)
            next_cache = Cache(*(buf[:, :, :t + 1] for buf in bufs))

        b, h, n, d = out.shape
        out = out.permute(0, 2, 1, 3).reshape(b, n, h * d)  # 'b h n d -> b n (h d)'
        out = self.combine_heads(out)
        if not return_next_cache:
            return out
        return out, next_cache
