"""Operator layer: the CASTLE attention core as torch-facing functions that hand
raw device pointers, strides and the current stream to the C-ABI library.

`castle_attention` mirrors the reference operator
`castle_attention_triton(qc, kc, vc, qu, ku, vu, scale, return_U_for_cache)`
(lookahead_keys_attention/lookahead_keys_attention_triton.py:416-605): same
argument order (causal triple first), unscaled inputs, returns `out` or
`(out, U)`, six input gradients, no gradient through U.
`castle_decode_step` replaces the single-token branch of the reference module
(lookahead_keys_attention/lookahead_keys_attention.py:166-203).
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib
from ._lib import CastleProblem, CastleTensor

_DTYPES = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}

_status_words: dict = {}
_workspaces: dict = {}


def _require_cuda(t: torch.Tensor, what: str):
    if not t.is_cuda:
        raise RuntimeError(f"{what}: expected CUDA tensors; this package has no CPU path")


def status_word(device) -> torch.Tensor:
    """Per-device int32 the kernels OR error bits into (0 = fine)."""
    device = torch.device(device)
    w = _status_words.get(device)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[device] = w
    return w


def check_status(device=None):
    """Synchronising check of the device status word; raises on a kernel-side failure."""
    devs = [torch.device(device)] if device is not None else list(_status_words)
    for d in devs:
        v = int(status_word(d).item())
        if v != 0:
            status_word(d).zero_()
            raise RuntimeError(f"castle kernels reported status {v} on {d} (1 = a bounded wait ran out)")


def _workspace(device, nbytes: int) -> torch.Tensor:
    """Scratch buffer per (device, stream), grown on demand and kept between calls (kernels of
    one stream run in order, so they can share it; two streams must not).  `release_workspaces()`
    gives the memory back."""
    key = (torch.device(device), torch.cuda.current_stream(device).cuda_stream)
    w = _workspaces.get(key)
    if w is None or w.numel() < nbytes:
        _workspaces.pop(key, None)   # drop the old buffer before allocating the larger one
        w = None
        w = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = w
    return w


def release_workspaces():
    """Free every cached scratch buffer (they are re-created on the next call)."""
    _workspaces.clear()


def _desc(t: torch.Tensor) -> CastleTensor:
    """(B, H, N, d) tensor or view with a contiguous last dim -> castle_tensor_t."""
    assert t.dim() == 4 and (t.stride(3) == 1 or t.shape[3] == 1)
    return CastleTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def _aligned_view(t: torch.Tensor) -> torch.Tensor:
    """Views into the packed projection are used as they are when the ABI's
    alignment rules hold (16-byte base and strides); otherwise copy."""
    es = t.element_size()
    ok = t.stride(3) == 1 and t.data_ptr() % 16 == 0 and all((t.stride(i) * es) % 16 == 0 for i in range(3))
    return t if ok else t.contiguous()


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


# Bound on the forward's scratch per launch.  The soft-max partials take N^2/128 * (8 + 2*d) bytes
# per (batch, head) pair (O(N^2), where the reference kernel needs O(N*d)), so a call is cut into
# launches over whole batch rows, or over head ranges of one batch row, that each stay below it.
MAX_WORKSPACE_BYTES = 16 << 30


def forward_chunks(B: int, H: int, per_pair: int, limit: int | None = None):
    """Rectangles (b0, b1, h0, h1) of the (batch, head) grid, each needing at most `limit` bytes of
    scratch at `per_pair` bytes per pair.  A rectangle spans several batch rows only with all heads,
    so that the per-pair fp32 buffers (lse, state) of a rectangle stay contiguous."""
    limit = MAX_WORKSPACE_BYTES if limit is None else limit
    pairs = limit // max(per_pair, 1)
    if pairs < 1:
        raise RuntimeError(f"castle_attention: one (batch, head) pair needs {per_pair} bytes of forward scratch, "
                           f"more than the {limit}-byte bound (sequence too long for this build)")
    def even(total, most):   # cut `total` into the fewest pieces of at most `most`, all about the same size
        n = -(-total // most)
        size = -(-total // n)
        return [(i, min(total, i + size)) for i in range(0, total, size)]

    if pairs >= H:
        return [(b0, b1, 0, H) for b0, b1 in even(B, min(B, pairs // H))]
    return [(b, b + 1, h0, h1) for b in range(B) for h0, h1 in even(H, pairs)]


# From this sequence length on, bf16 callers are computed with fp16 operands.  The lookahead state W grows
# like sqrt(N) (|W| ~ 100 at N = 8192) and the gate's and the state's 16-bit copies are what the long-range
# gradients are made of: with 8 significant bits dqc misses |a-b| <= 2e-2 + 1e-2|b| from N ~ 8192 on, with
# fp16's 11 bits it holds at N = 16384.  (The tensor cores cannot mix an fp16 operand with a bf16 one in a
# single product, so the inputs are converted once instead; at these lengths that pass is < 1 % of the work.)
# Costs: values beyond +-65504 in q/k/v saturate, and the upstream gradient is rescaled by a power of two
# (exactly) so that small gradients do not underflow.
LONG_SEQ_FP16 = 6144


def compute_dtype(dtype: torch.dtype, seq_len: int) -> torch.dtype:
    """Operand type of the kernels for a caller of `dtype`: fp16 for fp32 callers (as the reference
    operator does, lookahead_keys_attention_triton.py:437-442) and for bf16 callers at long sequences."""
    if dtype == torch.float16 or (dtype == torch.bfloat16 and seq_len < LONG_SEQ_FP16):
        return dtype
    return torch.float16


def prefill_writes_caches(dtype: torch.dtype, d: int, seq_len: int = 0) -> bool:
    """Whether the forward kernels can fill the decode caches themselves: they store their 16-bit
    operand tiles, so the caller's dtype must be the compute dtype and dim_head a tile width."""
    return dtype in (torch.bfloat16, torch.float16) and compute_dtype(dtype, seq_len) == dtype and d in (64, 128)


def _convert_16bit(t: torch.Tensor, mul: torch.Tensor | None = None) -> torch.Tensor:
    """One pass: contiguous bf16 -> fp16 (saturating) or fp16 -> bf16, times the device scalar `mul`."""
    lib = _lib.load()
    out = torch.empty_like(t, dtype=torch.float16 if t.dtype == torch.bfloat16 else torch.bfloat16)
    rc = lib.castle_convert_16bit(_DTYPES[t.dtype], t.data_ptr(), out.data_ptr(), t.numel(),
                                  mul.data_ptr() if mul is not None else None, _stream(t.device))
    _lib.check(rc, "castle_convert_16bit")
    return out


def _to_fp16(t: torch.Tensor) -> torch.Tensor:
    """fp16 copy that saturates instead of overflowing to infinity."""
    if t.dtype == torch.float16:
        return t
    if t.dtype == torch.bfloat16 and t.is_cuda and t.is_contiguous() and t.numel() % 8 == 0 and t.data_ptr() % 16 == 0:
        return _convert_16bit(t)
    return t.clamp(-65504.0, 65504.0).to(torch.float16)


class _CastleAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qc, kc, vc, qu, ku, vu, scale, return_U, cache_out=None):
        return _CastleAttention.run_forward(ctx, qc, kc, vc, qu, ku, vu, scale, return_U,
                                            any(ctx.needs_input_grad[:6]), cache_out)

    @staticmethod
    def run_forward(ctx, qc, kc, vc, qu, ku, vu, scale, return_U, need_grad, cache_out=None, out_dtype=None):
        """Shared by the six-view and the packed operator; `need_grad` says whether to save state.
        `cache_out` = four (B, H, N, d) views of decode-cache buffers the kernels fill (prefill)."""
        _require_cuda(qc, "castle_attention")
        lib = _lib.load()
        B, H, N, d = qc.shape
        orig_dtype = qc.dtype if out_dtype is None else out_dtype
        # compute dtype: 16-bit inputs run as they are; fp32 callers, and bf16 callers at long
        # sequences, run with fp16 operands
        cdtype = compute_dtype(orig_dtype, N)
        dp = 64 if d <= 64 else 128
        if d > 128 or d % 8:
            raise RuntimeError(f"castle_attention: dim_head {d} not supported (multiples of 8 up to 128)")
        if cache_out is not None:
            if not (return_U and prefill_writes_caches(orig_dtype, d, N)):
                raise RuntimeError("castle_attention: cache_out needs return_U, a 16-bit dtype and dim_head 64 or 128")
            for c in cache_out:
                if c.shape != (B, H, N, d) or c.dtype != orig_dtype or c.stride(3) != 1:
                    raise RuntimeError("castle_attention: cache_out tensors must be (B, H, N, d) views in the input dtype")

        def prep(t):
            if t.dtype != cdtype:
                t = _to_fp16(t)
            if dp != d:
                t = F.pad(t, (0, dp - d))  # zero columns change no dot product; scale uses the true d
            return _aligned_view(t)

        ins = [prep(t) for t in (qc, kc, vc, qu, ku, vu)]
        dev = qc.device
        # laid out (B, N, H, d): merging heads afterwards is a free reshape
        out = torch.empty(B, N, H, dp, dtype=cdtype, device=dev).permute(0, 2, 1, 3)
        lse = torch.empty(B, H, N, dtype=torch.float32, device=dev)
        if cache_out is not None:
            U = cache_out[0]
        else:
            U = torch.empty(B, H, N, dp, dtype=orig_dtype, device=dev) if return_U else None
        wst = torch.empty(B, H, N, dp, dtype=torch.float32, device=dev) if need_grad else None
        st = status_word(dev)
        # cut the (batch, head) grid so the partial-softmax scratch of one launch stays bounded
        prob1 = CastleProblem(1, 1, N, dp, _DTYPES[cdtype], float(scale))
        per_pair = max(int(lib.castle_fwd_workspace_bytes(ctypes.byref(prob1))), 1)
        chunks = forward_chunks(B, H, per_pair)
        ws = _workspace(dev, max(per_pair * (b1 - b0) * (h1 - h0) for b0, b1, h0, h1 in chunks))
        for b0, b1, h0, h1 in chunks:
            prob = CastleProblem(b1 - b0, h1 - h0, N, dp, _DTYPES[cdtype], float(scale))
            d6 = [_desc(t[b0:b1, h0:h1]) for t in ins]
            do = _desc(out[b0:b1, h0:h1])
            wptr = wst[b0:b1, h0:h1].data_ptr() if need_grad else None
            if cache_out is not None:
                dc = [_desc(c[b0:b1, h0:h1]) for c in cache_out]
                rc = lib.castle_fwd_prefill(ctypes.byref(prob), *[ctypes.byref(x) for x in d6], ctypes.byref(do),
                                            lse[b0:b1, h0:h1].data_ptr(), *[ctypes.byref(x) for x in dc], wptr,
                                            ws.data_ptr(), ws.numel(), st.data_ptr(), _stream(dev))
                _lib.check(rc, "castle_fwd_prefill")
                continue
            du = _desc(U[b0:b1, h0:h1]) if return_U else None
            rc = lib.castle_fwd(ctypes.byref(prob), *[ctypes.byref(x) for x in d6], ctypes.byref(do),
                                lse[b0:b1, h0:h1].data_ptr(), ctypes.byref(du) if return_U else None,
                                _DTYPES[orig_dtype], wptr, ws.data_ptr(), ws.numel(), st.data_ptr(), _stream(dev))
            _lib.check(rc, "castle_fwd")
        if need_grad:
            ctx.save_for_backward(*ins, out, lse, wst)
        ctx.scale, ctx.d, ctx.dp, ctx.orig_dtype, ctx.cdtype = float(scale), d, dp, orig_dtype, cdtype
        o = out[..., :d]
        if orig_dtype != cdtype:
            o = o.to(orig_dtype)
        if return_U:
            U = U[..., :d]
            ctx.mark_non_differentiable(U)
            return o, U
        return o

    @staticmethod
    def backward(ctx, do, dU=None, packed_out=False):
        lib = _lib.load()
        qc, kc, vc, qu, ku, vu, out, lse, wst = ctx.saved_tensors
        B, H, N, dp = qc.shape
        d, cdtype, dev = ctx.d, ctx.cdtype, qc.device
        inv_s = None
        if do.dtype != cdtype:
            # fp16 operands for a caller with a wider exponent range: bring the upstream gradient to a
            # fixed magnitude with a power of two (exact; every gradient is linear in it) and undo it on
            # the results, so that neither small gradients underflow nor large ones overflow in fp16.
            # Everything stays on the device: no host synchronisation.
            amax = do.detach().abs().amax().float().clamp_min(1e-30)
            # largest power of two <= 64 / amax, from the exponent field (frexp: x = m * 2^e, 0.5 <= m < 1)
            expo = torch.frexp(64.0 / amax)[1] - 1
            s = torch.ldexp(torch.ones_like(amax), expo.clamp(-24, 24))
            inv_s = (1.0 / s).reshape(1)
            if do.dtype == torch.bfloat16 and do.is_contiguous() and do.numel() % 8 == 0 and do.data_ptr() % 16 == 0:
                do = _convert_16bit(do, s.reshape(1))
            else:
                do = (do.float() * s).to(cdtype)
        if dp != d:
            do = F.pad(do, (0, dp - d))
        do = _aligned_view(do)
        # the six gradients in the packed layout the projection's backward consumes:
        # (B, N, 6, H, d) with order qu,ku,vu,qc,kc,vc, handed to the kernels as strided views
        packed = torch.empty(B, N, 6, H, dp, dtype=cdtype, device=dev)
        gqu, gku, gvu, gqc, gkc, gvc = (packed[:, :, i].permute(0, 2, 1, 3) for i in range(6))
        st = status_word(dev)
        prob = CastleProblem(B, H, N, dp, _DTYPES[cdtype], ctx.scale)
        nbytes = int(lib.castle_bwd_workspace_bytes(ctypes.byref(prob)))
        if dp == 128 and nbytes > MAX_WORKSPACE_BYTES:
            # the tile hand-over scratch of the dim_head-128 kernels may be smaller than asked for: the
            # (batch, head) pairs then run in smaller chunks, down to one pair at a time
            nblk = -(-N // 128)
            pair = nblk * (nblk + 1) // 2 * 3 * 32768
            asked_pairs = min(B * H, max(1, (8 << 30) // pair))
            least = nbytes - (asked_pairs - 1) * pair            # the accumulators and one pair's tiles
            nbytes = max(least, MAX_WORKSPACE_BYTES)
        ws = _workspace(dev, nbytes)
        args = [_desc(t) for t in (qc, kc, vc, qu, ku, vu, out, do)]
        grads = [_desc(t) for t in (gqc, gkc, gvc, gqu, gku, gvu)]
        rc = lib.castle_bwd(ctypes.byref(prob), *[ctypes.byref(x) for x in args], lse.data_ptr(), wst.data_ptr(),
                            *[ctypes.byref(x) for x in grads], ws.data_ptr(), ws.numel(), st.data_ptr(), _stream(dev))
        _lib.check(rc, "castle_bwd")
        def back(g):   # to the caller's dtype, undoing the power-of-two scale of the upstream gradient
            if ctx.orig_dtype == cdtype:
                return g
            if ctx.orig_dtype == torch.bfloat16 and g.is_contiguous() and g.numel() % 8 == 0:
                return _convert_16bit(g, inv_s)
            g = g.to(ctx.orig_dtype)
            return g.mul_(inv_s.to(ctx.orig_dtype)) if inv_s is not None else g

        if packed_out:
            return back(packed[..., :d])
        return (*[back(g[..., :d]) for g in (gqc, gkc, gvc, gqu, gku, gvu)], None, None, None)


class _CastleAttentionPacked(torch.autograd.Function):
    """Same kernels, one autograd input: the packed projection output (B, N, 6, H, d) in the
    order qu,ku,vu,qc,kc,vc.  Its gradient is the packed buffer the backward kernels write, so
    autograd has nothing to scatter or sum (six separate view-gradients cost ~10 extra passes)."""

    @staticmethod
    def forward(ctx, packed, scale, return_U, cache_out=None):
        out_dtype = packed.dtype
        if compute_dtype(out_dtype, packed.shape[1]) != out_dtype:
            packed = _to_fp16(packed)   # one pass over the whole projection output instead of six over its views
        qu, ku, vu, qc, kc, vc = (packed[:, :, i].permute(0, 2, 1, 3) for i in range(6))
        return _CastleAttention.run_forward(ctx, qc, kc, vc, qu, ku, vu, scale, return_U, ctx.needs_input_grad[0],
                                            cache_out, out_dtype)

    @staticmethod
    def backward(ctx, do, dU=None):
        return _CastleAttention.backward(ctx, do, dU, packed_out=True), None, None, None


def castle_attention_packed(packed, scale, return_U_for_cache=False, cache_out=None):
    """Parallel CASTLE attention on the packed projection output (B, N, 6, H, d), order
    qu,ku,vu,qc,kc,vc (the layout `to_all_qkv` produces).  Returns out (B, H, N, d) [, U].
    With `cache_out` = four (B, H, N, d) views (U, qu, kc, vc) of decode-cache buffers, the
    kernels write the cache rows themselves and the returned U is cache_out[0]."""
    return _CastleAttentionPacked.apply(packed, scale, bool(return_U_for_cache), cache_out)


def castle_attention(qc, kc, vc, qu, ku, vu, scale, return_U_for_cache=False, cache_out=None):
    """Parallel CASTLE attention on (B, H, N, d) tensors (views are fine).
    Returns `out`, or `(out, U)` when `return_U_for_cache`; `cache_out` as in `castle_attention_packed`."""
    return _CastleAttention.apply(qc, kc, vc, qu, ku, vu, scale, bool(return_U_for_cache), cache_out)


def castle_decode_step(qc, kc, vc, qu, ku, vu, U, qu_cache, kc_cache, vc_cache, cache_len: int, scale: float):
    """One cached token.  The four caches are (B, H, capacity, d) buffers with `cache_len`
    valid rows; they are updated IN PLACE (row `cache_len` appended, U[0:cache_len] rewritten).
    The six new-token tensors are (B, H, 1, d).  Returns out (B, H, 1, d)."""
    _require_cuda(qc, "castle_decode_step")
    lib = _lib.load()
    B, H, one, d = qc.shape
    assert one == 1
    dt = qc.dtype
    if dt not in _DTYPES:
        raise RuntimeError(f"castle_decode_step: dtype {dt} not supported")
    cap = U.shape[2]
    for c in (U, qu_cache, kc_cache, vc_cache):
        assert c.dtype == dt and c.shape == (B, H, cap, d) and c.stride(3) == 1
    dev = qc.device
    news = [_aligned_view(t) for t in (qc, kc, vc, qu, ku, vu)]
    out = torch.empty(B, H, 1, d, dtype=dt, device=dev)
    prob = CastleProblem(B, H, 1, d, _DTYPES[dt], float(scale))
    nbytes = int(lib.castle_decode_workspace_bytes(ctypes.byref(prob), cache_len))
    ws = _workspace(dev, nbytes)
    descs = [_desc(t) for t in (*news, U, qu_cache, kc_cache, vc_cache, out)]
    rc = lib.castle_decode_step(ctypes.byref(prob), cache_len, cap, *[ctypes.byref(x) for x in descs],
                                ws.data_ptr(), ws.numel(), status_word(dev).data_ptr(), _stream(dev))
    _lib.check(rc, "castle_decode_step")
    return out
