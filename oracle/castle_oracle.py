"""CPU oracle for CASTLE attention (TEST INFRASTRUCTURE - not a product path).

A restatement, in plain PyTorch CPU ops, of the reference's pure-PyTorch CASTLE
path.  It exists only so that tests, the smoke check and the bench's CPU
baseline can check / time the CUDA kernels against it; the shipped package
never imports it.

Pinned: `tests/golden/make_golden.py` imports the real reference
(`lookahead_keys_attention/lookahead_keys_attention.py`) and records its
outputs, autograd gradients and caches on seeded inputs; `tests/test_oracle.py`
checks every function below against those fixtures.

Reference lines followed (paths inside the reference project):
  parallel core   lookahead_keys_attention/lookahead_keys_attention.py:132-164
  decode core     lookahead_keys_attention/lookahead_keys_attention.py:166-203
  module glue     lookahead_keys_attention/lookahead_keys_attention.py:88-104,205-214
  backward math   lookahead_keys_attention/lookahead_keys_attention_triton.py:333-401
                  (the PyTorch path gets the same values from autograd)
"""
from __future__ import annotations

from collections import namedtuple

import torch
import torch.nn.functional as F

Cache = namedtuple("Cache", ("U", "qu_cache", "kc_cache", "vc_cache"))


def _neg_max(t):
    return -torch.finfo(t.dtype).max


def castle_parallel(qc, kc, vc, qu, ku, vu, scale, return_U=False, return_lse=False):
    """Parallel CASTLE core on (..., N, d) tensors; all arithmetic in the input dtype.

    Follows lookahead_keys_attention.py:134-163:
      T[i,j]  = (s*qc_i).vu_j           kept for j <= i        (:142-143)
      A[k,j]  = sigmoid((s*qu_k).ku_j)  kept for j >  k        (:145-146)
      Su      = T @ A^T                                        (:148)
      S       = (s*qc) @ kc^T - silu(Su), k > i -> -finfo.max  (:150-153)
      out     = softmax(S) @ vc                                (:156-159)
      U       = A @ vu                                         (:163)
    """
    n = qc.shape[-2]
    qu_s = qu * scale
    qc_s = qc * scale
    mask = torch.ones((n, n), dtype=torch.bool, device=qc.device).triu(1)
    T = (qc_s @ vu.transpose(-1, -2)).masked_fill(mask, 0.0)
    A = (qu_s @ ku.transpose(-1, -2)).sigmoid().masked_fill(~mask, 0.0)
    Su = T @ A.transpose(-1, -2)
    Sc = qc_s @ kc.transpose(-1, -2)
    S = (Sc - F.silu(Su)).masked_fill(mask, _neg_max(Sc))
    P = S.softmax(dim=-1)
    out = P @ vc
    res = [out]
    if return_U:
        res.append(A @ vu)
    if return_lse:
        res.append(torch.logsumexp(S.float(), dim=-1))
    return res[0] if len(res) == 1 else tuple(res)


def castle_parallel_bwd(qc, kc, vc, qu, ku, vu, scale, dout):
    """Closed-form gradients of `castle_parallel` w.r.t. its six inputs.

    Same algebra as lookahead_keys_attention_triton.py:333-401 and :591-592
    (delta, dS, dSu = -dS*silu'(Su), dT, dA, dZ, then the six products; the
    two query gradients are multiplied by `scale`).  No gradient flows
    through U (:512-515).  Returns (dqc, dkc, dvc, dqu, dku, dvu).
    """
    n = qc.shape[-2]
    qu_s = qu * scale
    qc_s = qc * scale
    mask = torch.ones((n, n), dtype=torch.bool, device=qc.device).triu(1)
    T = (qc_s @ vu.transpose(-1, -2)).masked_fill(mask, 0.0)
    A = (qu_s @ ku.transpose(-1, -2)).sigmoid().masked_fill(~mask, 0.0)
    Su = T @ A.transpose(-1, -2)
    Sc = qc_s @ kc.transpose(-1, -2)
    S = (Sc - F.silu(Su)).masked_fill(mask, _neg_max(Sc))
    P = S.softmax(dim=-1)
    out = P @ vc
    delta = (out * dout).sum(-1, keepdim=True)
    dP = dout @ vc.transpose(-1, -2)
    dS = P * (dP - delta)
    dvc = P.transpose(-1, -2) @ dout
    dkc = dS.transpose(-1, -2) @ qc_s
    dqc_s = dS @ kc
    sg = Su.sigmoid()
    dSu = -dS * (sg * (1 + Su * (1 - sg)))
    dT = (dSu @ A).masked_fill(mask, 0.0)
    dA = (dSu.transpose(-1, -2) @ T).masked_fill(~mask, 0.0)
    dZ = dA * A * (1 - A)
    dqc_s = dqc_s + dT @ vu
    dvu = dT.transpose(-1, -2) @ qc_s
    dqu_s = dZ @ ku
    dku = dZ.transpose(-1, -2) @ qu_s
    return dqc_s * scale, dkc, dvc, dqu_s * scale, dku, dvu


def castle_decode_step(qc, kc, vc, qu, ku, vu, cache, scale):
    """One cached single-token step; inputs are (..., 1, d).

    Follows lookahead_keys_attention.py:169-203: every cached lookahead key
    gets `sigmoid((s*qu_cache_k).ku_t) * vu_t` added (:182-183), a zero row is
    appended (:185), kc/vc/qu are appended (:187-188,202), and the scores
    `(s*qc).kc - silu((s*qc).U)` are soft-maxed without a mask (:190-200).
    Returns (out, Cache).
    """
    if cache is None:
        e = qu[..., 0:0, :]
        cache = (e,) * 4
    U_prev, qu_cache, kc_cache, vc_cache = cache
    qc_s = qc * scale
    a = ((qu_cache * scale) @ ku.transpose(-1, -2)).sigmoid()
    Ut = torch.cat((U_prev + a * vu, torch.zeros_like(qu)), dim=-2)
    kc_all = torch.cat((kc_cache, kc), dim=-2)
    vc_all = torch.cat((vc_cache, vc), dim=-2)
    Sc = qc_s @ kc_all.transpose(-1, -2)
    Su = qc_s @ Ut.transpose(-1, -2)
    P = (Sc - F.silu(Su)).softmax(dim=-1)
    out = P @ vc_all
    return out, Cache(Ut, torch.cat((qu_cache, qu), dim=-2), kc_all, vc_all)


def split_heads(qkvs, heads):
    """'b n (qkv h d) -> qkv b h n d', packed order qu,ku,vu,qc,kc,vc
    (lookahead_keys_attention.py:77,104)."""
    b, n, w = qkvs.shape
    d = w // (6 * heads)
    return qkvs.view(b, n, 6, heads, d).permute(2, 0, 3, 1, 4)


def castle_module_forward(x, w_qkv, w_out, heads, dim_head, norm_weight=None,
                          cache=None, return_next_cache=None, eps=None):
    """Module-level forward: (RMSNorm) -> 6-way projection -> core -> merge -> out
    projection (lookahead_keys_attention.py:88-104 and :205-214).  Rotary is
    not restated (third-party package absent; parity unpinned for it)."""
    n = x.shape[1]
    is_inference = n == 1
    if return_next_cache is None:
        return_next_cache = is_inference
    if norm_weight is not None:
        x = F.rms_norm(x, (x.shape[-1],), norm_weight, eps)
    qu, ku, vu, qc, kc, vc = split_heads(x @ w_qkv.t(), heads)
    scale = dim_head ** -0.5
    if not is_inference:
        assert cache is None, "must be inferencing single tokens if receiving cache"
        if return_next_cache:
            out, U = castle_parallel(qc, kc, vc, qu, ku, vu, scale, return_U=True)
            next_cache = Cache(U, qu, kc, vc)
        else:
            out = castle_parallel(qc, kc, vc, qu, ku, vu, scale)
    else:
        out, next_cache = castle_decode_step(qc, kc, vc, qu, ku, vu, cache, scale)
    b, h, n, d = out.shape
    out = out.permute(0, 2, 1, 3).reshape(b, n, h * d) @ w_out.t()
    return (out, next_cache) if return_next_cache else out


# ---------------------------------------------------------------------------
# Blockwise O(N^2 d) form.  Not in the reference: it is the recurrence the CUDA
# kernels evaluate, restated here so the CPU suite can check its algebra
# (forward and backward, including the descending "peel" of the state) against
# the dense functions above before any kernel runs.
# ---------------------------------------------------------------------------

def castle_parallel_blockwise(qc, kc, vc, qu, ku, vu, scale, block=32):
    """Key-stationary blockwise forward for one (N, d) head.  For key block K
    the state W_K = sum_{J<I} A[K,J] @ Vu[J] is carried over ascending query
    blocks I, and Su[I,K] = Qc[I] @ W_K^T + tril(T[I,I]) @ A[K,I]^T.
    Returns (out, U, lse)."""
    n, d = qc.shape
    nb = (n + block - 1) // block
    qc_s, qu_s = qc * scale, qu * scale
    m = torch.full((n,), -float("inf"), dtype=qc.dtype)
    l = torch.zeros(n, dtype=qc.dtype)
    acc = torch.zeros(n, d, dtype=qc.dtype)
    U = torch.zeros(n, d, dtype=qc.dtype)
    idx = torch.arange(n)
    for K in range(nb):
        ks = slice(K * block, min(n, (K + 1) * block))
        W = torch.zeros(ks.stop - ks.start, d, dtype=qc.dtype)
        for I in range(K, nb):
            i_s = slice(I * block, min(n, (I + 1) * block))
            ii, kk = idx[i_s], idx[ks]
            A = (qu_s[ks] @ ku[i_s].T).sigmoid() * (ii[None, :] > kk[:, None])
            T = (qc_s[i_s] @ vu[i_s].T) * (ii[None, :] <= ii[:, None])
            Su = qc_s[i_s] @ W.T + T @ A.T
            S = qc_s[i_s] @ kc[ks].T - F.silu(Su)
            S = S.masked_fill(kk[None, :] > ii[:, None], -float("inf"))
            W = W + A @ vu[i_s]
            m_t = S.max(dim=-1).values
            m_new = torch.maximum(m[i_s], m_t)
            p = torch.exp(S - m_new[:, None])
            alpha = torch.exp(m[i_s] - m_new)
            acc[i_s] = acc[i_s] * alpha[:, None] + p @ vc[ks]
            l[i_s] = l[i_s] * alpha + p.sum(-1)
            m[i_s] = m_new
        U[ks] = W
    return acc / l[:, None], U, m + l.log()


def castle_parallel_bwd_blockwise(qc, kc, vc, qu, ku, vu, scale, out, lse, U, dout, block=32):
    """Key-stationary blockwise backward for one (N, d) head: query blocks are
    visited in DESCENDING order, the forward state is recovered by peeling
    W_K -= A[K,I] @ Vu[I] from the final U[K], and the reverse state
    G_K = sum_{I'>I} dSu[I',K]^T @ Qc[I'] feeds dA and dvu."""
    n, d = qc.shape
    nb = (n + block - 1) // block
    qc_s, qu_s = qc * scale, qu * scale
    delta = (out * dout).sum(-1)
    dqc = torch.zeros_like(qc); dkc = torch.zeros_like(qc); dvc = torch.zeros_like(qc)
    dqu = torch.zeros_like(qc); dku = torch.zeros_like(qc); dvu = torch.zeros_like(qc)
    idx = torch.arange(n)
    for K in range(nb):
        ks = slice(K * block, min(n, (K + 1) * block))
        W = U[ks].clone()
        G = torch.zeros_like(W)
        for I in range(nb - 1, K - 1, -1):
            i_s = slice(I * block, min(n, (I + 1) * block))
            ii, kk = idx[i_s], idx[ks]
            A = (qu_s[ks] @ ku[i_s].T).sigmoid() * (ii[None, :] > kk[:, None])
            W = W - A @ vu[i_s]
            T = (qc_s[i_s] @ vu[i_s].T) * (ii[None, :] <= ii[:, None])
            Su = qc_s[i_s] @ W.T + T @ A.T
            S = qc_s[i_s] @ kc[ks].T - F.silu(Su)
            P = torch.exp(S - lse[i_s][:, None]) * (kk[None, :] <= ii[:, None])
            dP = dout[i_s] @ vc[ks].T
            dS = P * (dP - delta[i_s][:, None])
            dvc[ks] += P.T @ dout[i_s]
            dkc[ks] += dS.T @ qc_s[i_s]
            sg = Su.sigmoid()
            dSu = -dS * (sg * (1 + Su * (1 - sg)))
            dq = dS @ kc[ks] + dSu @ W
            dA = (G @ vu[i_s].T + dSu.T @ T) * (ii[None, :] > kk[:, None])
            dT = (dSu @ A) * (ii[None, :] <= ii[:, None])
            dq += dT @ vu[i_s]
            dvu[i_s] += A.T @ G + dT.T @ qc_s[i_s]
            G = G + dSu.T @ qc_s[i_s]
            dZ = dA * A * (1 - A)
            dqu[ks] += dZ @ ku[i_s]
            dku[i_s] += dZ.T @ qu_s[ks]
            dqc[i_s] += dq
    return dqc * scale, dkc, dvc, dqu * scale, dku, dvu
