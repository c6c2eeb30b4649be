"""Gated delta rule (GatedDeltaNet linear attention of Qwen3.5 / Qwen3-Next).

Per value head, with state ``S [dk, dv]``, decay ``a_t = exp(g_t)`` and write strength ``beta_t``::

    S_t = a_t S_{t-1} + k_t (beta_t (v_t - a_t S_{t-1}^T k_t))^T        o_t = S_t^T q_t

* :func:`gated_delta_recurrent` - the rule as written, one token at a time (the oracle).
* :func:`gated_delta_chunked`   - the same result from chunks of 64 tokens: inside a chunk the
  token-to-token dependence is a unit lower-triangular system that is solved once
  (``(I + tril(K_beta K^T * decay, -1))^-1``), so a chunk costs a handful of matrix products and only
  the chunk-to-chunk state update is sequential.  Used for prefill.
* :func:`gated_delta_step` / :func:`conv1d_step` - one decode step for a batch of sequences on state
  pools indexed by slot (CUDA kernels in csrc/linear_attn/gated_delta.cu; PyTorch on the CPU).

Reference: vllm/model_executor/models/qwen3_5.py:127-200 (chunk-64 rule), :203-260 (recurrent rule).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _DT, _count, _lib, _p, _stream


def gated_delta_recurrent(q, k, v, g, beta, S0=None):
    """q, k: [L, H, dk]; v: [L, H, dv]; g, beta: [L, H]; S0: [H, dk, dv] or None.  fp32 in, fp32 out.
    Returns (o [L, H, dv], S [H, dk, dv])."""
    L, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv, dtype=torch.float32, device=q.device) if S0 is None else S0.float().clone()
    o = torch.empty(L, H, dv, dtype=torch.float32, device=q.device)
    for t in range(L):
        S = S * torch.exp(g[t])[:, None, None]
        mem = torch.einsum("hkv,hk->hv", S, k[t])
        delta = (v[t] - mem) * beta[t][:, None]
        S = S + k[t][:, :, None] * delta[:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def gated_delta_chunked(q, k, v, g, beta, S0=None, chunk: int = 64):
    """Same contract as :func:`gated_delta_recurrent`, computed chunk-wise."""
    L, H, dk = q.shape
    dv = v.shape[-1]
    dev = q.device
    pad = (-L) % chunk
    if pad:
        # padded tokens: beta = 0 (no write), g = 0 (no decay), q = k = 0: they change nothing
        zp = lambda t: F.pad(t, (0, 0) * (t.dim() - 1) + (0, pad))
        q, k, v, g, beta = zp(q), zp(k), zp(v), zp(g), zp(beta)
    N = (L + pad) // chunk
    # [H, N, C, d]
    qc = q.float().permute(1, 0, 2).reshape(H, N, chunk, dk)
    kc = k.float().permute(1, 0, 2).reshape(H, N, chunk, dk)
    vc = v.float().permute(1, 0, 2).reshape(H, N, chunk, dv)
    bc = beta.float().t().reshape(H, N, chunk)
    gc = g.float().t().reshape(H, N, chunk).cumsum(-1)                 # log decay from the chunk start (inclusive)
    v_beta = vc * bc[..., None]
    k_beta = kc * bc[..., None]
    diff = gc[..., :, None] - gc[..., None, :]                          # log decay from token j to token i
    lower = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=dev))
    decay = torch.where(lower, diff, torch.full_like(diff, float("-inf"))).exp()
    # token i's write sees the writes of tokens j < i of its chunk: (I + A) U = V_beta with strictly lower A
    A = torch.tril((k_beta @ kc.transpose(-1, -2)) * decay, diagonal=-1)
    eye = torch.eye(chunk, dtype=torch.float32, device=dev)
    T = torch.linalg.solve_triangular(eye + A, eye.expand_as(A).contiguous(), upper=False)
    u = T @ v_beta                                                       # writes if the incoming state were zero
    w = T @ (k_beta * gc.exp()[..., None])                               # what each write reads from the incoming state
    S = torch.zeros(H, dk, dv, dtype=torch.float32, device=dev) if S0 is None else S0.float().clone()
    o = torch.empty(H, N, chunk, dv, dtype=torch.float32, device=dev)
    strict = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=dev), diagonal=0)
    for i in range(N):
        qi, ki = qc[:, i], kc[:, i]
        attn = torch.where(strict, (qi @ ki.transpose(-1, -2)) * decay[:, i], torch.zeros((), device=dev))
        v_new = u[:, i] - w[:, i] @ S
        o[:, i] = (qi * gc[:, i].exp()[..., None]) @ S + attn @ v_new
        g_last = gc[:, i, -1]
        S = S * g_last.exp()[:, None, None] + (ki * (g_last[:, None] - gc[:, i]).exp()[..., None]).transpose(-1, -2) @ v_new
    o = o.reshape(H, N * chunk, dv).permute(1, 0, 2)[:L].contiguous()
    return o, S


def gated_delta_step(pool: torch.Tensor, slots: torch.Tensor, q, k, v, g, beta, out=None):
    """One token per sequence.  pool: fp32 [num_slots, H, dk, dv] (updated in place); slots: int32 [B];
    q, k: fp32 [B, H, dk]; v: fp32 [B, H, dv]; g, beta: fp32 [B, H].  Returns o fp32 [B, H, dv]."""
    B, H, dk = q.shape
    dv = v.shape[-1]
    if out is None:
        out = torch.empty(B, H, dv, dtype=torch.float32, device=q.device)
    if not q.is_cuda:
        for b in range(B):
            s = int(slots[b])
            if s < 0:
                continue
            o, S = gated_delta_recurrent(q[b:b + 1], k[b:b + 1], v[b:b + 1], g[b:b + 1], beta[b:b + 1], pool[s])
            pool[s].copy_(S)
            out[b] = o[0]
        return out
    for t in (q, k, v, g, beta):
        assert t.dtype == torch.float32 and t.is_contiguous()
    assert pool.dtype == torch.float32 and pool.is_contiguous() and slots.dtype == torch.int32
    rc = _lib.kernels().fi_gdn_step(_p(pool), _p(slots), _p(q), _p(k), _p(v), _p(g), _p(beta), _p(out), B, H, dk, dv,
                                    _stream())
    _lib.check(rc, "fi_gdn_step")
    _count()
    return out


def conv1d_step(x: torch.Tensor, pool: torch.Tensor, slots: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Causal depthwise convolution + SiLU for one new input per sequence.  x: [B, C]; pool:
    [num_slots, C, kw - 1] (the previous inputs, updated in place); w: [C, kw].  Returns fp32 [B, C]."""
    B, C = x.shape
    kw = w.shape[1]
    if not x.is_cuda:
        y = torch.empty(B, C, dtype=torch.float32)
        for b in range(B):
            s = int(slots[b])
            if s < 0:
                y[b] = 0
                continue
            win = torch.cat([pool[s].float(), x[b].float()[:, None]], dim=1)        # [C, kw]
            y[b] = F.silu((win * w.float()).sum(-1))
            pool[s].copy_(win[:, 1:].to(pool.dtype))
        return y
    y = torch.empty(B, C, dtype=torch.float32, device=x.device)
    assert x.stride(1) == 1 and pool.is_contiguous() and w.is_contiguous() and pool.dtype == x.dtype == w.dtype
    rc = _lib.kernels().fi_conv1d_step(_p(x), x.stride(0), _p(pool), _p(slots), _p(w), _p(y), B, C, kw, _DT[x.dtype],
                                       _stream())
    _lib.check(rc, "fi_conv1d_step")
    _count()
    return y
