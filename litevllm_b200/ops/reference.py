"""Plain PyTorch fp32 implementations of every op.

They are the numerical oracle for the CUDA kernels (tests compare against them) and the execution
path for CPU tensors, so the whole engine also runs on a machine without a GPU.  Semantics follow
the reference project's eager code: RMSNorm rounds the normalised value to the storage dtype before
the weight multiply (vllm/model_executor/layers/layernorm.py:17-21), neox rotary pairs (i, i+d/2)
(vllm/model_executor/layers/rotary_embedding/common.py:139-168), softcap = cap*tanh(s/cap) before
masking (vllm/kernels/triton/paged_attention.py:306-582), fp8 KV stored as x/scale and read as
x*scale.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def apply_act(x: torch.Tensor, act: str | None) -> torch.Tensor:
    if act in (None, "none"):
        return x
    if act == "silu":
        return F.silu(x)
    if act in ("gelu_tanh", "gelu_pytorch_tanh", "gelu"):
        return F.gelu(x, approximate="tanh")
    raise ValueError(f"unknown activation {act}")


def linear(x, w, bias=None, residual=None, act=None, out_dtype=None):
    y = x.float() @ w.float().t()
    if act:
        y = apply_act(y, act)
    if bias is not None:
        y = y + bias.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype or x.dtype)


def gated_linear(x, w_gate_up, act="silu", out_dtype=None):
    inter = w_gate_up.shape[0] // 2
    y = x.float() @ w_gate_up.float().t()
    return (apply_act(y[:, :inter], act) * y[:, inter:]).to(out_dtype or x.dtype)


def rmsnorm(x, w, eps, residual=None, w_mode=0, out_scale=1.0):
    """Returns (out, new_residual).  w_mode 0: *w, 1: *(1+w), 2: no weight."""
    if residual is not None:
        x = (x.float() + residual.float()).to(x.dtype)
        residual = x
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * out_scale
    normed = (xf * inv).to(x.dtype).float()
    if w_mode == 0:
        normed = normed * w.float()
    elif w_mode == 1:
        normed = normed * (1.0 + w.float())
    return normed.to(x.dtype), residual


def build_cos_sin(rot_dim: int, max_pos: int, base: float, scaling: float = 1.0,
                  inv_freq: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 table [max_pos, rot_dim] = [cos | sin] used by ``rope_and_cache``."""
    if inv_freq is None:
        inv_freq = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
    t = torch.arange(max_pos, dtype=torch.float64) / scaling
    ang = torch.outer(t, inv_freq.double())
    return torch.cat([ang.cos(), ang.sin()], dim=-1).float()


def _head_norm(x, w, eps, mode):
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = (xf * inv).to(x.dtype).float()
    if w is not None:
        y = y * ((1.0 + w.float()) if mode == 1 else w.float())
    return y.to(x.dtype)


def fp8_quant(x: torch.Tensor, scale: float) -> torch.Tensor:
    return (x.float() / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)


def rope_and_cache(qkv, positions, cos_sin, slot_mapping, k_cache, v_cache, nh, nkv, hd, rot_dim,
                   freq_stream=None, q_norm_w=None, k_norm_w=None, qk_norm_mode=-1, v_norm=False,
                   eps=1e-6, k_scale=1.0, v_scale=1.0):
    """In place: normalise/rotate q and k inside ``qkv`` and scatter k, v into the paged cache
    ``[num_blocks, nkv, block_size, hd]``.  positions: [T] or [streams, T]."""
    T = qkv.shape[0]
    if T == 0:
        return
    x = qkv.view(T, nh + 2 * nkv, hd)
    q, k, v = x[:, :nh], x[:, nh:nh + nkv], x[:, nh + nkv:]
    if qk_norm_mode >= 0:
        q.copy_(_head_norm(q, q_norm_w, eps, qk_norm_mode))
        k.copy_(_head_norm(k, k_norm_w, eps, qk_norm_mode))
    if v_norm:
        v.copy_(_head_norm(v, None, eps, 0))
    half = rot_dim // 2
    pos = positions.view(-1, T).long()
    if freq_stream is None:
        rows = cos_sin[pos[0]]  # [T, rot_dim]
        cos, sin = rows[:, :half], rows[:, half:]
    else:
        fs = freq_stream.long()
        p_sel = pos[fs, :].t()  # [T, half]
        idx = torch.arange(half, device=qkv.device)
        cos = cos_sin[p_sel, idx]
        sin = cos_sin[p_sel, idx + half]
    cos, sin = cos[:, None, :].float(), sin[:, None, :].float()
    for t in (q, k):
        a, b = t[..., :half].float(), t[..., half:rot_dim].float()
        ra = (a * cos - b * sin).to(qkv.dtype)
        rb = (b * cos + a * sin).to(qkv.dtype)
        t[..., :half] = ra
        t[..., half:rot_dim] = rb
    reshape_and_cache(k, v, slot_mapping, k_cache, v_cache, k_scale, v_scale)


# ---- row-scaled cache formats: one fp32 scale per (token, kv head) row, kept in ``cache.fi_scales``
# [num_blocks, nkv, block_size]; ``cache.fi_mode`` = 2 (e4m3 rows, "block-scaled" fp8) or 3 (packed int4)
def kv_mode(cache) -> int:
    m = getattr(cache, "fi_mode", None)
    if m is not None:
        return int(m)
    return 1 if cache.dtype == torch.float8_e4m3fn else 0


def quant_rows(x: torch.Tensor, mode: int):
    """x [..., hd] -> (stored rows, fp32 scales [...]).  mode 3: packed int4 uint8 [..., hd/2] (byte d = channel d
    in the low nibble, channel d + hd/2 in the high nibble, q = clamp(floor(x / s + 0.5), -7, 7), s = max(amax / 7,
    1e-4)); mode 2: e4m3 of x / s with s = amax / 448."""
    xf = x.float()
    amax = xf.abs().amax(-1)
    if mode == 3:
        sc = (amax / 7.0).clamp_min(1e-4)
        q = torch.floor(xf / sc[..., None] + 0.5).clamp(-7, 7).to(torch.int16)
        half = x.shape[-1] // 2
        packed = (q[..., :half] & 0x0F) | ((q[..., half:] & 0x0F) << 4)
        return packed.to(torch.uint8), sc
    sc = (amax / 448.0).clamp_min(1e-12)
    return (xf / sc[..., None]).to(torch.float8_e4m3fn), sc


def dequant_rows(stored: torch.Tensor, scales: torch.Tensor, mode: int) -> torch.Tensor:
    """Inverse of :func:`quant_rows` -> float32 [..., hd]."""
    if mode == 3:
        b = stored.to(torch.int16)
        lo = ((b & 0x0F) ^ 8) - 8
        hi = ((b >> 4) ^ 8) - 8
        return torch.cat([lo, hi], dim=-1).float() * scales[..., None]
    return stored.float() * scales[..., None]


def reshape_and_cache(k, v, slot_mapping, k_cache, v_cache, k_scale=1.0, v_scale=1.0):
    """k, v: [T, nkv, hd] -> paged cache at slot_mapping (negative slot = skip)."""
    bs = k_cache.shape[2]
    valid = slot_mapping >= 0
    if not bool(valid.any()):
        return
    slots = slot_mapping[valid].long()
    blk, off = slots // bs, slots % bs
    kk, vv = k[valid], v[valid]
    mode = kv_mode(k_cache)
    if mode >= 2:
        for cache, rows in ((k_cache, kk), (v_cache, vv)):
            stored, sc = quant_rows(rows, mode)
            cache[blk, :, off] = stored
            cache.fi_scales[blk, :, off] = sc
        return
    if k_cache.dtype == torch.float8_e4m3fn:
        k_cache[blk, :, off] = fp8_quant(kk, k_scale)
        v_cache[blk, :, off] = fp8_quant(vv, v_scale)
    else:
        k_cache[blk, :, off] = kk.to(k_cache.dtype)
        v_cache[blk, :, off] = vv.to(v_cache.dtype)


def _gather_kv(cache, block_table, n_tokens, scale):
    bs = cache.shape[2]
    nb = (n_tokens + bs - 1) // bs
    mode = kv_mode(cache)
    if mode >= 2:
        idx = block_table[:nb].long()
        blocks = dequant_rows(cache[idx], cache.fi_scales[idx], mode)       # [nb, nkv, bs, hd]
        return blocks.permute(1, 0, 2, 3).reshape(cache.shape[1], nb * bs, blocks.shape[3])[:, :n_tokens]
    blocks = cache[block_table[:nb].long()]  # [nb, nkv, bs, hd]
    x = blocks.permute(1, 0, 2, 3).reshape(cache.shape[1], nb * bs, cache.shape[3])[:, :n_tokens]
    x = x.float()
    if cache.dtype == torch.float8_e4m3fn:
        x = x * scale
    return x  # [nkv, n, hd]


def paged_attention(q, k_cache, v_cache, block_tables, seq_lens, cu_q, nh, nkv, hd, sm_scale,
                    window=0, softcap=0.0, k_scale=1.0, v_scale=1.0, out_dtype=None):
    """Varlen causal attention over the paged cache.  q: [T, >= nh*hd] (first nh*hd columns are the
    query heads); query tokens of sequence b are rows cu_q[b]:cu_q[b+1] and sit at absolute
    positions seq_lens[b]-q_len .. seq_lens[b]-1.  Returns [T, nh*hd]."""
    T = q.shape[0]
    out = torch.zeros(T, nh * hd, dtype=torch.float32, device=q.device)
    B = seq_lens.shape[0]
    g = nh // nkv
    cu = cu_q.tolist()
    sl = seq_lens.tolist()
    for b in range(B):
        q0, q1 = cu[b], cu[b + 1]
        qlen, n = q1 - q0, sl[b]
        if qlen <= 0:
            continue
        qq = q[q0:q1, :nh * hd].float().view(qlen, nh, hd).permute(1, 0, 2)  # [nh, qlen, hd]
        K = _gather_kv(k_cache, block_tables[b], n, k_scale).repeat_interleave(g, dim=0)
        V = _gather_kv(v_cache, block_tables[b], n, v_scale).repeat_interleave(g, dim=0)
        s = torch.einsum("hqd,hkd->hqk", qq, K) * sm_scale
        if softcap and softcap > 0:
            s = softcap * torch.tanh(s / softcap)
        qpos = torch.arange(n - qlen, n, device=q.device)[:, None]
        kpos = torch.arange(n, device=q.device)[None, :]
        mask = kpos > qpos
        if window and window > 0:
            mask = mask | (kpos <= qpos - window)
        s = s.masked_fill(mask[None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("hqk,hkd->hqd", p, V)  # [nh, qlen, hd]
        out[q0:q1] = o.permute(1, 0, 2).reshape(qlen, nh * hd)
    return out.to(out_dtype or q.dtype)


def embedding(ids, table, scale=1.0, vocab_start=0, vocab_end=None):
    vocab_end = table.shape[0] + vocab_start if vocab_end is None else vocab_end
    mine = (ids >= vocab_start) & (ids < vocab_end)
    local = (ids - vocab_start).clamp(0, table.shape[0] - 1)
    out = table[local]
    if scale != 1.0:
        out = (out.float() * scale).to(table.dtype)
    return out * mine[:, None].to(out.dtype)


def act_mul(x, act="silu"):
    d = x.shape[-1] // 2
    return (apply_act(x[..., :d].float(), act) * x[..., d:].float()).to(x.dtype)


def slot_mapping(positions, token_seq, block_tables, block_size):
    seq = token_seq.long().clamp(min=0)
    blk = block_tables[seq, (positions.long().clamp(min=0) // block_size)]
    slots = blk * block_size + positions % block_size
    bad = (blk <= 0) | (token_seq < 0) | (positions < 0)
    return torch.where(bad, torch.full_like(slots, -1), slots).to(torch.int32)


def argmax(logits):
    return torch.argmax(logits.float(), dim=-1)


def default_sm_scale(hd: int) -> float:
    return 1.0 / math.sqrt(hd)
