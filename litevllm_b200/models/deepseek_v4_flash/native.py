"""Fused per-token kernels of the DeepSeek-V4-Flash layer (``csrc/deepseek/dsv4_token_kernels.cu``) with the
PyTorch formulation of each as the CPU path and the oracle of the GPU tests.  All tensors are fp32.
Reference: vllm/model_executor/models/deepseek_v4_flash/hyper_connection.py:16-129, attention.py:141-197,
665-760, ops.py."""
from __future__ import annotations

import torch

from ... import ops
from ...ops import _lib
from .attention import CompressorState, compressor_step
from .hyper_connection import HyperConnectionState, hyper_connection_post, hyper_connection_pre
from .ops import fp8_kv_qat, q8_k_roundtrip


def _gpu(*ts) -> bool:
    for t in ts:
        if t is not None and not (t.is_cuda and t.dtype == torch.float32):
            return False
    return True


_lib_handle = None


def _k():
    global _lib_handle
    if _lib_handle is None:
        _lib_handle = _lib.kernels()
    return _lib_handle


def _call(rc: int, what: str) -> None:
    if rc != 0:
        _lib.check(rc, what)
    ops._launches[0] += 1


def _p(t):
    return None if t is None else t.data_ptr()


_s = ops._stream


def rms(x: torch.Tensor, w: torch.Tensor | None, eps: float) -> torch.Tensor:
    y = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w.float()


def rotate_tail(x: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """Rotary embedding on the last ``2 * len(inv_freq)`` channels of ``[T, ..., D]`` at positions ``pos`` ``[T]``;
    adjacent channels (2i, 2i+1) form a pair.  ``inverse`` rotates back."""
    rot = 2 * inv_freq.numel()
    if rot == 0:
        return x
    ang = (-pos if inverse else pos).float().reshape(-1, *([1] * (x.dim() - 1))) * inv_freq
    c, s = torch.cos(ang), torch.sin(ang)
    pairs = x[..., -rot:].unflatten(-1, (rot // 2, 2))
    a, b = pairs[..., 0], pairs[..., 1]
    tail = torch.stack((a * c - b * s, a * s + b * c), dim=-1).flatten(-2)
    return torch.cat([x[..., :-rot], tail], dim=-1)


def norm_rope(x: torch.Tensor, w: torch.Tensor | None, inv_freq: torch.Tensor | None, pos: torch.Tensor | None,
              eps: float, norm: bool = True, inverse: bool = False, fp8: bool = False) -> torch.Tensor:
    """``x`` ``[T, D]`` or ``[T, heads, D]``: optional RMS norm (weight ``w`` or none), optional rotary on the tail
    channels at ``pos`` ``[T]``, optional FP8 round trip of the non-rotary channels.  One kernel on a GPU."""
    D = x.shape[-1]
    rot = 0 if inv_freq is None else 2 * inv_freq.numel()
    if _gpu(x, w, inv_freq) and D <= 12288:
        xc = x.contiguous()
        rows = xc.numel() // D
        y = torch.empty_like(xc)
        rc = _k().fi_dsv4_norm_rope(_p(xc), _p(w), _p(inv_freq), _p(pos), rows, rows // xc.shape[0], D, rot,
                                    int(norm), int(inverse), int(fp8), float(eps), _p(y), _s())
        _call(rc, "fi_dsv4_norm_rope")
        return y
    y = rms(x, w, eps) if norm else x.float()
    if rot:
        y = rotate_tail(y, pos, inv_freq, inverse)
    if fp8:
        y = fp8_kv_qat(y, D, rot)
    return y


def hc_pre(streams: torch.Tensor, fn_weight: torch.Tensor, base: torch.Tensor, scale: torch.Tensor,
           eps: float, iterations: int = 20) -> HyperConnectionState:
    """``fn_weight`` ``[hc * H, 2 hc + hc^2]``.  On a GPU: one GEMM for the mixing logits and one kernel for the
    rest (RMS scale, gates, Sinkhorn, mixed input)."""
    T, hc, H = streams.shape
    if _gpu(streams, fn_weight, base, scale) and hc <= 8 and fn_weight.shape[0] == hc * H:
        st = streams.contiguous()
        raw = st.view(T, hc * H) @ fn_weight
        mixed = torch.empty(T, H, dtype=torch.float32, device=st.device)
        post = torch.empty(T, hc, dtype=torch.float32, device=st.device)
        combine = torch.empty(T, hc, hc, dtype=torch.float32, device=st.device)
        rc = _k().fi_dsv4_hc_pre(_p(st), _p(raw), _p(base), _p(scale), T, hc, H, float(eps), int(iterations),
                                 _p(mixed), _p(post), _p(combine), _s())
        _call(rc, "fi_dsv4_hc_pre")
        return HyperConnectionState(mixed, post, combine)
    return hyper_connection_pre(streams, fn_weight, base, scale, iterations, eps)


def hc_post(output: torch.Tensor, streams: torch.Tensor, state: HyperConnectionState) -> torch.Tensor:
    T, hc, H = streams.shape
    if _gpu(output, streams, state.post, state.combine) and hc <= 8:
        nxt = torch.empty_like(streams)
        rc = _k().fi_dsv4_hc_post(_p(output.contiguous()), _p(streams.contiguous()), _p(state.post), _p(state.combine),
                                  T, hc, H, _p(nxt), _s())
        _call(rc, "fi_dsv4_hc_post")
        return nxt
    return hyper_connection_post(output, streams, state)


def hc_collapse(streams: torch.Tensor, fn_weight: torch.Tensor, base: torch.Tensor, scale: torch.Tensor,
                eps: float) -> torch.Tensor:
    """Sigmoid-gated sum of the streams after the last layer; ``fn_weight`` ``[hc, hc * H]``."""
    T, hc, H = streams.shape
    flat = streams.reshape(T, hc * H)
    if _gpu(streams, fn_weight, base, scale) and hc <= 8:
        raw = flat @ fn_weight.t()
        out = torch.empty(T, H, dtype=torch.float32, device=streams.device)
        rc = _k().fi_dsv4_hc_collapse(_p(streams.contiguous()), _p(raw), _p(base), _p(scale), T, hc, H, float(eps),
                                      _p(out), _s())
        _call(rc, "fi_dsv4_hc_collapse")
        return out
    flat = flat.float() * torch.rsqrt(flat.float().pow(2).mean(-1, keepdim=True) + eps)
    gains = torch.sigmoid((flat @ fn_weight.float().t()) * scale.float()[0] + base.float()) + 1e-6
    return (gains.unsqueeze(-1) * streams.float()).sum(1)


def compressor_step_(state: CompressorState, kv_cur: torch.Tensor, score_cur: torch.Tensor, ape: torch.Tensor,
                     token_idx: int, head_dim: int, ratio: int) -> torch.Tensor | None:
    """Feed one token into ``state`` (updated in place); returns the emitted row every ``ratio`` tokens."""
    emits = (token_idx + 1) % ratio == 0
    width = (2 if ratio == 4 else 1) * head_dim
    if _gpu(state.kv, state.score, kv_cur, score_cur, ape):
        sp, sc = (ape.stride(1), ape.stride(0)) if ape.shape == (width, ratio) else (ape.stride(0), ape.stride(1))
        out = torch.empty(head_dim, dtype=torch.float32, device=kv_cur.device) if emits else state.kv
        rc = _k().fi_dsv4_compressor_step(_p(state.kv), _p(state.score), _p(kv_cur.contiguous()),
                                          _p(score_cur.contiguous()), _p(ape), sp, sc, int(token_idx), int(ratio),
                                          int(head_dim), _p(out), _s())
        _call(rc, "fi_dsv4_compressor_step")
        return out if emits else None
    new, emitted = compressor_step(state, kv_cur, score_cur, ape, token_idx, head_dim, ratio)
    state.kv, state.score = new.kv, new.score
    return emitted


def compressor_run_(state: CompressorState, kv_run: torch.Tensor, score_run: torch.Tensor, ape: torch.Tensor,
                    p0: int, head_dim: int, ratio: int) -> torch.Tensor:
    """``n`` consecutive tokens starting at position ``p0`` into ``state`` (updated in place); returns the rows of
    every window the run completes, ``[n_emit, head_dim]``.  An emission only depends on the tokens of its own
    window (and of the window before it for ratio 4), so all windows of the run are pooled at once from the
    carried-in rows followed by the run's rows."""
    n = kv_run.shape[0]
    coff = 2 if ratio == 4 else 1
    width = coff * head_dim
    dev = kv_run.device
    ape_rows = (ape.t() if ape.shape == (width, ratio) else ape).float()
    slots = (p0 + torch.arange(n, device=dev)) % ratio
    sc_run = score_run.float() + ape_rows[slots]
    kv_run = kv_run.float()
    part = p0 % ratio                 # tokens already in the current window
    base = p0 - part                  # position where the current window starts
    if ratio == 4:                    # rows 0..3: previous window, rows 4..: current window
        hist_kv = torch.cat([state.kv[:4], state.kv[4:4 + part], kv_run])
        hist_sc = torch.cat([state.score[:4], state.score[4:4 + part], sc_run])
        origin = base - 4
    else:
        hist_kv = torch.cat([state.kv[:part], kv_run])
        hist_sc = torch.cat([state.score[:part], sc_run])
        origin = base
    end = p0 + n
    n_emit = (end - base) // ratio
    emitted = kv_run.new_zeros(0, head_dim)
    if n_emit > 0:
        cur = (base - origin + ratio * torch.arange(n_emit, device=dev))[:, None] + torch.arange(ratio, device=dev)[None]
        if ratio == 4:
            prev = cur - 4
            sc = torch.cat([hist_sc[prev][:, :, :head_dim], hist_sc[cur][:, :, head_dim:]], 1)
            vals = torch.cat([hist_kv[prev][:, :, :head_dim], hist_kv[cur][:, :, head_dim:]], 1)
        else:
            sc, vals = hist_sc[cur][:, :, :head_dim], hist_kv[cur][:, :, :head_dim]
        emitted = (torch.nan_to_num(torch.softmax(sc, dim=1)) * vals).sum(1)
    new_part = end % ratio
    i0 = end - new_part - origin
    if ratio == 4:
        if end - new_part > base:     # a window was completed: it becomes the previous window
            state.kv[:4] = hist_kv[i0 - 4:i0]
            state.score[:4] = hist_sc[i0 - 4:i0]
        state.kv[4:4 + new_part] = hist_kv[i0:i0 + new_part]
        state.score[4:4 + new_part] = hist_sc[i0:i0 + new_part]
    else:
        state.kv[:new_part] = hist_kv[i0:i0 + new_part]
        state.score[:new_part] = hist_sc[i0:i0 + new_part]
    return emitted


def q8k(x: torch.Tensor) -> torch.Tensor:
    if _gpu(x) and x.numel() % 256 == 0 and x.shape[-1] % 256 == 0:
        xc = x.contiguous()
        y = torch.empty_like(xc)
        _call(_k().fi_dsv4_q8k_roundtrip(_p(xc), _p(y), xc.numel(), _s()), "fi_dsv4_q8k_roundtrip")
        return y
    return q8_k_roundtrip(x)
