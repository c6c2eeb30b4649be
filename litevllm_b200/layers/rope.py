"""Rotary-embedding tables.  The kernels consume one fp32 table ``[max_pos, rot_dim] = [cos | sin]``
per distinct (base, scaling) pair; this module builds and caches them, including llama3 / linear /
yarn frequency scaling and Gemma4's proportional partial rotation.
Reference: vllm/model_executor/layers/rotary_embedding/{base,common}.py, gemma4/rope.py:31-194.
"""
from __future__ import annotations

import math

import torch

from ..ops.reference import build_cos_sin

_CACHE: dict[tuple, torch.Tensor] = {}


def scaled_inv_freq(rot_dim: int, base: float, scaling: dict | None) -> tuple[torch.Tensor, float]:
    """-> (inv_freq [rot_dim/2] float64, attention scale factor)."""
    inv = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
    if not scaling:
        return inv, 1.0
    kind = str(scaling.get("rope_type", scaling.get("type", "default"))).lower()
    factor = float(scaling.get("factor", 1.0))
    if kind in ("default", "mrope", "none"):
        return inv, 1.0
    if kind == "linear":
        return inv / factor, 1.0
    if kind == "llama3":
        lo = float(scaling.get("low_freq_factor", 1.0))
        hi = float(scaling.get("high_freq_factor", 4.0))
        orig = float(scaling.get("original_max_position_embeddings", 8192))
        wavelen = 2 * math.pi / inv
        smooth = ((orig / wavelen) - lo) / (hi - lo)
        mid = (1 - smooth) * inv / factor + smooth * inv
        out = torch.where(wavelen > orig / lo, inv / factor, torch.where(wavelen < orig / hi, inv, mid))
        return out, 1.0
    if kind == "yarn":
        orig = float(scaling.get("original_max_position_embeddings", 4096))
        beta_fast = float(scaling.get("beta_fast", 32.0))
        beta_slow = float(scaling.get("beta_slow", 1.0))

        def corr_dim(n_rot):
            return rot_dim * math.log(orig / (n_rot * 2 * math.pi)) / (2 * math.log(base))
        low = max(math.floor(corr_dim(beta_fast)), 0)
        high = min(math.ceil(corr_dim(beta_slow)), rot_dim // 2 - 1)
        ramp = ((torch.arange(rot_dim // 2, dtype=torch.float64) - low) / max(high - low, 1e-3)).clamp(0, 1)
        mask = 1.0 - ramp
        out = inv / factor * (1 - mask) + inv * mask
        mscale = float(scaling.get("mscale", 1.0))
        attn = (0.1 * mscale * math.log(factor) + 1.0) if factor > 1 else 1.0
        return out, attn
    raise ValueError(f"unsupported rope scaling type {kind!r}")


def get_cos_sin(rot_dim: int, max_pos: int, base: float, scaling: dict | None, device,
                attn_factor_into_table: bool = False) -> torch.Tensor:
    key = (rot_dim, max_pos, float(base), repr(sorted((scaling or {}).items())), str(device))
    tab = _CACHE.get(key)
    if tab is None:
        inv, attn = scaled_inv_freq(rot_dim, base, scaling)
        tab = build_cos_sin(rot_dim, max_pos, base, inv_freq=inv)
        if attn_factor_into_table and attn != 1.0:
            tab = tab * attn
        tab = tab.to(device)
        _CACHE[key] = tab
    return tab


def clear_cache() -> None:
    _CACHE.clear()
