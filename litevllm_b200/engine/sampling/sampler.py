"""Batched token sampling.

All-greedy batches take one arg-max kernel.  Otherwise: temperature, then on the descending-sorted
row top-k, top-p (the first token that crosses the threshold is kept) and min-p masks, softmax, and
one multinomial draw per row with the request's own generator.  Rows whose probability mass is
zero or NaN fall back to the arg-max of the original logits.
Reference: vllm/engine/sampling/sampler.py:9-114 (min_p is accepted but ignored there).
"""
from __future__ import annotations

import torch

from ... import ops
from ..request_state import RequestState


class Sampler:
    def __init__(self):
        import os
        # the native kernel (threshold selection instead of a sort); FI_NATIVE_SAMPLER=0 keeps the PyTorch form
        self.native = os.environ.get("FI_NATIVE_SAMPLER", "1") != "0"

    def _sample_native(self, logits: torch.Tensor, reqs: list[RequestState], sps) -> torch.Tensor:
        """One kernel for the whole batch: per-row parameters go up in one small copy, each sampled row
        draws one uniform number from its request's own generator (greedy rows pass temperature 0)."""
        n = logits.shape[0]
        dev = logits.device
        host = torch.empty(4, n, dtype=torch.float32)
        for i, sp in enumerate(sps):
            host[0, i] = 0.0 if sp.is_greedy else max(sp.temperature, 1e-6)
            host[1, i] = float(sp.top_k) if sp.top_k and sp.top_k > 0 else 0.0
            host[2, i] = sp.top_p
            host[3, i] = sp.min_p
        par = host.to(dev, non_blocking=True)
        uni = torch.zeros(n, dtype=torch.float32, device=dev)
        for i, st in enumerate(reqs):
            if not sps[i].is_greedy:
                uni[i:i + 1] = torch.rand(1, generator=st.rng, device=dev, dtype=torch.float32)
        return ops.sample(logits, par[0], par[1].to(torch.int32), par[2], par[3], uni)

    def sample(self, logits: torch.Tensor, reqs: list[RequestState]) -> torch.Tensor:
        """logits [n, V] float32 -> int64 [n] on the same device."""
        sps = [st.sampling_params for st in reqs]
        if all(sp.is_greedy for sp in sps):
            return ops.argmax(logits)
        n, V = logits.shape
        dev = logits.device
        if logits.is_cuda and logits.dtype == torch.float32 and self.native:
            return self._sample_native(logits, reqs, sps)
        greedy_tokens = ops.argmax(logits)
        temps = torch.tensor([max(sp.temperature, 1e-6) for sp in sps], device=dev, dtype=torch.float32)[:, None]
        scaled = logits / temps
        sorted_logits, sorted_idx = torch.sort(scaled, dim=-1, descending=True)
        ranks = torch.arange(V, device=dev)[None, :]
        top_k = torch.tensor([sp.top_k if sp.top_k and sp.top_k > 0 else V for sp in sps], device=dev)[:, None]
        mask = ranks >= top_k
        probs_sorted = torch.softmax(sorted_logits.masked_fill(mask, float("-inf")), dim=-1)
        top_p = torch.tensor([sp.top_p for sp in sps], device=dev, dtype=torch.float32)[:, None]
        cum = probs_sorted.cumsum(dim=-1)
        # keep a token if the mass *before* it is still below top_p (first crossing token survives)
        mask |= (cum - probs_sorted) >= top_p
        min_p = torch.tensor([sp.min_p for sp in sps], device=dev, dtype=torch.float32)[:, None]
        mask |= probs_sorted < (min_p * probs_sorted[:, :1])
        mask[:, 0] = False
        final = torch.softmax(sorted_logits.masked_fill(mask, float("-inf")), dim=-1)
        out = torch.empty(n, dtype=torch.long, device=dev)
        for i, st in enumerate(reqs):
            if sps[i].is_greedy:
                out[i] = greedy_tokens[i]
                continue
            row = final[i]
            if not bool(torch.isfinite(row).all()) or float(row.sum()) <= 0.0:
                out[i] = greedy_tokens[i]
                continue
            pick = torch.multinomial(row, 1, generator=st.rng)
            out[i] = sorted_idx[i, pick[0]]
        return out
