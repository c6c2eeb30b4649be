"""Logit adjustments before sampling, vectorised over the batch.

* repetition penalty (multiplicative, generated tokens only): positive logits are divided, negative
  multiplied;
* frequency / presence penalties (additive, by generated-token counts);
* EOS masking while ``min_tokens`` is not reached or when ``ignore_eos`` is set;
* ``logit_bias``;
* structured-output token masks (per row, through the request's constraint object).
Reference: vllm/engine/sampling/penalty_encoder.py:13-308 (penalties apply to generated tokens only,
:146-149,193-196).
"""
from __future__ import annotations

import torch

from ..request_state import RequestState


class PenaltyEncoder:
    def __init__(self, vocab_size: int):
        self.vocab_size = vocab_size

    @staticmethod
    def needs_encoding(reqs: list[RequestState]) -> bool:
        for st in reqs:
            sp = st.sampling_params
            if sp.has_penalties or sp.logit_bias or st.structured_output_constraint is not None:
                return True
            if st.eos_token_ids and (sp.ignore_eos or len(st.generated_ids) < sp.min_tokens):
                return True
        return False

    def encode(self, logits: torch.Tensor, reqs: list[RequestState]) -> torch.Tensor:
        """logits: [n, V] float32, modified in place and returned."""
        n, V = logits.shape
        dev = logits.device
        # ---- penalties from generated-token counts
        pen_rows = [i for i, st in enumerate(reqs) if st.sampling_params.has_penalties and st.generated_ids]
        if pen_rows:
            rows, toks = [], []
            for i in pen_rows:
                g = reqs[i].generated_ids
                rows.extend([i] * len(g))
                toks.extend(g)
            r = torch.tensor(rows, dtype=torch.long, device=dev)
            t = torch.tensor(toks, dtype=torch.long, device=dev).clamp_(0, V - 1)
            counts = torch.zeros(n, V, dtype=torch.float32, device=dev)
            counts.index_put_((r, t), torch.ones_like(t, dtype=torch.float32), accumulate=True)
            seen = counts > 0
            rep = torch.tensor([reqs[i].sampling_params.repetition_penalty for i in range(n)], device=dev)[:, None]
            freq = torch.tensor([reqs[i].sampling_params.frequency_penalty for i in range(n)], device=dev)[:, None]
            pres = torch.tensor([reqs[i].sampling_params.presence_penalty for i in range(n)], device=dev)[:, None]
            rep = torch.where(rep > 1.0, rep, torch.ones_like(rep))
            scaled = torch.where(logits > 0, logits / rep, logits * rep)
            logits.copy_(torch.where(seen, scaled, logits))
            logits.sub_(freq * counts).sub_(pres * seen.float())
        # ---- EOS masking / logit bias / structured outputs
        for i, st in enumerate(reqs):
            sp = st.sampling_params
            if st.eos_token_ids and (sp.ignore_eos or len(st.generated_ids) < sp.min_tokens):
                idx = torch.tensor([e for e in st.eos_token_ids if 0 <= e < V], dtype=torch.long, device=dev)
                if idx.numel():
                    logits[i, idx] = float("-inf")
            if sp.logit_bias:
                keys = [int(k) for k in sp.logit_bias if 0 <= int(k) < V]
                if keys:
                    vals = torch.tensor([float(sp.logit_bias[k]) if k in sp.logit_bias else float(sp.logit_bias[str(k)])
                                         for k in keys], device=dev)
                    logits[i, torch.tensor(keys, dtype=torch.long, device=dev)] += vals
            c = st.structured_output_constraint
            if c is not None:
                c.apply_mask(logits[i])
        return logits
