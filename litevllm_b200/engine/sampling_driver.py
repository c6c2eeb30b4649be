"""Glue between executor logits and sampled token ids (reference: vllm/engine/sampling_driver.py:
14-251).  ``sample_device`` leaves the tokens on the device (greedy fast path); ``sample_batch_tokens``
returns Python ints with a single device-to-host copy for the whole batch."""
from __future__ import annotations

import torch

from .request_state import RequestState
from .sampling.penalty_encoder import PenaltyEncoder
from .sampling.sampler import Sampler


class SamplingDriver:
    def __init__(self, vocab_size: int):
        self.encoder = PenaltyEncoder(vocab_size)
        self.sampler = Sampler()
        self.vocab_size = vocab_size

    def sample_device(self, logits: torch.Tensor, reqs: list[RequestState]) -> torch.Tensor:
        logits = logits[: len(reqs)]
        if logits.dtype != torch.float32:
            logits = logits.float()
        if self.encoder.needs_encoding(reqs):
            logits = self.encoder.encode(logits.clone() if logits.is_cuda else logits, reqs)
        return self.sampler.sample(logits, reqs)

    def sample_batch_tokens(self, logits: torch.Tensor, reqs: list[RequestState]) -> list[int]:
        return self.sample_device(logits, reqs).tolist()

    @staticmethod
    def can_stay_on_device(st: RequestState, policy) -> bool:
        """Greedy, penalty-free, unconstrained requests whose stop condition is max_tokens only."""
        sp = st.sampling_params
        if not policy.gpu_greedy_sampling or not sp.is_greedy or sp.has_penalties or sp.logit_bias:
            return False
        if st.structured_output_constraint is not None or sp.stop:
            return False
        if policy.gpu_greedy_max_tokens_only and st.eos_token_ids and not sp.ignore_eos:
            return False
        return True
