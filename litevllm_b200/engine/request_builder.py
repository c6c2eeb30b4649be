"""Builds a :class:`RequestState` from user input: prompt normalisation and tokenisation, token
caps, length checks, seeded generator, structured-output constraint.
Reference: vllm/engine/request_builder.py:15-184 (which always re-tokenises; token-id prompts are
taken as they are here)."""
from __future__ import annotations

import time

import torch

from ..inputs import normalize_prompt
from ..sampling_params import SamplingParams
from .errors import InvalidRequestError
from .request_state import RequestState
from .sampling.utils import collect_eos_ids


class LiteRequestBuilder:
    def __init__(self, tokenizer, max_model_len: int, vocab_size: int, hf_eos_ids, device: torch.device,
                 max_tokens_cap: int | None = None, default_min_new_tokens: int = 0,
                 structured_factory=None, multimodal=None, chunked_prefill: bool = True):
        self.tokenizer = tokenizer
        self.max_model_len = max_model_len
        self.vocab_size = vocab_size
        self.hf_eos_ids = list(hf_eos_ids or [])
        self.device = device
        self.max_tokens_cap = max_tokens_cap
        self.default_min_new_tokens = default_min_new_tokens
        self.structured_factory = structured_factory
        self.multimodal = multimodal
        self.chunked_prefill = chunked_prefill

    def build(self, request_id: str, prompt, sampling_params: SamplingParams | None,
              lora_request=None, multi_modal_data=None) -> RequestState:
        sp = (sampling_params or SamplingParams()).clone()
        if sp.n != 1:
            raise InvalidRequestError("n > 1 is not supported")
        text, ids, mm = normalize_prompt(prompt)
        mm = multi_modal_data or mm
        mm_inputs = None
        if mm and self.multimodal is not None:
            text, ids, mm_inputs = self.multimodal.expand_prompt(text, ids, mm, self.tokenizer)
        if ids is None:
            if self.tokenizer is None:
                raise InvalidRequestError("text prompt given but no tokenizer is loaded")
            ids = list(self.tokenizer.encode(text))
        if not ids:
            raise InvalidRequestError("empty prompt")
        if sp.truncate_prompt_tokens:
            ids = ids[-int(sp.truncate_prompt_tokens):]
        bad = [t for t in (min(ids), max(ids)) if t < 0 or t >= self.vocab_size]
        if bad:
            raise InvalidRequestError(f"prompt token id {bad[0]} outside the vocabulary [0, {self.vocab_size})")
        if sp.max_tokens is None:
            sp.max_tokens = max(1, self.max_model_len - len(ids))
        if self.max_tokens_cap is not None:
            sp.max_tokens = min(sp.max_tokens, self.max_tokens_cap)
        if sp.min_tokens == 0 and self.default_min_new_tokens:
            sp.min_tokens = min(self.default_min_new_tokens, sp.max_tokens)
        sp.min_tokens = min(sp.min_tokens, sp.max_tokens)
        if len(ids) + sp.max_tokens > self.max_model_len:
            raise InvalidRequestError(
                f"prompt ({len(ids)} tokens) + max_tokens ({sp.max_tokens}) exceeds max_model_len "
                f"({self.max_model_len})")
        rng = None
        if not sp.is_greedy:
            rng = torch.Generator(device=self.device)
            if sp.seed is not None:
                rng.manual_seed(int(sp.seed))
            else:
                rng.seed()
        constraint = None
        if sp.structured_outputs is not None and sp.structured_outputs.kind() is not None:
            if self.structured_factory is None:
                raise InvalidRequestError("structured outputs are not available in this engine build")
            constraint = self.structured_factory(sp.structured_outputs)
        return RequestState(
            request_id=request_id, prompt=text, prompt_token_ids=ids, sampling_params=sp,
            arrival_time=time.monotonic(), eos_token_ids=collect_eos_ids(self.tokenizer, self.hf_eos_ids, sp),
            rng=rng, lora_request=lora_request, multi_modal_data=mm, multimodal_inputs=mm_inputs,
            structured_output_constraint=constraint,
            rope_delta=int((mm_inputs or {}).get("rope_delta", 0)))
