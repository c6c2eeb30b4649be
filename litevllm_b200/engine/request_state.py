"""Per-request runtime record (reference: vllm/engine/request_state.py:12-74).

``seq_len`` counts tokens whose KV is already in the cache.  While ``is_prefill`` the request
consumes prompt chunks; afterwards each step feeds the last sampled token at position ``seq_len``.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any

import torch

from ..sampling_params import SamplingParams


@dataclass
class RequestState:
    request_id: str
    prompt: str | None
    prompt_token_ids: list[int]
    sampling_params: SamplingParams
    arrival_time: float = field(default_factory=time.monotonic)
    admitted_time: float | None = None
    first_token_time: float | None = None
    finished_time: float | None = None
    slot_idx: int = -1
    seq_len: int = 0
    is_prefill: bool = True
    prefill_deferrals: int = 0
    generated_ids: list[int] = field(default_factory=list)
    finished: bool = False
    finish_reason: str | None = None
    eos_token_ids: frozenset[int] = frozenset()
    rng: torch.Generator | None = None
    lora_request: Any = None
    multi_modal_data: dict | None = None
    multimodal_inputs: dict | None = None
    structured_output_constraint: Any = None
    # device-resident sampling (greedy fast path): tokens not yet copied to the host
    last_token_tensor: torch.Tensor | None = None
    pending_token_tensors: list = field(default_factory=list)
    # recurrent state of linear-attention layers (Qwen3.5), carried between steps
    linear_attn_carry: Any = None
    linear_conv_carry: Any = None
    # rotary position of token index i is i + rope_delta (multimodal rotary: an image advances the position
    # by the larger side of its grid, not by its token count; 0 for text-only requests)
    rope_delta: int = 0
    prefix_cache_hit_tokens: int = 0
    cached_first_logits: torch.Tensor | None = None

    @property
    def prompt_len(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def remaining_prefill(self) -> int:
        return max(0, self.prompt_len - self.seq_len) if self.is_prefill else 0

    @property
    def num_generated(self) -> int:
        return len(self.generated_ids) + len(self.pending_token_tensors)

    @property
    def total_len(self) -> int:
        return self.prompt_len + self.num_generated

    def last_token(self) -> int:
        return self.generated_ids[-1] if self.generated_ids else self.prompt_token_ids[-1]
