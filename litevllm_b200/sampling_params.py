"""Sampling parameters (field names and defaults follow vllm/sampling_params.py:5-64 of the
reference so user code carries over unchanged)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass
class StructuredOutputsParams:
    json: Any = None            # JSON schema (dict or str)
    regex: str | None = None
    grammar: str | None = None  # EBNF
    structural_tag: str | None = None
    json_object: bool | None = None
    choice: list[str] | None = None

    def kind(self) -> str | None:
        for name in ("json", "regex", "grammar", "choice", "structural_tag"):
            if getattr(self, name) is not None:
                return name
        if self.json_object:
            return "json_object"
        return None


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repetition_penalty: float = 1.0
    max_tokens: int | None = 16
    min_tokens: int = 0
    stop: list[str] = field(default_factory=list)
    stop_token_ids: list[int] = field(default_factory=list)
    skip_special_tokens: bool = True
    spaces_between_special_tokens: bool = True
    ignore_eos: bool = False
    n: int = 1
    logprobs: int | None = None
    prompt_logprobs: int | None = None
    seed: int | None = None
    include_stop_str_in_output: bool = False
    logit_bias: dict[int, float] | None = None
    truncate_prompt_tokens: int | None = None
    structured_outputs: StructuredOutputsParams | None = None
    detokenize: bool = True
    output_kind: str = "final_only"

    def __post_init__(self):
        if isinstance(self.stop, str):
            self.stop = [self.stop]
        if self.stop is None:
            self.stop = []
        if self.stop_token_ids is None:
            self.stop_token_ids = []
        if isinstance(self.structured_outputs, dict):
            self.structured_outputs = StructuredOutputsParams(**self.structured_outputs)
        if self.temperature < 0:
            raise ValueError("temperature must be non-negative")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < -1 or self.top_k == 0:
            raise ValueError("top_k must be -1 (disabled) or >= 1")
        if self.max_tokens is not None and self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if self.min_tokens < 0:
            raise ValueError("min_tokens must be >= 0")
        if self.n < 1:
            raise ValueError("n must be >= 1")

    @property
    def is_greedy(self) -> bool:
        return self.temperature <= 1e-6

    @property
    def has_penalties(self) -> bool:
        return (self.frequency_penalty != 0.0 or self.presence_penalty != 0.0
                or self.repetition_penalty != 1.0)

    def clone(self) -> "SamplingParams":
        import copy
        return copy.deepcopy(self)
