"""Request outputs.  ``CompletionOutput.text`` is decoded lazily the first time it is read, so
streaming intermediate outputs cost nothing unless the consumer looks at the text
(reference: vllm/outputs.py:6-81)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable


class CompletionOutput:
    __slots__ = ("index", "token_ids", "cumulative_logprob", "finish_reason", "_text", "_decode")

    def __init__(self, index: int, token_ids: list[int], text: str | None = None,
                 decode: Callable[[list[int]], str] | None = None, cumulative_logprob: float = 0.0,
                 finish_reason: str | None = None):
        self.index = index
        self.token_ids = token_ids
        self.cumulative_logprob = cumulative_logprob
        self.finish_reason = finish_reason
        self._text = text
        self._decode = decode

    @property
    def text(self) -> str:
        if self._text is None:
            self._text = self._decode(self.token_ids) if self._decode is not None else ""
        return self._text

    @text.setter
    def text(self, value: str) -> None:
        self._text = value

    def finished(self) -> bool:
        return self.finish_reason is not None

    # An output that leaves its process (data-parallel replicas hand theirs to the caller's rank) carries
    # its text, not the tokenizer closure that would have produced it.
    def __getstate__(self):
        return {"index": self.index, "token_ids": self.token_ids, "cumulative_logprob": self.cumulative_logprob,
                "finish_reason": self.finish_reason, "_text": self.text, "_decode": None}

    def __setstate__(self, state):
        for k, v in state.items():
            setattr(self, k, v)

    def __repr__(self) -> str:
        return (f"CompletionOutput(index={self.index}, n_tokens={len(self.token_ids)}, "
                f"finish_reason={self.finish_reason!r})")


@dataclass
class RequestOutput:
    request_id: str
    prompt: str | None
    prompt_token_ids: list[int]
    outputs: list[CompletionOutput]
    finished: bool = False
    finish_reason: str | None = None
    metrics: dict[str, Any] = field(default_factory=dict)


@dataclass
class PoolingOutput:
    data: Any = None


@dataclass
class PoolingRequestOutput:
    request_id: str
    outputs: PoolingOutput
    prompt_token_ids: list[int]
    finished: bool = True
