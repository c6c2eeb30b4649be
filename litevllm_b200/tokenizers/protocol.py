"""What the engine needs from a tokenizer (reference: vllm/tokenizers/protocol.py)."""
from __future__ import annotations

from typing import Protocol, runtime_checkable


@runtime_checkable
class TokenizerLike(Protocol):
    eos_token_id: int | None
    bos_token_id: int | None

    def encode(self, text: str, add_special_tokens: bool = True) -> list[int]: ...

    def decode(self, ids, skip_special_tokens: bool = True) -> str: ...

    def __len__(self) -> int: ...
