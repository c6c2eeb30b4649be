"""Name -> tokenizer factory registry (reference: vllm/tokenizers/registry.py).  ``"hf"`` is the
default; tests and embedders register their own."""
from __future__ import annotations

from typing import Callable

from .hf import get_cached_tokenizer


class TokenizerRegistry:
    _factories: dict[str, Callable] = {"hf": get_cached_tokenizer}

    @classmethod
    def register(cls, name: str, factory: Callable) -> None:
        cls._factories[name] = factory

    @classmethod
    def get(cls, name: str) -> Callable:
        if name not in cls._factories:
            raise KeyError(f"unknown tokenizer mode {name!r}; registered: {sorted(cls._factories)}")
        return cls._factories[name]


def get_tokenizer(path: str, tokenizer_mode: str = "hf", **kw):
    return TokenizerRegistry.get(tokenizer_mode)(path, **kw)
