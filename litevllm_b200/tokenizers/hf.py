"""Hugging Face tokenizers, loaded once per (path, revision) and given cheap cached properties
(``len(tokenizer)``, special ids) that the per-token paths read.  Reference: vllm/tokenizers/hf.py."""
from __future__ import annotations

import threading

_lock = threading.Lock()
_cache: dict[tuple, object] = {}


def get_cached_tokenizer(path: str, trust_remote_code: bool = False, revision: str | None = None,
                         vocab_size: int = 32000):
    key = (str(path), bool(trust_remote_code), revision)
    with _lock:
        tok = _cache.get(key)
        if tok is None:
            from ..loaders import get_tokenizer as _load
            tok = _load(path, trust_remote_code=trust_remote_code, revision=revision, vocab_size=vocab_size)
            try:                                   # freeze the values the hot path asks for repeatedly
                n = len(tok)
                specials = set(getattr(tok, "all_special_ids", []) or [])
                tok._fi_len, tok._fi_special_ids = n, specials
            except Exception:
                pass
            _cache[key] = tok
        return tok


def clear_cache() -> None:
    with _lock:
        _cache.clear()
