"""Incremental detokenisation: text deltas for a growing token list without re-decoding the whole
sequence and without emitting half of a multi-byte character.
Reference: vllm/tokenizers/detokenizer_utils.py (helper, not on the engine's main path, which
decodes lazily in the output pipeline)."""
from __future__ import annotations

REPLACEMENT = "�"


def detokenize_incrementally(tokenizer, all_ids: list[int], prefix_offset: int, read_offset: int,
                             skip_special_tokens: bool = True) -> tuple[str, int, int]:
    """Returns (new text, new prefix offset, new read offset).  Decodes a short window
    ``[prefix_offset:]`` twice (with and without the unread tail) and emits the difference once it
    no longer ends in an incomplete UTF-8 sequence."""
    prefix_text = tokenizer.decode(all_ids[prefix_offset:read_offset], skip_special_tokens=skip_special_tokens)
    full_text = tokenizer.decode(all_ids[prefix_offset:], skip_special_tokens=skip_special_tokens)
    if len(full_text) > len(prefix_text) and not full_text.endswith(REPLACEMENT):
        return full_text[len(prefix_text):], read_offset, len(all_ids)
    return "", prefix_offset, read_offset


class IncrementalDetokenizer:
    """Stateful wrapper: ``push(token_id) -> text delta``."""

    def __init__(self, tokenizer, prompt_ids: list[int] | None = None, skip_special_tokens: bool = True,
                 context: int = 6):
        self.tokenizer, self.skip = tokenizer, skip_special_tokens
        self.ids = list(prompt_ids or [])
        self.prefix_offset = max(len(self.ids) - context, 0)
        self.read_offset = len(self.ids)
        self.text = ""

    def push(self, token_id: int) -> str:
        self.ids.append(int(token_id))
        delta, self.prefix_offset, self.read_offset = detokenize_incrementally(
            self.tokenizer, self.ids, self.prefix_offset, self.read_offset, self.skip)
        self.text += delta
        return delta
