"""Prompt input types (reference: vllm/inputs/data.py:9-24).  Unlike the reference, token-id prompts
are forwarded natively instead of being re-tokenised."""
from __future__ import annotations

from typing import Any, TypedDict, Union


class TextPrompt(TypedDict, total=False):
    prompt: str
    multi_modal_data: dict[str, Any]


class TokensPrompt(TypedDict, total=False):
    prompt_token_ids: list[int]
    prompt: str
    multi_modal_data: dict[str, Any]


class EmbedsPrompt(TypedDict, total=False):
    prompt_embeds: Any


PromptType = Union[str, TextPrompt, TokensPrompt, list]


def normalize_prompt(prompt: PromptType) -> tuple[str | None, list[int] | None, dict | None]:
    """-> (text, token_ids, multi_modal_data)."""
    if isinstance(prompt, str):
        return prompt, None, None
    if isinstance(prompt, dict):
        if "prompt_token_ids" in prompt:
            return prompt.get("prompt"), [int(t) for t in prompt["prompt_token_ids"]], prompt.get("multi_modal_data")
        if "prompt" in prompt:
            return prompt["prompt"], None, prompt.get("multi_modal_data")
        raise ValueError("prompt dict needs 'prompt' or 'prompt_token_ids'")
    if isinstance(prompt, (list, tuple)) and all(isinstance(t, int) for t in prompt):
        return None, [int(t) for t in prompt], None
    raise TypeError(f"unsupported prompt type {type(prompt).__name__}")
