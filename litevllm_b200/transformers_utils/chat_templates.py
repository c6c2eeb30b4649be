"""Chat-template registry with built-in fallbacks for tokenizers that ship no template
(reference: vllm/transformers_utils/chat_templates/ — registry plus five jinja files)."""
from __future__ import annotations

_TEMPLATES = {
    "chatml": ("<|im_start|>{role}\n{content}<|im_end|>\n", "<|im_start|>assistant\n"),
    "llama2": ("[{role}] {content}\n", "[assistant] "),
    "gemma": ("<start_of_turn>{role}\n{content}<end_of_turn>\n", "<start_of_turn>model\n"),
    "deepseek": ("<｜{role}｜>{content}", "<｜Assistant｜>"),
    "plain": ("{role}: {content}\n", "assistant: "),
}
_BY_FAMILY = {"qwen2": "chatml", "qwen3_5": "chatml", "qwen2_vl": "chatml", "llama": "llama2",
              "gemma4": "gemma", "deepseek_mla": "deepseek"}


def template_for_family(family: str) -> str:
    return _BY_FAMILY.get(family, "plain")


def render_fallback(messages: list[dict], name: str = "plain", add_generation_prompt: bool = True) -> str:
    turn, gen = _TEMPLATES.get(name, _TEMPLATES["plain"])
    text = "".join(turn.format(role=("model" if name == "gemma" and m["role"] == "assistant" else m["role"]),
                               content=m["content"]) for m in messages)
    return text + (gen if add_generation_prompt else "")
