"""Chat-template registry with built-in fallbacks for tokenizers that ship no template.

The fallbacks are jinja files next to this module (``plain``, ``chatml``, ``llama2``, ``gemma``,
``deepseek``), rendered in jinja2's immutable sandbox with the same variables a tokenizer's own template
gets (``messages``, ``add_generation_prompt``).  A message's ``content`` may be a string or a list of
content blocks; the ``text`` filter joins the text blocks and writes ``<image>`` for image blocks.
``register_chat_template_fallback`` maps a model type to a template file, or to a callable that picks
one from the tokenizer's name.  Reference: vllm/transformers_utils/chat_templates/registry.py:31-79 (model
type -> template path registry) and the jinja files beside it.
"""
from __future__ import annotations

from functools import lru_cache
from pathlib import Path
from typing import Callable, Union

TEMPLATE_DIR = Path(__file__).parent
TemplateChoice = Union[Path, Callable[[str], "Path | None"]]

_BY_FAMILY = {"qwen2": "chatml", "qwen3_5": "chatml", "qwen2_vl": "chatml", "llama": "llama2",
              "gemma4": "gemma", "deepseek_mla": "deepseek"}


def _qwen_choice(tokenizer_name: str) -> Path:
    # base Qwen checkpoints have no turn markers of their own
    return TEMPLATE_DIR / ("chatml.jinja" if "chat" in tokenizer_name.lower() or "instruct" in tokenizer_name.lower()
                           else "plain.jinja")


_BY_MODEL_TYPE: dict[str, TemplateChoice] = {
    "llama": TEMPLATE_DIR / "llama2.jinja", "qwen": _qwen_choice, "qwen2": TEMPLATE_DIR / "chatml.jinja",
    "qwen3": TEMPLATE_DIR / "chatml.jinja", "qwen3_5": TEMPLATE_DIR / "chatml.jinja",
    "qwen2_vl": TEMPLATE_DIR / "chatml.jinja", "gemma4": TEMPLATE_DIR / "gemma.jinja",
    "deepseek_v3": TEMPLATE_DIR / "deepseek.jinja", "deepseek_v4_flash": TEMPLATE_DIR / "deepseek.jinja",
}


def register_chat_template_fallback(model_type: str, choice: TemplateChoice) -> None:
    """Later registrations replace earlier ones."""
    _BY_MODEL_TYPE[model_type] = choice


def get_chat_template_fallback(model_type: str, tokenizer_name: str = "") -> Path | None:
    choice = _BY_MODEL_TYPE.get(model_type)
    if callable(choice):
        choice = choice(tokenizer_name)
    return choice


def template_for_family(family: str) -> str:
    return _BY_FAMILY.get(family, "plain")


def _text(content) -> str:
    if isinstance(content, str):
        return content
    if content is None:
        return ""
    parts = []
    for block in content:
        if isinstance(block, str):
            parts.append(block)
        elif block.get("type") == "text":
            parts.append(block.get("text", ""))
        elif block.get("type") in ("image", "image_url"):
            parts.append("<image>")
    return "".join(parts)


@lru_cache(maxsize=32)
def _compiled(source: str):
    from jinja2.sandbox import ImmutableSandboxedEnvironment
    env = ImmutableSandboxedEnvironment(trim_blocks=False, lstrip_blocks=False, keep_trailing_newline=True)
    env.filters["text"] = _text
    return env.from_string(source)


def render_template(source: str, messages: list[dict], add_generation_prompt: bool = True, **variables) -> str:
    return _compiled(source).render(messages=messages, add_generation_prompt=add_generation_prompt, **variables)


def render_fallback(messages: list[dict], name: str = "plain", add_generation_prompt: bool = True) -> str:
    """Render with the built-in template ``name`` (or the file at ``name``)."""
    path = Path(name) if str(name).endswith(".jinja") else TEMPLATE_DIR / f"{name}.jinja"
    if not path.is_file():
        path = TEMPLATE_DIR / "plain.jinja"
    return render_template(path.read_text(encoding="utf-8"), messages, add_generation_prompt)
