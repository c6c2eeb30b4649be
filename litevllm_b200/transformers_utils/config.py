"""Model configuration loading: ``config.json`` of a checkpoint directory, GGUF metadata, a Gemma4
fallback when the installed transformers release does not know the architecture, and GGUF path
helpers.  Reference: vllm/transformers_utils/config.py, configs/gemma4.py, gguf_utils.py."""
from __future__ import annotations

import json
from pathlib import Path


def is_gguf_path(path: str) -> bool:
    return str(path).lower().endswith(".gguf")


def find_gguf_file(path: str) -> str | None:
    """A ``.gguf`` file itself, or the first (sorted) one inside a directory; split files
    (``-00001-of-0000N.gguf``) resolve to their first shard."""
    p = Path(path)
    if p.is_file() and is_gguf_path(str(p)):
        return str(p)
    if p.is_dir():
        files = sorted(p.glob("*.gguf"))
        return str(files[0]) if files else None
    return None


def load_hf_config_dict(path: str) -> dict:
    """Plain dict of the model configuration (no transformers classes involved)."""
    if is_gguf_path(path):
        from ..loaders.gguf import GGUFFile, hf_config_from_gguf
        with GGUFFile(path) as f:
            return hf_config_from_gguf(f)
    cfg = Path(path) / "config.json"
    if not cfg.exists():
        raise FileNotFoundError(f"{cfg} not found")
    return json.loads(cfg.read_text())


def build_fallback_hf_config(cfg: dict) -> dict:
    """Normalise a Gemma4 configuration whose text part sits under ``text_config`` (multimodal
    checkpoints) into the flat form the architecture parser reads; vision settings stay under
    ``vision_config``."""
    if "text_config" not in cfg:
        return cfg
    flat = dict(cfg["text_config"])
    flat.setdefault("architectures", cfg.get("architectures"))
    flat.setdefault("model_type", cfg["text_config"].get("model_type", cfg.get("model_type")))
    for k in ("vision_config", "quantization_config", "torch_dtype", "image_token_id", "mm_tokens_per_image"):
        if k in cfg and k not in flat:
            flat[k] = cfg[k]
    return flat
