"""PEFT-format LoRA loader: ``adapter_config.json`` + ``adapter_model.safetensors``.
Reference: vllm/lora/loader.py:16-102 (PEFT safetensors only)."""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from pathlib import Path

import torch


@dataclass
class LoRAWeights:
    name: str
    rank: int
    alpha: float
    # module path (e.g. "model.layers.0.self_attn.q_proj") -> (A [r, in], B [out, r])
    modules: dict[str, tuple[torch.Tensor, torch.Tensor]] = field(default_factory=dict)

    @property
    def scale(self) -> float:
        return self.alpha / max(self.rank, 1)


_KEY = re.compile(r"^(?:base_model\.model\.)?(.*)\.lora_([AB])(?:\.default)?\.weight$")


def load_lora(name: str, path: str | Path) -> LoRAWeights:
    from safetensors.torch import load_file
    p = Path(path)
    cfg_file = p / "adapter_config.json"
    if not cfg_file.is_file():
        raise FileNotFoundError(f"{cfg_file} not found (only PEFT adapters are supported)")
    cfg = json.loads(cfg_file.read_text())
    st_file = p / "adapter_model.safetensors"
    if not st_file.is_file():
        raise FileNotFoundError(f"{st_file} not found (only safetensors adapters are supported)")
    tensors = load_file(str(st_file))
    halves: dict[str, dict[str, torch.Tensor]] = {}
    for key, t in tensors.items():
        m = _KEY.match(key)
        if not m:
            continue
        halves.setdefault(m.group(1), {})[m.group(2)] = t
    out = LoRAWeights(name=name, rank=int(cfg.get("r", 8)), alpha=float(cfg.get("lora_alpha", cfg.get("r", 8))))
    for mod, ab in halves.items():
        if "A" in ab and "B" in ab:
            out.modules[mod] = (ab["A"], ab["B"])
    if not out.modules:
        raise ValueError(f"no lora_A/lora_B pairs found in {st_file}")
    return out
