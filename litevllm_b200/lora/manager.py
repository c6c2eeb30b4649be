"""Applies LoRA deltas ``(x A^T) B^T * alpha/r`` on top of the base linear layers.

Adapters attach to the engine's merged layers: ``q_proj/k_proj/v_proj`` deltas land in their row
ranges of the merged QKV output, ``gate_proj/up_proj`` in the merged gate|up output.  A gated layer
with an active adapter runs unfused (GEMM -> add delta -> activation*up), because the delta must be
added before the activation.  Mixed batches apply each adapter to its own token rows.
Reference: vllm/lora/manager.py:51-147, vllm/model_executor/layers/lite_linear.py:65-80.
"""
from __future__ import annotations

import torch

from .. import ops
from ..layers.linear import LiteLinear
from .loader import LoRAWeights, load_lora

_PIECE_OF = {"q_proj": ("qkv_proj", 0), "k_proj": ("qkv_proj", 1), "v_proj": ("qkv_proj", 2),
             "gate_proj": ("gate_up_proj", 0), "up_proj": ("gate_up_proj", 1)}


class LoRAManager:
    def __init__(self, model, device):
        self.model = model
        self.device = device
        self.adapters: dict[str, dict] = {}
        self._layers: dict[str, LiteLinear] = {}
        self.bind_to_model(model)

    def bind_to_model(self, model) -> None:
        for name, mod in model.named_modules():
            if isinstance(mod, LiteLinear):
                self._layers[name] = mod
                mod.lora = self
                mod._lora_key = name

    def _resolve(self, hf_module: str):
        """HF module path -> (engine layer name, piece index)."""
        parent, _, leaf = hf_module.rpartition(".")
        parent = parent[len("model."):] if parent.startswith("model.") and parent not in self._layers else parent
        if leaf in _PIECE_OF:
            merged, piece = _PIECE_OF[leaf]
            key = f"{parent}.{merged}"
            if key in self._layers:
                return key, piece
        key = f"{parent}.{leaf}" if parent else leaf
        if key in self._layers:
            return key, 0
        return None, 0

    def load_adapter(self, name: str, path: str) -> None:
        self.add_adapter(load_lora(name, path))

    def add_adapter(self, w: LoRAWeights) -> None:
        table: dict[str, list] = {}
        for hf_mod, (A, B) in w.modules.items():
            key, piece = self._resolve(hf_mod)
            if key is None:
                continue
            layer = self._layers[key]
            dt = layer.weight.dtype if hasattr(layer, "weight") and layer.quant_method is None else torch.bfloat16
            if self.device.type == "cpu":
                dt = torch.float32 if dt == torch.float32 else dt
            table.setdefault(key, []).append(
                (piece, A.to(self.device, dt).contiguous(), B.to(self.device, dt).contiguous(), w.scale))
        if not table:
            raise ValueError(f"LoRA adapter {w.name!r} matches no layer of this model")
        self.adapters[w.name] = table

    def remove_adapter(self, name: str) -> None:
        self.adapters.pop(name, None)

    def compute_delta(self, x: torch.Tensor, A: torch.Tensor, B: torch.Tensor, scale: float) -> torch.Tensor:
        return ((x.to(A.dtype) @ A.t()) @ B.t()) * scale

    def has_active(self, layer: LiteLinear, mapping) -> bool:
        key = getattr(layer, "_lora_key", None)
        return any(key in self.adapters.get(n, {}) for n in mapping.adapters)

    def apply(self, layer: LiteLinear, x: torch.Tensor, y: torch.Tensor, mapping) -> torch.Tensor:
        key = getattr(layer, "_lora_key", None)
        active = [(n, self.adapters[n][key]) for n in mapping.adapters if key in self.adapters.get(n, {})]
        if not active:
            return y
        if layer.gated_act is not None:
            # redo the projection unfused so the delta enters before the activation
            full = ops.linear(x, layer.weight) if layer.quant_method is None else \
                layer.quant_method.apply(layer, x, ungated=True)
            self._add(full, x, layer, active, mapping)
            return ops.act_mul(full, layer.gated_act)
        self._add(y, x, layer, active, mapping)
        return y

    def _add(self, y, x, layer, active, mapping) -> None:
        for name, entries in active:
            for start, n in mapping.rows_of(name):
                xs = x[start:start + n]
                for piece, A, B, scale in entries:
                    r0 = layer.piece_offset(piece)
                    rows = B.shape[0]
                    y[start:start + n, r0:r0 + rows] += self.compute_delta(xs, A, B, scale).to(y.dtype)
