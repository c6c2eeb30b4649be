"""Name mapping from HuggingFace checkpoints to this engine's merged / sharded parameters.

A checkpoint is consumed as a stream of ``(name, tensor)`` pairs, each copied straight into its
destination slice (no full-model staging copy).  Quantised tensors keep their on-disk suffixes
(``qweight/scales/qzeros`` for AWQ, ``weight_packed/weight_scale/weight_zero/weight_shape`` for
compressed-tensors) and are routed to the layer's quantisation method.
Reference: vllm/model_executor/model_loader/__init__.py:535-812 (suffix aliases, language_model
prefix handling, mtp.* ignored).
"""
from __future__ import annotations

import re
from collections.abc import Iterable

import torch

_SUFFIX_ALIAS = {"weight_packed": "qweight", "weight_scale": "scales", "weight_zero": "qzeros",
                 "weight_zero_point": "qzeros"}
_IGNORED = re.compile(r"(^|\.)(mtp|rotary_emb\.inv_freq)(\.|$)")


def normalize_name(name: str) -> str:
    for pre in ("model.language_model.", "language_model.model."):
        if name.startswith(pre):
            return "model." + name[len(pre):]
    if name.startswith("language_model."):
        return name[len("language_model."):]
    return name


def split_suffix(name: str) -> tuple[str, str]:
    mod, _, suffix = name.rpartition(".")
    return mod, _SUFFIX_ALIAS.get(suffix, suffix)


def llama_param_map(model) -> dict:
    """module path -> (target, piece, src_rows).  target is a LiteLinear, an nn.Parameter holder
    (``("param", tensor)``) or a norm module."""
    m: dict = {"model.embed_tokens": ("param", model.embed_tokens), "model.norm": ("norm", model.norm)}
    if not model.tie:
        m["lm_head"] = ("linear", model.lm_head, 0, None)
    for i, layer in enumerate(model.layers):
        p = f"model.layers.{i}."
        at = layer.self_attn
        m[p + "self_attn.q_proj"] = ("linear", at.qkv_proj, 0, at.qkv_source_rows("q"))
        m[p + "self_attn.k_proj"] = ("linear", at.qkv_proj, 1, at.qkv_source_rows("k"))
        m[p + "self_attn.v_proj"] = ("linear", at.qkv_proj, 2, at.qkv_source_rows("v"))
        m[p + "self_attn.o_proj"] = ("linear", at.o_proj, 0, None)
        if getattr(at, "qk_norm", False):
            m[p + "self_attn.q_norm"] = ("norm", at.q_norm)
            m[p + "self_attn.k_norm"] = ("norm", at.k_norm)
        m[p + "mlp.gate_proj"] = ("linear", layer.mlp.gate_up_proj, 0, None)
        m[p + "mlp.up_proj"] = ("linear", layer.mlp.gate_up_proj, 1, None)
        m[p + "mlp.down_proj"] = ("linear", layer.mlp.down_proj, 0, None)
        m[p + "input_layernorm"] = ("norm", layer.input_layernorm)
        m[p + "post_attention_layernorm"] = ("norm", layer.post_attention_layernorm)
    return m


def load_mapped(param_map: dict, weights: Iterable[tuple[str, torch.Tensor]], strict: bool = False) -> set[str]:
    consumed: set[str] = set()
    for raw_name, tensor in weights:
        name = normalize_name(raw_name)
        if _IGNORED.search(name):
            continue
        mod, suffix = split_suffix(name)
        entry = param_map.get(mod)
        if entry is None:
            if strict:
                raise KeyError(f"no destination for checkpoint tensor {raw_name}")
            continue
        kind = entry[0]
        if kind == "param":
            entry[1].data.copy_(tensor.to(entry[1].dtype))
        elif kind == "norm":
            entry[1].weight.data.copy_(tensor.to(entry[1].weight.dtype))
        elif kind == "linear":
            _, lin, piece, rows = entry
            lin.load_piece(piece, tensor, suffix, rows)
        elif kind == "custom":
            entry[1](suffix, tensor)
        consumed.add(raw_name)
    return consumed


def load_llama_style(model, weights) -> set[str]:
    consumed = load_mapped(llama_param_map(model), weights)
    finalize_quantized(model)
    return consumed


def finalize_quantized(model) -> None:
    """Give quantised layers the chance to repack once all pieces have arrived."""
    for mod in model.modules():
        qm = getattr(mod, "quant_method", None)
        if qm is not None and hasattr(qm, "process_weights_after_loading"):
            qm.process_weights_after_loading(mod)
