"""Normalised architecture description read from a HuggingFace ``config.json`` dict (or a GGUF
header).  Model classes and the runtime planner only look at this record, never at raw HF keys.
Reference counterpart: vllm/model_executor/models/lite_config.py:11-158.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass
class QuantSpec:
    method: str = "none"          # none | awq | compressed-tensors | gguf
    bits: int = 16
    group_size: int = 128
    zero_point: bool = True
    symmetric: bool = False


@dataclass
class MoESpec:
    num_experts: int = 0
    top_k: int = 0
    expert_intermediate: int = 0
    shared_intermediate: int = 0     # dense/shared branch width (0 = none)
    n_shared_experts: int = 0
    router: str = "softmax"          # softmax | sigmoid | sqrt_softplus
    renormalize: bool = True
    routed_scaling: float = 1.0
    first_dense_layers: int = 0      # leading layers with a dense MLP instead of experts


@dataclass
class MLASpec:
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_rope_dim: int = 0
    qk_nope_dim: int = 0
    v_head_dim: int = 0


@dataclass
class ModelArch:
    family: str                      # llama | qwen2 | qwen3_5 | gemma4 | deepseek_mla | qwen2_vl
    architecture: str
    hidden_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: dict[str, Any] | None = None
    rotary_dim: int | None = None
    max_position: int = 4096
    tie_embeddings: bool = False
    act: str = "silu"
    attn_bias: bool = False
    mlp_bias: bool = False
    sliding_window: int = 0
    layer_types: list[str] = field(default_factory=list)   # per layer: "full" | "sliding" | "linear"
    attn_softcap: float = 0.0
    final_softcap: float = 0.0
    qk_norm: bool = False
    norm_plus_one: bool = False      # RMSNorm multiplies by (1 + w)
    embed_scale: float = 1.0
    global_head_dim: int | None = None       # Gemma4: global layers may use another head_dim
    global_kv_heads: int | None = None
    global_rope_theta: float | None = None
    partial_rotary_factor: float = 1.0
    eos_token_ids: list[int] = field(default_factory=list)
    bos_token_id: int | None = None
    quant: QuantSpec = field(default_factory=QuantSpec)
    moe: MoESpec = field(default_factory=MoESpec)
    mla: MLASpec = field(default_factory=MLASpec)
    vision: dict[str, Any] | None = None
    extra: dict[str, Any] = field(default_factory=dict)

    def layer_type(self, i: int) -> str:
        if self.layer_types:
            return self.layer_types[i]
        return "full"

    def kv_shape(self, i: int) -> tuple[int, int]:
        """(kv heads, head_dim) of layer i."""
        if self.family == "gemma4" and self.layer_type(i) == "full":
            return (self.global_kv_heads or self.num_kv_heads, self.global_head_dim or self.head_dim)
        return (self.num_kv_heads, self.head_dim)


def _eos_list(cfg: dict) -> list[int]:
    eos = cfg.get("eos_token_id")
    if eos is None:
        return []
    if isinstance(eos, (list, tuple)):
        return [int(e) for e in eos]
    return [int(eos)]


def _quant_from_hf(cfg: dict) -> QuantSpec:
    q = cfg.get("quantization_config") or {}
    if not q:
        return QuantSpec()
    method = str(q.get("quant_method", "")).lower()
    if "awq" in method:
        return QuantSpec("awq", int(q.get("bits", q.get("w_bit", 4))),
                         int(q.get("group_size", q.get("q_group_size", 128))),
                         bool(q.get("zero_point", True)), not bool(q.get("zero_point", True)))
    if method == "compressed-tensors" or q.get("format") == "pack-quantized":
        bits, group, sym = 4, 32, True
        for grp in (q.get("config_groups") or {}).values():
            w = (grp or {}).get("weights") or {}
            bits = int(w.get("num_bits", bits))
            group = int(w.get("group_size", group) or group)
            sym = bool(w.get("symmetric", sym))
            break
        return QuantSpec("compressed-tensors", bits, group, not sym, sym)
    if "gguf" in method:
        return QuantSpec("gguf", 8, 32, False, True)
    return QuantSpec()


def arch_from_hf_config(cfg: dict) -> ModelArch:
    """Build a :class:`ModelArch` from a HF config dict (text sub-config is unwrapped)."""
    archs = cfg.get("architectures") or ["LlamaForCausalLM"]
    architecture = archs[0]
    text = cfg.get("text_config") or cfg
    name = architecture.lower()
    model_type = str(text.get("model_type", cfg.get("model_type", ""))).lower()
    if "gemma4" in name or "gemma4" in model_type or "gemma3n" in name:
        family = "gemma4"
    elif "deepseekv4" in name.replace("_", "") or "deepseek_v4" in model_type:
        family = "deepseek_v4_flash"
    elif "deepseek" in name or "deepseek" in model_type:
        family = "deepseek_mla"
    elif "qwen3_5" in model_type or "qwen3_5" in name or "qwen3next" in name or "qwen3_next" in model_type:
        family = "qwen3_5"
    elif "qwen2vl" in name.replace("_", "") or model_type == "qwen2_vl":
        family = "qwen2_vl"
    elif "qwen2" in name or "qwen3" in name:
        family = "qwen2"
    else:
        family = "llama"
    hidden = int(text["hidden_size"])
    heads = int(text["num_attention_heads"])
    kv_heads = int(text.get("num_key_value_heads", heads) or heads)
    head_dim = int(text.get("head_dim") or hidden // heads)
    arch = ModelArch(
        family=family, architecture=architecture, hidden_size=hidden,
        num_layers=int(text["num_hidden_layers"]), num_heads=heads, num_kv_heads=kv_heads,
        head_dim=head_dim, intermediate_size=int(text.get("intermediate_size", 4 * hidden)),
        vocab_size=int(text["vocab_size"]), rms_eps=float(text.get("rms_norm_eps", 1e-5)),
        rope_theta=float(text.get("rope_theta", (text.get("rope_parameters") or {}).get("rope_theta", 10000.0))),
        rope_scaling=text.get("rope_scaling"),
        max_position=int(text.get("max_position_embeddings", 4096)),
        tie_embeddings=bool(text.get("tie_word_embeddings", cfg.get("tie_word_embeddings", False))),
        act=str(text.get("hidden_act", text.get("hidden_activation", "silu"))),
        attn_bias=bool(text.get("attention_bias", family == "qwen2" and "qwen3" not in name)),
        mlp_bias=bool(text.get("mlp_bias", False)),
        sliding_window=int(text.get("sliding_window") or 0),
        eos_token_ids=_eos_list(text) or _eos_list(cfg),
        bos_token_id=text.get("bos_token_id", cfg.get("bos_token_id")),
        quant=_quant_from_hf(cfg),
        vision=cfg.get("vision_config"),
    )
    arch.partial_rotary_factor = float(text.get("partial_rotary_factor", 1.0))
    arch.rotary_dim = int(head_dim * arch.partial_rotary_factor)
    if family == "qwen2" and "qwen3" in name:
        arch.qk_norm = True
    if family == "gemma4":
        lt = text.get("layer_types") or []
        arch.layer_types = ["sliding" if "sliding" in t else "full" for t in lt]
        if not arch.layer_types:
            pat = int(text.get("sliding_window_pattern", 6))
            arch.layer_types = ["full" if (i + 1) % pat == 0 else "sliding" for i in range(arch.num_layers)]
        arch.attn_softcap = float(text.get("attn_logit_softcapping") or 0.0)
        arch.final_softcap = float(text.get("final_logit_softcapping") or 0.0)
        arch.qk_norm = True
        arch.embed_scale = float(hidden) ** 0.5
        arch.global_head_dim = text.get("global_head_dim")
        arch.global_kv_heads = text.get("num_global_key_value_heads")
        arch.global_rope_theta = text.get("rope_global_base_freq", text.get("global_rope_theta"))
        arch.rope_theta = float(text.get("rope_local_base_freq", arch.rope_theta))
        arch.act = "gelu_tanh"
        n_exp = int(text.get("num_experts", 0) or 0)
        if n_exp:
            arch.moe = MoESpec(num_experts=n_exp, top_k=int(text.get("top_k_experts", text.get("num_experts_per_tok", 8))),
                               expert_intermediate=int(text.get("moe_intermediate_size", text.get("expert_intermediate_size", 704))),
                               shared_intermediate=arch.intermediate_size, router="softmax", renormalize=True)
        arch.extra["attention_k_eq_v"] = bool(text.get("attention_k_eq_v", False))
    if family == "deepseek_mla":
        arch.mla = MLASpec(int(text.get("q_lora_rank") or 0), int(text.get("kv_lora_rank", 512)),
                           int(text.get("qk_rope_head_dim", 64)), int(text.get("qk_nope_head_dim", 128)),
                           int(text.get("v_head_dim", 128)))
        arch.head_dim = arch.mla.qk_nope_dim + arch.mla.qk_rope_dim
        arch.moe = MoESpec(num_experts=int(text.get("n_routed_experts", 0) or 0),
                           top_k=int(text.get("num_experts_per_tok", 6)),
                           expert_intermediate=int(text.get("moe_intermediate_size", 2048)),
                           n_shared_experts=int(text.get("n_shared_experts", 1)),
                           shared_intermediate=int(text.get("moe_intermediate_size", 2048)) * int(text.get("n_shared_experts", 1)),
                           router=str(text.get("scoring_func", "sigmoid")),
                           renormalize=bool(text.get("norm_topk_prob", True)),
                           routed_scaling=float(text.get("routed_scaling_factor", 1.0)),
                           first_dense_layers=int(text.get("first_k_dense_replace", 0)))
        if text.get("expert_staging_gb"):       # e.g. hf_overrides={"expert_staging_gb": 40}
            arch.extra["expert_staging_gb"] = float(text["expert_staging_gb"])
    if family == "deepseek_v4_flash":
        arch.extra["v4_rows"] = {k: text[k] for k in ("num_hidden_layers", "head_dim", "sliding_window",
                                                      "compress_ratio_coarse", "layer_compress_ratios")
                                 if text.get(k) is not None}
    if family == "qwen3_5":
        lt = text.get("layer_types") or []
        interval = int(text.get("full_attention_interval", 4))
        arch.layer_types = (["linear" if "linear" in t else "full" for t in lt] if lt else
                            ["full" if (i + 1) % interval == 0 else "linear" for i in range(arch.num_layers)])
        arch.qk_norm = True
        arch.norm_plus_one = True
        arch.extra.update({k: text.get(k) for k in (
            "linear_num_key_heads", "linear_num_value_heads", "linear_key_head_dim",
            "linear_value_head_dim", "linear_conv_kernel_dim", "mrope_section", "attn_output_gate")
            if text.get(k) is not None})
        n_exp = int(text.get("num_experts", 0) or 0)
        if n_exp:
            arch.moe = MoESpec(num_experts=n_exp, top_k=int(text.get("num_experts_per_tok", 8)),
                               expert_intermediate=int(text.get("moe_intermediate_size", 512)),
                               shared_intermediate=int(text.get("shared_expert_intermediate_size", 0)),
                               router="softmax", renormalize=bool(text.get("norm_topk_prob", True)))
    if family == "qwen2_vl":
        rs = text.get("rope_scaling") or cfg.get("rope_scaling") or {}
        if rs.get("mrope_section"):
            arch.extra["mrope_section"] = list(rs["mrope_section"])
    return arch
