"""GGUF checkpoints: reader (native header parser in csrc/host/gguf_reader.cpp + zero-copy numpy
memory maps for the payloads), a writer for synthetic files, the GGUF -> HF config translation and
the GGUF -> engine tensor-name mapping.

Quantised tensors are yielded as :class:`GGUFTensor` (raw block bytes + type + logical shape) and are
consumed in place by the GGUF kernels; F32/F16/BF16 tensors are yielded as ordinary torch tensors.
Reference: vllm/model_executor/models/deepseek_v4_flash/gguf_reader.py:13-366 and weight_store.py
(semantic tensor binding), vllm/model_executor/model_loader/__init__.py:55-338 (generic GGUF path).
"""
from __future__ import annotations

import ctypes
import json
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

from ..ops import _lib
from ..ops.gguf_quant import BLOCK, TYPE_NAMES

_NP = {0: np.float32, 1: np.float16, 26: np.int32}


@dataclass
class GGUFTensor:
    """A quantised GGUF tensor: ``raw`` is uint8 [..., rows, row_bytes]; ``shape`` the logical shape
    (outermost first), ``ggml_type`` the block format id."""
    raw: torch.Tensor
    ggml_type: int
    shape: tuple

    @property
    def K(self) -> int:
        return self.shape[-1]


class GGUFFile:
    def __init__(self, path: str | Path):
        self.path = str(path)
        lib = _lib.host()
        err = ctypes.create_string_buffer(256)
        lib.fi_gguf_open.restype = ctypes.c_void_p
        h = lib.fi_gguf_open(self.path.encode(), err, 256)
        if not h:
            raise ValueError(f"cannot read GGUF file {self.path}: {err.value.decode()}")
        try:
            n = lib.fi_gguf_meta_json_len(ctypes.c_void_p(h))
            buf = ctypes.create_string_buffer(n + 1)
            lib.fi_gguf_meta_json(ctypes.c_void_p(h), buf, n + 1)
            self.metadata: dict = json.loads(buf.value.decode("utf-8", errors="replace"))
            self.alignment = int(lib.fi_gguf_alignment(ctypes.c_void_p(h)))
            self.tensors: dict[str, dict] = {}
            name = ctypes.create_string_buffer(512)
            dims = (ctypes.c_long * 4)()
            info = (ctypes.c_int * 2)()
            sizes = (ctypes.c_long * 2)()
            for i in range(lib.fi_gguf_num_tensors(ctypes.c_void_p(h))):
                rc = lib.fi_gguf_tensor_info(ctypes.c_void_p(h), i, name, 512, dims, info, sizes)
                if rc != 0:
                    raise ValueError(f"bad tensor record {i} in {self.path}")
                nd = info[0]
                shape = tuple(int(dims[d]) for d in range(nd))[::-1]     # outermost first
                self.tensors[name.value.decode()] = {"shape": shape, "type": int(info[1]),
                                                     "offset": int(sizes[0]), "nbytes": int(sizes[1])}
        finally:
            lib.fi_gguf_close(ctypes.c_void_p(h))

    def arch(self) -> str:
        return str(self.metadata.get("general.architecture", ""))

    def get(self, key: str, default=None):
        a = self.arch()
        return self.metadata.get(f"{a}.{key}", self.metadata.get(key, default))

    def load(self, name: str):
        """-> torch tensor (float types) or GGUFTensor (block-quantised), backed by the memory map."""
        t = self.tensors[name]
        ty, shape = t["type"], t["shape"]
        if ty in _NP:
            arr = np.memmap(self.path, dtype=_NP[ty], mode="r", offset=t["offset"], shape=shape)
            return torch.from_numpy(np.ascontiguousarray(arr))
        if ty == 30:
            arr = np.memmap(self.path, dtype=np.int16, mode="r", offset=t["offset"], shape=shape)
            return torch.from_numpy(np.ascontiguousarray(arr)).view(torch.bfloat16)
        if ty in BLOCK:
            vals, nb = BLOCK[ty]
            raw_shape = shape[:-1] + (shape[-1] // vals * nb,)
            arr = np.memmap(self.path, dtype=np.uint8, mode="r", offset=t["offset"], shape=raw_shape)
            return GGUFTensor(torch.from_numpy(np.ascontiguousarray(arr)), ty, shape)
        raise ValueError(f"tensor {name}: unsupported GGML type {ty} ({TYPE_NAMES.get(ty, '?')})")


# ----------------------------------------------------------------------------- writer
_KV = {"u32": (4, "<I"), "i32": (5, "<i"), "f32": (6, "<f"), "bool": (7, "<B"), "u64": (10, "<Q")}


def _kv_bytes(key: str, value) -> bytes:
    out = struct.pack("<Q", len(key.encode())) + key.encode()
    if isinstance(value, bool):
        return out + struct.pack("<I", 7) + struct.pack("<B", int(value))
    if isinstance(value, int):
        return out + (struct.pack("<I", 4) + struct.pack("<I", value) if 0 <= value < 2 ** 32
                      else struct.pack("<I", 11) + struct.pack("<q", value))
    if isinstance(value, float):
        return out + struct.pack("<I", 6) + struct.pack("<f", value)
    if isinstance(value, str):
        b = value.encode()
        return out + struct.pack("<I", 8) + struct.pack("<Q", len(b)) + b
    if isinstance(value, (list, tuple)):
        if all(isinstance(v, int) for v in value):
            body = b"".join(struct.pack("<i", v) for v in value)
            return out + struct.pack("<I", 9) + struct.pack("<I", 5) + struct.pack("<Q", len(value)) + body
        if all(isinstance(v, float) for v in value):
            body = b"".join(struct.pack("<f", v) for v in value)
            return out + struct.pack("<I", 9) + struct.pack("<I", 6) + struct.pack("<Q", len(value)) + body
    raise TypeError(f"unsupported metadata value for {key}: {type(value).__name__}")


def write_gguf(path: str | Path, metadata: dict, tensors: dict, alignment: int = 32) -> None:
    """tensors: name -> torch tensor (F32/F16/BF16/I32) or GGUFTensor."""
    metadata = dict(metadata)
    metadata.setdefault("general.alignment", alignment)
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(metadata))
    head += b"".join(_kv_bytes(k, v) for k, v in metadata.items())
    infos, blobs, off = b"", [], 0
    for name, t in tensors.items():
        if isinstance(t, GGUFTensor):
            ty, shape, data = t.ggml_type, t.shape, t.raw.contiguous().numpy().tobytes()
        else:
            ty = {torch.float32: 0, torch.float16: 1, torch.int32: 26, torch.bfloat16: 30}[t.dtype]
            shape = tuple(t.shape)
            data = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).contiguous().numpy().tobytes()
        nb = name.encode()
        infos += struct.pack("<Q", len(nb)) + nb + struct.pack("<I", len(shape))
        infos += b"".join(struct.pack("<Q", d) for d in shape[::-1])
        infos += struct.pack("<I", ty) + struct.pack("<Q", off)
        blobs.append((off, data))
        off = (off + len(data) + alignment - 1) // alignment * alignment
    pre = head + infos
    pad = (-len(pre)) % alignment
    with open(path, "wb") as f:
        f.write(pre + b"\0" * pad)
        base = f.tell()
        for o, data in blobs:
            f.seek(base + o)
            f.write(data)
        f.truncate(base + off if blobs else base)


# ----------------------------------------------------------------------------- config translation
def hf_config_from_gguf(path: str | Path) -> dict:
    g = GGUFFile(path)
    a = g.arch()
    for key in ("embedding_length", "block_count"):
        if g.get(key) is None:
            raise ValueError(f"{g.path}: GGUF metadata lacks {a}.{key}")
    heads = int(g.get("attention.head_count", 32))
    hidden = int(g.get("embedding_length"))
    cfg = {
        "hidden_size": hidden, "num_hidden_layers": int(g.get("block_count")), "num_attention_heads": heads,
        "num_key_value_heads": int(g.get("attention.head_count_kv", heads)),
        "intermediate_size": int(g.get("feed_forward_length", 4 * hidden)),
        "rms_norm_eps": float(g.get("attention.layer_norm_rms_epsilon", 1e-5)),
        "rope_theta": float(g.get("rope.freq_base", 10000.0)),
        "max_position_embeddings": int(g.get("context_length", 4096)),
        "vocab_size": int(g.get("vocab_size", 0)) or g.tensors.get("token_embd.weight", {"shape": (32000,)})["shape"][0],
        "quantization_config": {"quant_method": "gguf"},
        "eos_token_id": g.metadata.get("tokenizer.ggml.eos_token_id"),
        "bos_token_id": g.metadata.get("tokenizer.ggml.bos_token_id"),
        "tie_word_embeddings": "output.weight" not in g.tensors,
    }
    if a in ("deepseek2", "deepseek3", "deepseek_v3"):
        cfg.update({
            "architectures": ["DeepseekV3ForCausalLM"], "model_type": "deepseek_v3",
            "q_lora_rank": int(g.get("attention.q_lora_rank", 0)) or None,
            "kv_lora_rank": int(g.get("attention.kv_lora_rank", 512)),
            "qk_rope_head_dim": int(g.get("rope.dimension_count", 64)),
            "qk_nope_head_dim": int(g.get("attention.key_length", 192)) - int(g.get("rope.dimension_count", 64)),
            "v_head_dim": int(g.get("attention.value_length", 128)),
            "n_routed_experts": int(g.get("expert_count", 0)), "num_experts_per_tok": int(g.get("expert_used_count", 6)),
            "n_shared_experts": int(g.get("expert_shared_count", 1)),
            "moe_intermediate_size": int(g.get("expert_feed_forward_length", 2048)),
            "first_k_dense_replace": int(g.get("leading_dense_block_count", 0)),
            "routed_scaling_factor": float(g.get("expert_weights_scale", 1.0)),
            "norm_topk_prob": bool(g.get("expert_weights_norm", True)),
            "scoring_func": "sigmoid" if int(g.get("expert_gating_func", 2)) == 2 else "softmax",
        })
    elif a == "deepseek4":
        cfg.update(_deepseek4_config(g))
    elif a.startswith("qwen2"):
        cfg.update({"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2"})
    else:
        cfg.update({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    return cfg


def _deepseek4_config(g: "GGUFFile") -> dict:
    """DeepSeek-V4-Flash: head counts, window, indexer and expert counts come from the ``deepseek4.*`` metadata;
    the low-rank widths, the group count, the expert width and the number of hash-routed layers are read off the
    tensor shapes; the rest defaults to the checkpoint family's constants.  Reference (fixed shape validated
    against the metadata): vllm/model_executor/models/deepseek_v4_flash/gguf_reader.py:100-111, config.py:41-67."""
    def shape(name, default=None):
        t = g.tensors.get(name)
        return t["shape"] if t is not None else default

    for key in ("block_count", "embedding_length", "attention.head_count"):
        if g.get(key) is None:
            raise ValueError(f"{g.path}: deepseek4 metadata lacks {key!r}")
    for name in ("token_embd.weight", "blk.0.attn_q_a.weight", "blk.0.attn_output_b.weight", "blk.0.ffn_gate_exps.weight"):
        if name not in g.tensors:
            raise ValueError(f"{g.path}: deepseek4 file lacks the tensor {name!r}")
    layers = int(g.get("block_count"))
    head_dim = int(g.get("attention.key_length", 512))
    heads = int(g.get("attention.head_count", 64))
    q_a = shape("blk.0.attn_q_a.weight", (1024, 0))
    o_a = shape("blk.0.attn_output_a.weight")          # [groups * rank, heads/groups * head_dim] (or 3-D)
    o_b = shape("blk.0.attn_output_b.weight")          # [hidden, groups * rank]
    groups = int(g.get("attention.output_group_count", 0))
    if not groups and o_a is not None:
        groups = o_a[0] if len(o_a) == 3 else max(1, heads * head_dim // o_a[-1])
    groups = groups or 8
    experts = shape("blk.0.ffn_gate_exps.weight", (0, 2048, 0))
    shared = shape("blk.0.ffn_gate_shexp.weight", (experts[1], 0))
    hc_fn = shape("output_hc_fn.weight")
    out = {
        "architectures": ["DeepseekV4FlashForCausalLM"], "model_type": "deepseek_v4_flash", "head_dim": head_dim,
        "qk_rope_head_dim": int(g.get("rope.dimension_count", 64)), "q_lora_rank": int(q_a[0]),
        "sliding_window": int(g.get("attention.sliding_window", 128)),
        "index_n_heads": int(g.get("attention.indexer.head_count", 64)),
        "index_topk": int(g.get("attention.indexer.top_k", 512)),
        "hc_mult": int(min(hc_fn)) if hc_fn is not None else 4, "o_groups": int(groups),
        "o_lora_rank": int(o_b[1] // groups) if o_b is not None else 1024,
        "n_routed_experts": int(g.get("expert_count", experts[0])),
        "num_experts_per_tok": int(g.get("expert_used_count", 6)),
        "moe_intermediate_size": int(g.get("expert_feed_forward_length", experts[1])),
        "shared_intermediate_size": int(shared[0]),
        "num_hash_layers": sum(1 for i in range(layers) if f"blk.{i}.ffn_gate_tid2eid.weight" in g.tensors),
        "routed_scaling_factor": float(g.get("expert_weights_scale", 1.5)),
        "swiglu_limit": float(g.get("swiglu_clamp", 10.0)),
        "compress_ratio_coarse": int(g.get("attention.compress_ratio_coarse", 128)),
        "compressed_rope_theta": float(g.get("rope.compressed_freq_base", 160000.0)),
        "rope_scaling_factor": float(g.get("rope.scaling.factor", 16.0)),
        "rope_original_context": int(g.get("rope.scaling.original_context_length", 65536)),
        "rope_beta_fast": float(g.get("rope.scaling.yarn_beta_fast", 32.0)),
        "rope_beta_slow": float(g.get("rope.scaling.yarn_beta_slow", 1.0)),
        "tie_word_embeddings": False,
    }
    return out


# GGUF tensor name -> HF-style module path used by the model classes
_LAYER_MAP = {
    "attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm",
    "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj",
    "attn_output": "self_attn.o_proj", "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj",
    "ffn_down": "mlp.down_proj",
    "attn_q_a": "self_attn.q_a_proj", "attn_q_a_norm": "self_attn.q_a_layernorm", "attn_q_b": "self_attn.q_b_proj",
    "attn_kv_a_mqa": "self_attn.kv_a_proj_with_mqa", "attn_kv_a_norm": "self_attn.kv_a_layernorm",
    "attn_kv_b": "self_attn.kv_b_proj",
    "ffn_gate_inp": "mlp.gate", "exp_probs_b": "mlp.gate.e_score_correction_bias",
    "ffn_gate_exps": "mlp.experts.gate_proj", "ffn_up_exps": "mlp.experts.up_proj",
    "ffn_down_exps": "mlp.experts.down_proj",
    "ffn_gate_shexp": "mlp.shared_experts.gate_proj", "ffn_up_shexp": "mlp.shared_experts.up_proj",
    "ffn_down_shexp": "mlp.shared_experts.down_proj",
}


def gguf_to_hf_name(name: str) -> str | None:
    if name == "token_embd.weight":
        return "model.embed_tokens.weight"
    if name == "output_norm.weight":
        return "model.norm.weight"
    if name == "output.weight":
        return "lm_head.weight"
    parts = name.split(".")
    if parts[0] == "blk" and len(parts) >= 4:
        mod = _LAYER_MAP.get(parts[2])
        if mod is None:
            return None
        suffix = parts[3]
        if parts[2] == "exp_probs_b":
            return f"model.layers.{parts[1]}.{mod}"
        return f"model.layers.{parts[1]}.{mod}.{suffix}"
    return None


# ----------------------------------------------------------------------------- Qwen3.5 (gated delta-net hybrid)
# GGUF files of this family differ from the HF checkpoint in three ways (the exporter's conventions): value heads
# of the linear-attention tensors are stored tiled ([per-key-head copy, key head, dim]) instead of grouped
# ([key head, copy, dim]); every RMSNorm gain except the gated linear-attention norm has 1 added; the depthwise
# convolution is [kernel, channels].  ``ssm_a`` holds -exp(A_log).
# Reference: vllm/model_executor/model_loader/__init__.py:74-215 (the same fix-ups, per tensor at load time).
_QWEN35_LAYER_MAP = {
    "attn_norm": "input_layernorm", "post_attention_norm": "post_attention_layernorm", "ffn_norm": "post_attention_layernorm",
    "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj",
    "attn_output": "self_attn.o_proj", "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm",
    "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj",
    "attn_qkv": "linear_attn.in_proj_qkv", "attn_gate": "linear_attn.in_proj_z", "ssm_alpha": "linear_attn.in_proj_a",
    "ssm_beta": "linear_attn.in_proj_b", "ssm_out": "linear_attn.out_proj", "ssm_conv1d": "linear_attn.conv1d",
    "ssm_norm": "linear_attn.norm", "ffn_gate_inp": "mlp.gate", "ffn_gate_shexp": "mlp.shared_expert.gate_proj",
    "ffn_up_shexp": "mlp.shared_expert.up_proj", "ffn_down_shexp": "mlp.shared_expert.down_proj",
    "ffn_gate_inp_shexp": "mlp.shared_expert_gate",
}
_QWEN35_EXPERTS = {"ffn_gate_exps": "gate_proj", "ffn_up_exps": "up_proj", "ffn_down_exps": "down_proj"}


def tiled_to_grouped(t: torch.Tensor, dim: int, num_k: int, per_k: int, head_dim: int) -> torch.Tensor:
    """Value heads along ``dim`` from the file's tiled order to the grouped order of the HF checkpoint."""
    shape = list(t.shape)
    dim %= len(shape)
    u = t.reshape(*shape[:dim], per_k, num_k, head_dim, *shape[dim + 1:])
    return u.transpose(dim, dim + 1).contiguous().reshape(shape)


def grouped_to_tiled(t: torch.Tensor, dim: int, num_k: int, per_k: int, head_dim: int) -> torch.Tensor:
    """Inverse of :func:`tiled_to_grouped` (what an exporter applies)."""
    shape = list(t.shape)
    dim %= len(shape)
    u = t.reshape(*shape[:dim], num_k, per_k, head_dim, *shape[dim + 1:])
    return u.transpose(dim, dim + 1).contiguous().reshape(shape)


def qwen35_fixup(kind: str, suffix: str, t: torch.Tensor, extra: dict) -> torch.Tensor:
    """One dense tensor of a Qwen3.5 GGUF file -> the HF layout the model's loader expects."""
    nk, nv = int(extra.get("linear_num_key_heads", 0) or 0), int(extra.get("linear_num_value_heads", 0) or 0)
    dk, dv = int(extra.get("linear_key_head_dim", 0) or 0), int(extra.get("linear_value_head_dim", 0) or 0)
    tiled = nk > 0 and nv > nk and nv % nk == 0 and dk > 0 and dv > 0
    per = nv // nk if tiled else 1
    if kind == "ssm_conv1d" and suffix == "weight":
        if t.dim() == 2 and t.shape[0] < t.shape[1]:
            t = t.t()                                           # [kernel, channels] -> [channels, kernel]
        t = t.reshape(t.shape[0], -1)
        if tiled and t.shape[0] == 2 * nk * dk + nv * dv:
            qk = 2 * nk * dk
            t = torch.cat([t[:qk], tiled_to_grouped(t[qk:], 0, nk, per, dv)])
        return t.unsqueeze(1).contiguous()                      # [channels, 1, kernel]
    if kind.endswith("norm") and suffix == "weight" and t.dim() == 1 and kind != "ssm_norm":
        return t.float() - 1.0
    if not tiled:
        return t
    if kind == "attn_qkv" and suffix == "weight" and t.shape[0] == 2 * nk * dk + nv * dv:
        qk = 2 * nk * dk
        return torch.cat([t[:qk], tiled_to_grouped(t[qk:], 0, nk, per, dv)])
    if kind == "attn_gate" and suffix == "weight" and t.shape[0] == nv * dv:
        return tiled_to_grouped(t, 0, nk, per, dv)
    if kind == "ssm_out" and suffix == "weight" and t.shape[-1] == nv * dv:
        return tiled_to_grouped(t, 1, nk, per, dv)
    if kind in ("ssm_alpha", "ssm_beta") and suffix == "weight" and t.shape[0] == nv:
        return tiled_to_grouped(t, 0, nk, per, 1)
    if kind in ("ssm_a", "ssm_dt") and t.dim() == 1 and t.shape[0] == nv:
        return tiled_to_grouped(t.unsqueeze(-1), 0, nk, per, 1).squeeze(-1)
    return t


def _iter_qwen35(g: "GGUFFile", arch):
    from ..ops import gguf_quant as gq

    def dense(name):
        t = g.load(name)
        if isinstance(t, GGUFTensor):
            t = gq.dequantize(t.raw.reshape(-1, t.raw.shape[-1]), t.ggml_type, t.K).reshape(t.shape)
        return t

    extra = getattr(arch, "extra", {}) or {}
    for name in g.tensors:
        hf = {"token_embd.weight": "model.embed_tokens.weight", "output_norm.weight": "model.norm.weight",
              "output.weight": "lm_head.weight"}.get(name)
        if hf is not None:
            t = dense(name)
            yield hf, (t.float() - 1.0 if name == "output_norm.weight" else t)
            continue
        parts = name.split(".")
        if parts[0] != "blk" or len(parts) < 3:
            continue
        layer, kind, suffix = parts[1], parts[2], ".".join(parts[3:])
        prefix = f"model.layers.{layer}."
        if kind == "ssm_a":                                      # the file stores -exp(A_log)
            t = qwen35_fixup(kind, suffix, dense(name).float(), extra)
            yield prefix + "linear_attn.A_log", (torch.log(-t) if bool((t < 0).all()) else t)
        elif kind == "ssm_dt":
            yield prefix + "linear_attn.dt_bias", qwen35_fixup(kind, suffix, dense(name).float(), extra)
        elif kind in _QWEN35_EXPERTS:                            # [E, rows, cols] -> one tensor per expert
            t = dense(name)
            for e in range(t.shape[0]):
                yield prefix + f"mlp.experts.{e}.{_QWEN35_EXPERTS[kind]}.weight", t[e]
        elif kind in _QWEN35_LAYER_MAP:
            yield prefix + _QWEN35_LAYER_MAP[kind] + "." + suffix, qwen35_fixup(kind, suffix, dense(name), extra)


def iter_gguf_weights(path: str | Path, arch=None):
    p = Path(path)
    if p.is_dir():
        p = sorted(p.glob("*.gguf"))[0]
    g = GGUFFile(p)
    if g.arch() == "deepseek4":          # the model binds the checkpoint's own tensor names
        for name in g.tensors:
            yield name, g.load(name)
        return
    if getattr(arch, "family", "") == "qwen3_5":
        yield from _iter_qwen35(g, arch)
        return
    for name in g.tensors:
        hf = gguf_to_hf_name(name)
        if hf is None:
            continue
        yield hf, g.load(name)
