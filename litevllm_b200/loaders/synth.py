"""Random-init weight streams in HuggingFace naming, so synthetic models load through the same
path as real checkpoints.  Every tensor is drawn from its own generator seeded by
(seed, tensor name): the stream is identical on every rank and for any loading order, which is what
tensor-parallel runs and the CPU oracle comparison need.

Dense weights ~ N(0, 0.02); norm weights = 1; AWQ tensors are random int4 codes with
|N(0, 0.01)| scales; GGUF-quantised tensors are random block payloads with small fp16 scales.
"""
from __future__ import annotations

import zlib
from collections.abc import Iterator

import torch

from ..models.arch import ModelArch


def _gen(seed: int, name: str, device: str = "cpu") -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed((seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFF)
    return g


def normal(name: str, shape, seed: int, std: float = 0.02, dtype=torch.float32, device="cpu") -> torch.Tensor:
    g = _gen(seed, name, device)
    return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * std).to(dtype)


def awq_pieces(name: str, out_f: int, in_f: int, group: int, seed: int, zero_point: bool, device="cpu",
               scale_dtype=torch.float16):
    """Random packed int4 in the row-major layout: qweight int32 [N, K/8] (nibble j of a word =
    column 8w+j), scales [N, K/G], qzeros int32 [N, K/G/8]."""
    g = _gen(seed, name, device)
    qweight = torch.randint(-2 ** 31, 2 ** 31 - 1, (out_f, in_f // 8), generator=g, device=device,
                            dtype=torch.int64).to(torch.int32)
    scales = (torch.randn(out_f, in_f // group, generator=g, device=device) * 0.01).abs().add_(1e-4).to(scale_dtype)
    out = {"qweight": qweight, "scales": scales}
    if zero_point:
        ng = in_f // group
        out["qzeros"] = torch.randint(-2 ** 31, 2 ** 31 - 1, (out_f, (ng + 7) // 8), generator=g,
                                      device=device, dtype=torch.int64).to(torch.int32)
    return out


def iter_llama_weights(arch: ModelArch, seed: int = 0, dtype=torch.float32, device="cpu") -> Iterator[tuple[str, torch.Tensor]]:
    H, I, V = arch.hidden_size, arch.intermediate_size, arch.vocab_size
    q_rows, kv_rows = arch.num_heads * arch.head_dim, arch.num_kv_heads * arch.head_dim
    quant = arch.quant.method != "none"

    def lin(name, out_f, in_f):
        if quant:
            sfx = {"qweight": "qweight", "scales": "scales", "qzeros": "qzeros"}
            if arch.quant.method == "compressed-tensors":
                sfx = {"qweight": "weight_packed", "scales": "weight_scale", "qzeros": "weight_zero"}
            pieces = awq_pieces(name, out_f, in_f, arch.quant.group_size, seed, arch.quant.zero_point, device,
                                torch.float16 if dtype == torch.float16 else torch.bfloat16 if dtype == torch.bfloat16 else torch.float16)
            for k, t in pieces.items():
                yield f"{name}.{sfx[k]}", t
        else:
            yield f"{name}.weight", normal(name, (out_f, in_f), seed, dtype=dtype, device=device)

    yield "model.embed_tokens.weight", normal("model.embed_tokens", (V, H), seed, dtype=dtype, device=device)
    for i in range(arch.num_layers):
        p = f"model.layers.{i}."
        yield from lin(p + "self_attn.q_proj", q_rows, H)
        yield from lin(p + "self_attn.k_proj", kv_rows, H)
        yield from lin(p + "self_attn.v_proj", kv_rows, H)
        yield from lin(p + "self_attn.o_proj", H, q_rows)
        yield from lin(p + "mlp.gate_proj", I, H)
        yield from lin(p + "mlp.up_proj", I, H)
        yield from lin(p + "mlp.down_proj", H, I)
        if arch.attn_bias:
            for n, r in (("q", q_rows), ("k", kv_rows), ("v", kv_rows)):
                yield p + f"self_attn.{n}_proj.bias", normal(p + n + "b", (r,), seed, dtype=dtype, device=device)
        if V <= 1024:   # the tiny test shapes get non-trivial norm weights (the benchmark shapes keep ones)
            base = 0.0 if arch.norm_plus_one else 1.0
            for n in ("input_layernorm", "post_attention_layernorm"):
                yield p + n + ".weight", (base + 10.0 * normal(p + n, (H,), seed, dtype=torch.float32, device=device)).to(dtype)
            if arch.qk_norm:
                for n in ("q_norm", "k_norm"):
                    yield p + f"self_attn.{n}.weight", (base + 10.0 * normal(p + n, (arch.head_dim,), seed, dtype=torch.float32, device=device)).to(dtype)
    if V <= 1024:
        yield "model.norm.weight", (1.0 + 10.0 * normal("model.norm", (H,), seed, dtype=torch.float32, device=device)).to(dtype)
    if not arch.tie_embeddings:
        yield "lm_head.weight", normal("lm_head", (V, H), seed, dtype=dtype, device=device)


def iter_gemma4_weights(arch: ModelArch, seed: int = 0, dtype=torch.bfloat16, device="cpu") -> Iterator[tuple[str, torch.Tensor]]:
    """Gemma4 (dense or MoE) with compressed-tensors style int4 tensors when the arch is quantised."""
    H, V = arch.hidden_size, arch.vocab_size
    quant = arch.quant.method != "none"
    G = arch.quant.group_size if quant else 32
    sdt = torch.float16 if dtype == torch.float32 else dtype

    def lin(name, out_f, in_f):
        if quant:
            pieces = awq_pieces(name, out_f, in_f, G, seed, False, device, sdt)
            yield f"{name}.weight_packed", pieces["qweight"]
            yield f"{name}.weight_scale", pieces["scales"]
        else:
            yield f"{name}.weight", normal(name, (out_f, in_f), seed, dtype=dtype, device=device)

    yield "model.embed_tokens.weight", normal("model.embed_tokens", (V, H), seed, dtype=dtype, device=device)
    for i in range(arch.num_layers):
        p = f"model.layers.{i}."
        nkv, hd = arch.kv_shape(i)
        yield from lin(p + "self_attn.q_proj", arch.num_heads * hd, H)
        yield from lin(p + "self_attn.k_proj", nkv * hd, H)
        yield from lin(p + "self_attn.v_proj", nkv * hd, H)
        yield from lin(p + "self_attn.o_proj", H, arch.num_heads * hd)
        if arch.moe.num_experts:
            E, I = arch.moe.num_experts, arch.moe.expert_intermediate
            sh = arch.moe.shared_intermediate or arch.intermediate_size
            mp = p + "mlp.shared_mlp."
            yield p + "mlp.router.proj.weight", normal(p + "router", (E, H), seed, dtype=dtype, device=device)
            gu = awq_pieces(p + "experts.gu", E * 2 * I, H, G, seed, False, device, sdt)
            dn = awq_pieces(p + "experts.dn", E * H, I, G, seed, False, device, sdt)
            yield p + "mlp.experts.gate_up_proj.weight_packed", gu["qweight"].view(E, 2 * I, H // 8)
            yield p + "mlp.experts.gate_up_proj.weight_scale", gu["scales"].view(E, 2 * I, H // G)
            yield p + "mlp.experts.down_proj.weight_packed", dn["qweight"].view(E, H, I // 8)
            yield p + "mlp.experts.down_proj.weight_scale", dn["scales"].view(E, H, I // G)
        else:
            sh = arch.intermediate_size
            mp = p + "mlp."
        yield from lin(mp + "gate_proj", sh, H)
        yield from lin(mp + "up_proj", sh, H)
        yield from lin(mp + "down_proj", H, sh)
    if not arch.tie_embeddings:
        yield "lm_head.weight", normal("lm_head", (V, H), seed, dtype=dtype, device=device)


def iter_deepseek_weights(arch: ModelArch, seed: int = 0, dtype=torch.bfloat16, device="cpu") -> Iterator[tuple[str, object]]:
    """DeepSeek MLA+MoE in GGUF block formats: routed experts IQ2_XXS (gate, up) and Q2_K (down),
    every other matrix Q8_0, norms and router in float."""
    from ..loaders.gguf import GGUFTensor
    from ..ops import gguf_quant as gq
    H, V, m, mo = arch.hidden_size, arch.vocab_size, arch.mla, arch.moe
    qk = m.qk_nope_dim + m.qk_rope_dim

    def q8(name, rows, K, scale=0.004):
        return GGUFTensor(gq.random_blocks(8, rows, K, zlib.crc32(name.encode()) + seed, scale, device), 8, (rows, K))

    def blocks(name, ty, E, rows, K, scale):
        raw = gq.random_blocks(ty, E * rows, K, zlib.crc32(name.encode()) + seed, scale, device)
        return GGUFTensor(raw.view(E, rows, -1), ty, (E, rows, K))

    yield "model.embed_tokens.weight", normal("embed", (V, H), seed, dtype=dtype, device=device)
    for i in range(arch.num_layers):
        p = f"model.layers.{i}."
        if m.q_lora_rank:
            yield p + "self_attn.q_a_proj.weight", q8(p + "qa", m.q_lora_rank, H)
            yield p + "self_attn.q_b_proj.weight", q8(p + "qb", arch.num_heads * qk, m.q_lora_rank)
        else:
            yield p + "self_attn.q_proj.weight", q8(p + "q", arch.num_heads * qk, H)
        yield p + "self_attn.kv_a_proj_with_mqa.weight", q8(p + "kva", m.kv_lora_rank + m.qk_rope_dim, H)
        yield p + "self_attn.kv_b_proj.weight", q8(p + "kvb", arch.num_heads * (m.qk_nope_dim + m.v_head_dim), m.kv_lora_rank)
        yield p + "self_attn.o_proj.weight", q8(p + "o", H, arch.num_heads * m.v_head_dim)
        if mo.num_experts and i >= mo.first_dense_layers:
            yield p + "mlp.gate.weight", normal(p + "router", (mo.num_experts, H), seed, dtype=torch.float32, device=device)
            yield p + "mlp.gate.e_score_correction_bias", normal(p + "rb", (mo.num_experts,), seed, 0.01, torch.float32, device)
            I = mo.expert_intermediate
            yield p + "mlp.experts.gate_proj.weight", blocks(p + "eg", 16, mo.num_experts, I, H, 0.02)
            yield p + "mlp.experts.up_proj.weight", blocks(p + "eu", 16, mo.num_experts, I, H, 0.02)
            yield p + "mlp.experts.down_proj.weight", blocks(p + "ed", 10, mo.num_experts, H, I, 0.02)
            if mo.shared_intermediate:
                yield p + "mlp.shared_experts.gate_proj.weight", q8(p + "sg", mo.shared_intermediate, H)
                yield p + "mlp.shared_experts.up_proj.weight", q8(p + "su", mo.shared_intermediate, H)
                yield p + "mlp.shared_experts.down_proj.weight", q8(p + "sd", H, mo.shared_intermediate)
        else:
            yield p + "mlp.gate_proj.weight", q8(p + "g", arch.intermediate_size, H)
            yield p + "mlp.up_proj.weight", q8(p + "u", arch.intermediate_size, H)
            yield p + "mlp.down_proj.weight", q8(p + "d", H, arch.intermediate_size)
    yield "lm_head.weight", q8("lm_head", V, H)


def iter_qwen35_weights(arch: ModelArch, seed: int = 0, dtype=torch.float32, device="cpu") -> Iterator[tuple[str, torch.Tensor]]:
    e = arch.extra
    nk, nv = int(e.get("linear_num_key_heads", 4)), int(e.get("linear_num_value_heads", 8))
    dk, dv, kw = int(e.get("linear_key_head_dim", 64)), int(e.get("linear_value_head_dim", 64)), int(e.get("linear_conv_kernel_dim", 4))
    H, I, V, hd = arch.hidden_size, arch.intermediate_size, arch.vocab_size, arch.head_dim
    gated = bool(e.get("attn_output_gate", True))

    def w(name, *shape, std=0.02):
        return normal(name, shape, seed, std, dtype, device)
    yield "model.embed_tokens.weight", w("embed", V, H)
    for i in range(arch.num_layers):
        p = f"model.layers.{i}."
        if arch.layer_type(i) == "linear":
            C = 2 * nk * dk + nv * dv
            yield p + "linear_attn.in_proj_qkv.weight", w(p + "qkv", C, H)
            yield p + "linear_attn.in_proj_z.weight", w(p + "z", nv * dv, H)
            yield p + "linear_attn.in_proj_b.weight", w(p + "b", nv, H)
            yield p + "linear_attn.in_proj_a.weight", w(p + "a", nv, H)
            yield p + "linear_attn.conv1d.weight", w(p + "conv", C, 1, kw, std=0.3)
            yield p + "linear_attn.A_log", w(p + "alog", nv, std=0.5).float()
            yield p + "linear_attn.dt_bias", w(p + "dt", nv, std=0.5).float()
            yield p + "linear_attn.out_proj.weight", w(p + "o", H, nv * dv)
        else:
            yield p + "self_attn.q_proj.weight", w(p + "q", arch.num_heads * hd * (2 if gated else 1), H)
            yield p + "self_attn.k_proj.weight", w(p + "k", arch.num_kv_heads * hd, H)
            yield p + "self_attn.v_proj.weight", w(p + "v", arch.num_kv_heads * hd, H)
            yield p + "self_attn.o_proj.weight", w(p + "o", H, arch.num_heads * hd)
        if arch.moe.num_experts > 0:
            EI = arch.moe.expert_intermediate
            yield p + "mlp.gate.weight", w(p + "router", arch.moe.num_experts, H, std=0.5)
            for ex in range(arch.moe.num_experts):
                yield p + f"mlp.experts.{ex}.gate_proj.weight", w(p + f"eg{ex}", EI, H)
                yield p + f"mlp.experts.{ex}.up_proj.weight", w(p + f"eu{ex}", EI, H)
                yield p + f"mlp.experts.{ex}.down_proj.weight", w(p + f"ed{ex}", H, EI)
            if arch.moe.shared_intermediate > 0:
                SI = arch.moe.shared_intermediate
                yield p + "mlp.shared_expert.gate_proj.weight", w(p + "sg", SI, H)
                yield p + "mlp.shared_expert.up_proj.weight", w(p + "su", SI, H)
                yield p + "mlp.shared_expert.down_proj.weight", w(p + "sd", H, SI)
                yield p + "mlp.shared_expert_gate.weight", w(p + "sgate", 1, H, std=0.5)
        else:
            yield p + "mlp.gate_proj.weight", w(p + "g", I, H)
            yield p + "mlp.up_proj.weight", w(p + "u", I, H)
            yield p + "mlp.down_proj.weight", w(p + "d", H, I)
    yield "lm_head.weight", w("lm_head", V, H)
