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
    if not arch.tie_embeddings:
        yield "lm_head.weight", normal("lm_head", (V, H), seed, dtype=dtype, device=device)
