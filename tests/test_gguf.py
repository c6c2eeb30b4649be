"""GGUF reader/writer round trip and header validation (CPU)."""
import struct

import pytest
import torch

from litevllm_b200.loaders.gguf import GGUFFile, GGUFTensor, gguf_to_hf_name, hf_config_from_gguf, write_gguf
from litevllm_b200.ops import gguf_quant as gq


def test_round_trip(tmp_path):
    raw = gq.random_blocks(gq.GGML_TYPES["Q2_K"], 6, 512, seed=1)
    tensors = {"token_embd.weight": torch.randn(10, 8), "blk.0.attn_q.weight": GGUFTensor(raw, 10, (6, 512)),
               "blk.0.ffn_down_exps.weight": GGUFTensor(gq.random_blocks(16, 2 * 4, 256, 2).view(2, 4, -1), 16, (2, 4, 256)),
               "blk.0.attn_norm.weight": torch.ones(8, dtype=torch.float16)}
    meta = {"general.architecture": "llama", "llama.block_count": 1, "llama.embedding_length": 8,
            "llama.attention.head_count": 2, "llama.rope.freq_base": 10000.0, "general.name": "t",
            "llama.some_list": [1, 2, 3]}
    f = tmp_path / "m.gguf"
    write_gguf(f, meta, tensors)
    g = GGUFFile(f)
    assert g.arch() == "llama" and g.metadata["llama.some_list"] == [1, 2, 3]
    assert torch.equal(g.load("token_embd.weight"), tensors["token_embd.weight"])
    q = g.load("blk.0.attn_q.weight")
    assert q.ggml_type == 10 and q.shape == (6, 512) and torch.equal(q.raw, raw)
    e = g.load("blk.0.ffn_down_exps.weight")
    assert e.shape == (2, 4, 256) and e.raw.shape == (2, 4, 66)
    cfg = hf_config_from_gguf(f)
    assert cfg["hidden_size"] == 8 and cfg["architectures"] == ["LlamaForCausalLM"]
    assert gguf_to_hf_name("blk.3.ffn_gate_exps.weight") == "model.layers.3.mlp.experts.gate_proj.weight"
    assert gguf_to_hf_name("blk.3.exp_probs_b.bias") == "model.layers.3.mlp.gate.e_score_correction_bias"


def test_rejects_bad_files(tmp_path):
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"NOPE" + b"\0" * 64)
    with pytest.raises(ValueError, match="magic"):
        GGUFFile(bad)
    v2 = tmp_path / "v2.gguf"
    v2.write_bytes(struct.pack("<IIQQ", 0x46554747, 2, 0, 0) + b"\0" * 32)
    with pytest.raises(ValueError, match="version 3"):
        GGUFFile(v2)
    trunc = tmp_path / "trunc.gguf"
    write_gguf(trunc, {"general.architecture": "llama"}, {"a.weight": torch.randn(64, 64)})
    data = trunc.read_bytes()
    trunc.write_bytes(data[: len(data) - 4096])
    with pytest.raises(ValueError, match="past the end"):
        GGUFFile(trunc)


def _gguf_str(b: bytes) -> bytes:
    return struct.pack("<Q", len(b)) + b


def test_rejects_overflowing_sizes(tmp_path):
    """Sizes taken from an untrusted file must not wrap a pointer or a 64-bit product."""
    head = struct.pack("<IIQQ", 0x46554747, 3, 1, 0)
    # (a) a tensor name whose length field is close to 2^64
    f = tmp_path / "hugestr.gguf"
    f.write_bytes(head + struct.pack("<Q", 0xFFFFFFFFFFFFFFF0) + b"x" * 64)
    with pytest.raises(ValueError):
        GGUFFile(f)
    # (b) dims whose product wraps to a small number
    f = tmp_path / "hugedims.gguf"
    f.write_bytes(head + _gguf_str(b"a.weight") + struct.pack("<I", 2) + struct.pack("<QQ", 1 << 63, 4) +
                  struct.pack("<IQ", 0, 0) + b"\0" * 64)
    with pytest.raises(ValueError, match="overflow"):
        GGUFFile(f)
    # (c) offset = UINT64_MAX with alignment 1: data_start + offset + nbytes must not wrap below the file size
    kv = _gguf_str(b"general.alignment") + struct.pack("<II", 4, 1)
    f = tmp_path / "hugeoff.gguf"
    f.write_bytes(struct.pack("<IIQQ", 0x46554747, 3, 1, 1) + kv + _gguf_str(b"a.weight") + struct.pack("<I", 1) +
                  struct.pack("<Q", 8) + struct.pack("<IQ", 0, 0xFFFFFFFFFFFFFFFF) + b"\0" * 64)
    with pytest.raises(ValueError, match="past the end"):
        GGUFFile(f)
    # (d) a tensor count that the file cannot possibly hold
    f = tmp_path / "manytensors.gguf"
    f.write_bytes(struct.pack("<IIQQ", 0x46554747, 3, 1 << 23, 0) + b"\0" * 64)
    with pytest.raises(ValueError, match="implausible"):
        GGUFFile(f)


def _hf_to_gguf_name(name: str) -> str:
    from litevllm_b200.loaders.gguf import _LAYER_MAP
    if name == "model.embed_tokens.weight":
        return "token_embd.weight"
    if name == "lm_head.weight":
        return "output.weight"
    if name == "model.norm.weight":
        return "output_norm.weight"
    parts = name.split(".")
    layer, rest = parts[2], ".".join(parts[3:])
    inv = {v: k for k, v in _LAYER_MAP.items()}
    if rest == "mlp.gate.e_score_correction_bias":
        return f"blk.{layer}.exp_probs_b.bias"
    mod, _, suffix = rest.rpartition(".")
    return f"blk.{layer}.{inv[mod]}.{suffix}"


def test_deepseek_gguf_file_end_to_end(tmp_path):
    """A synthetic DeepSeek-style GGUF file (Q8_0 / IQ2_XXS / Q2_K tensors under GGUF names) loads
    through ``LLM(path)`` and generates exactly what the in-memory synthetic model generates."""
    from litevllm_b200 import LLM, SamplingParams
    from litevllm_b200.loaders import synth
    from litevllm_b200.models.arch import arch_from_hf_config
    from litevllm_b200.models.presets import get_preset
    cfg = get_preset("tiny-deepseek-test")
    arch = arch_from_hf_config(cfg)
    tensors = {_hf_to_gguf_name(n): t for n, t in synth.iter_deepseek_weights(arch, 0, torch.float32, "cpu")}
    meta = {"general.architecture": "deepseek2", "deepseek2.block_count": 2, "deepseek2.embedding_length": 256,
            "deepseek2.attention.head_count": 4, "deepseek2.attention.head_count_kv": 4,
            "deepseek2.feed_forward_length": 256, "deepseek2.attention.layer_norm_rms_epsilon": 1e-6,
            "deepseek2.rope.freq_base": 10000.0, "deepseek2.context_length": 512, "deepseek2.vocab_size": 512,
            "deepseek2.attention.q_lora_rank": 64, "deepseek2.attention.kv_lora_rank": 64,
            "deepseek2.rope.dimension_count": 64, "deepseek2.attention.key_length": 128,
            "deepseek2.attention.value_length": 64, "deepseek2.expert_count": 8, "deepseek2.expert_used_count": 2,
            "deepseek2.expert_shared_count": 1, "deepseek2.expert_feed_forward_length": 256,
            "deepseek2.leading_dense_block_count": 0, "deepseek2.expert_weights_scale": 1.0,
            "deepseek2.expert_weights_norm": True, "deepseek2.expert_gating_func": 2,
            "tokenizer.ggml.eos_token_id": 1}
    f = tmp_path / "tiny-deepseek.gguf"
    write_gguf(f, meta, tensors)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (5, 20)]
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    kw = dict(dtype="float32", device="cpu", max_num_seqs=2, max_model_len=64)
    from_file = [o.outputs[0].token_ids for o in LLM(str(f), **kw).generate(prompts, sp)]
    in_memory = [o.outputs[0].token_ids for o in LLM("synthetic:tiny-deepseek-test", **kw).generate(prompts, sp)]
    assert from_file == in_memory


# ----------------------------------------------------------------------------- block decoders, weights, policy
@pytest.mark.parametrize("name", ["Q4_0", "Q4_K", "Q6_K", "Q8_0", "Q2_K", "IQ2_XXS"])
def test_block_decoders_match_the_gguf_package(name):
    """The PyTorch reference decoder of every supported block type against the ``gguf`` package's own
    numpy decoder (bit-exact: both are straight transcriptions of the block layouts)."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    ty = gq.GGML_TYPES[name]
    raw = gq.random_blocks(ty, 7, 768, seed=11)
    mine = gq.dequantize(raw, ty, 768)
    want = torch.from_numpy(quants.dequantize(raw.numpy(), getattr(gguf.GGMLQuantizationType, name)))
    assert torch.equal(mine, want)


def test_gguf_weight_policy_and_audit_cpu():
    from litevllm_b200.layers.quantization import tensor as qt
    K, N = 256, 24
    raw = gq.random_blocks(gq.GGML_TYPES["Q4_K"], N, K, seed=2)
    w = qt.GGUFWeight(raw, "Q4_K", K, prefix="model.layers.0.mlp.down_proj")
    x = torch.randn(5, K)
    want = x @ gq.dequantize(raw, 12, K).t()
    qt.reset_runtime_stats()
    qt.enable_audit(True)
    try:
        pol_all = qt.resolve_execution_policy(scope="all")
        pol_attn = qt.resolve_execution_policy(scope="attention_only")
        pol_hf = qt.resolve_execution_policy(scope="all", high_fidelity_prefixes=("down_proj",))
        assert qt.should_use_native_path(w.prefix, pol_all) == (True, "scope all")
        assert qt.should_use_native_path(w.prefix, pol_attn)[0] is False
        assert qt.should_use_native_path("model.layers.0.self_attn.qkv_proj", pol_attn)[0] is True
        assert qt.should_use_native_path(w.prefix, pol_hf) == (False, "high-fidelity prefix 'down_proj'")
        with pytest.raises(ValueError):
            qt.resolve_execution_policy(scope="sometimes")
        for pol in (pol_all, pol_attn, pol_attn, pol_hf):
            y = w.matmul(x, policy=pol)
            assert torch.allclose(y, want, atol=1e-4, rtol=1e-4)
        summ = qt.audit_summary()
        assert summ["counters"]["gguf.native"] == 1 and summ["counters"]["gguf.dense"] == 1
        assert summ["counters"]["gguf.dense_cached"] == 2          # the dense copy was reused twice
        row = summ["prefixes"][w.prefix]
        assert row["calls"] == 4 and row["tokens"] == 20 and row["native"] == 1 and row["dense"] == 3
        assert summ["recent_events"][-1]["reason"].startswith("high-fidelity")
        assert summ["dense_cache"]["entries"] >= 1
    finally:
        qt.enable_audit(False)
        qt.clear_global_weight_cache()
    with pytest.raises(ValueError):
        qt.GGUFWeight(raw[:, :-1], "Q4_K", K)
    # byte-bounded LRU
    c = qt.LRUWeightCache(max_size=8, max_bytes=4 * 100 * 4)
    for i in range(6):
        c.put(i, torch.zeros(100))
    assert c.get_memory_stats()["entries"] == 4 and c.get(0) is None and c.get(5) is not None
    assert c.put(99, torch.zeros(10000)) is False
