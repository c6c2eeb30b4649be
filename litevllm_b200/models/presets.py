"""HF-style config dicts for the architectures the benchmarks name.  ``synthetic:<name>`` as a model
path builds one of these with random-init weights (no checkpoint files needed)."""
from __future__ import annotations

import copy

PRESETS: dict[str, dict] = {
    # TinyLlama-1.1B: 22 layers, hidden 2048, 32 q / 4 kv heads, head_dim 64, FFN 5632, vocab 32000
    "tinyllama-1.1b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 2048,
        "num_hidden_layers": 22, "num_attention_heads": 32, "num_key_value_heads": 4,
        "intermediate_size": 5632, "vocab_size": 32000, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
        "max_position_embeddings": 4096, "hidden_act": "silu", "tie_word_embeddings": False,
        "eos_token_id": 2, "bos_token_id": 1,
    },
    # 9B dense GQA decoder with zero-point AWQ int4 (group 128)
    "dense-9b-awq": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 4096,
        "num_hidden_layers": 36, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
        "intermediate_size": 12288, "vocab_size": 151936, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
        "max_position_embeddings": 4096, "hidden_act": "silu", "tie_word_embeddings": False,
        "eos_token_id": 151645,
        "quantization_config": {"quant_method": "awq", "bits": 4, "group_size": 128, "zero_point": True},
    },
    # Gemma4-26B-A4B-shaped MoE
    "gemma4-26b-a4b": {
        "architectures": ["Gemma4ForConditionalGeneration"], "model_type": "gemma4",
        "text_config": {
            "model_type": "gemma4_text", "hidden_size": 2816, "num_hidden_layers": 30,
            "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 256,
            "intermediate_size": 2112, "vocab_size": 262144, "rms_norm_eps": 1e-6,
            "sliding_window": 1024, "sliding_window_pattern": 6, "attn_logit_softcapping": 50.0,
            "final_logit_softcapping": 30.0, "rope_local_base_freq": 10000.0,
            "rope_global_base_freq": 1000000.0, "max_position_embeddings": 4096,
            "num_experts": 128, "top_k_experts": 8, "moe_intermediate_size": 704,
            "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True, "eos_token_id": 1,
        },
        "quantization_config": {"quant_method": "compressed-tensors", "format": "pack-quantized",
                                "config_groups": {"group_0": {"weights": {"num_bits": 4, "group_size": 32,
                                                                           "symmetric": True}}}},
    },
    # DeepSeek-V3-style MLA + MoE (GGUF-quantised in the named config)
    "deepseek-mla-moe": {
        "architectures": ["DeepseekV3ForCausalLM"], "model_type": "deepseek_v3", "hidden_size": 4096,
        "num_hidden_layers": 43, "num_attention_heads": 64, "num_key_value_heads": 64,
        "q_lora_rank": 1024, "kv_lora_rank": 512, "qk_rope_head_dim": 64, "qk_nope_head_dim": 128,
        "v_head_dim": 128, "intermediate_size": 2048, "moe_intermediate_size": 2048,
        "n_routed_experts": 256, "num_experts_per_tok": 6, "n_shared_experts": 1,
        "scoring_func": "sigmoid", "norm_topk_prob": True, "routed_scaling_factor": 1.0,
        "first_k_dense_replace": 0, "vocab_size": 129280, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
        "max_position_embeddings": 4096, "eos_token_id": 1,
        "quantization_config": {"quant_method": "gguf"},
    },
}

# Small variants for tests (same code paths, seconds on a CPU).
PRESETS["tiny-llama-test"] = dict(PRESETS["tinyllama-1.1b"], hidden_size=256, num_hidden_layers=2,
                                  num_attention_heads=4, num_key_value_heads=2, intermediate_size=256,
                                  vocab_size=512, max_position_embeddings=512)
PRESETS["tiny-llama-awq-test"] = dict(PRESETS["tiny-llama-test"], quantization_config={
    "quant_method": "awq", "bits": 4, "group_size": 128, "zero_point": True})
PRESETS["tiny-llama-ct-test"] = dict(PRESETS["tiny-llama-test"], quantization_config={
    "quant_method": "compressed-tensors", "format": "pack-quantized",
    "config_groups": {"group_0": {"weights": {"num_bits": 4, "group_size": 32, "symmetric": True}}}})
PRESETS["tiny-gemma4-moe-test"] = {
    "architectures": ["Gemma4ForConditionalGeneration"], "model_type": "gemma4",
    "text_config": {"model_type": "gemma4_text", "hidden_size": 256, "num_hidden_layers": 3,
                    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 192,
                    "vocab_size": 512, "rms_norm_eps": 1e-6, "sliding_window": 32, "sliding_window_pattern": 3,
                    "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0, "rope_local_base_freq": 10000.0,
                    "rope_global_base_freq": 1000000.0, "max_position_embeddings": 512, "num_experts": 8,
                    "top_k_experts": 2, "moe_intermediate_size": 128, "tie_word_embeddings": True, "eos_token_id": 1},
    "quantization_config": {"quant_method": "compressed-tensors", "format": "pack-quantized",
                            "config_groups": {"group_0": {"weights": {"num_bits": 4, "group_size": 32,
                                                                       "symmetric": True}}}},
}
PRESETS["tiny-deepseek-test"] = dict(PRESETS["deepseek-mla-moe"], hidden_size=256, num_hidden_layers=2,
                                     num_attention_heads=4, num_key_value_heads=4, q_lora_rank=64, kv_lora_rank=64,
                                     qk_rope_head_dim=64, qk_nope_head_dim=64, v_head_dim=64, intermediate_size=256,
                                     moe_intermediate_size=256, n_routed_experts=8, num_experts_per_tok=2,
                                     vocab_size=512, max_position_embeddings=512)
# the latent geometry of the full-size model (512 + 64) with 20 heads: exercises the absorbed attention kernel
PRESETS["tiny-deepseek-mla512-test"] = dict(PRESETS["tiny-deepseek-test"], num_attention_heads=20, num_key_value_heads=20,
                                            kv_lora_rank=512, qk_nope_head_dim=128, v_head_dim=128)
# DeepSeek-V4-Flash geometry in miniature: 512-wide shared latent rows, a window shorter than the test prompts,
# two window-only layers, then a fine (ratio 4, indexer top-k smaller than the emitted rows) and a coarse
# (ratio 8, all rows) compressed layer
PRESETS["tiny-deepseek-v4-flash-test"] = {
    "architectures": ["DeepseekV4FlashForCausalLM"], "model_type": "deepseek_v4_flash", "hidden_size": 256,
    "num_hidden_layers": 4, "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 512,
    "qk_rope_head_dim": 64, "q_lora_rank": 64, "sliding_window": 8, "compress_ratio_coarse": 8, "index_n_heads": 2,
    "index_topk": 3, "hc_mult": 4, "o_groups": 2, "o_lora_rank": 32, "n_routed_experts": 8,
    "num_experts_per_tok": 2, "moe_intermediate_size": 256, "num_hash_layers": 1, "routed_scaling_factor": 1.5,
    "vocab_size": 512, "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "max_position_embeddings": 512,
    "intermediate_size": 256, "eos_token_id": 1,
}
# the same with random weights in the checkpoint's block formats (IQ2_XXS / Q2_K routed experts, Q8_0 projections)
PRESETS["tiny-deepseek-v4-flash-blocks-test"] = dict(PRESETS["tiny-deepseek-v4-flash-test"], synthetic_block_weights=True)
# the full-size geometry of the DeepSeek-V4-Flash checkpoint family; as a synthetic model its weights are random
# blocks in the checkpoint's formats (IQ2_XXS / Q2_K experts, Q8_0 projections: about 90 GB)
PRESETS["deepseek-v4-flash"] = {
    "architectures": ["DeepseekV4FlashForCausalLM"], "model_type": "deepseek_v4_flash", "hidden_size": 4096,
    "num_hidden_layers": 43, "num_attention_heads": 64, "num_key_value_heads": 1, "head_dim": 512,
    "qk_rope_head_dim": 64, "q_lora_rank": 1024, "sliding_window": 128, "index_n_heads": 64, "index_topk": 512,
    "hc_mult": 4, "o_groups": 8, "o_lora_rank": 1024, "n_routed_experts": 256, "num_experts_per_tok": 6,
    "moe_intermediate_size": 2048, "num_hash_layers": 3, "routed_scaling_factor": 1.5, "swiglu_limit": 10.0,
    "vocab_size": 129280, "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "max_position_embeddings": 65536,
    "intermediate_size": 2048, "eos_token_id": 1, "synthetic_block_weights": True,
}
PRESETS["tiny-qwen35-test"] = {
    "architectures": ["Qwen3_5ForCausalLM"], "model_type": "qwen3_5", "hidden_size": 256, "num_hidden_layers": 4,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 256, "vocab_size": 512,
    "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "max_position_embeddings": 512, "partial_rotary_factor": 0.25,
    "full_attention_interval": 4, "linear_num_key_heads": 2, "linear_num_value_heads": 4, "linear_key_head_dim": 32,
    "linear_value_head_dim": 32, "linear_conv_kernel_dim": 4, "attn_output_gate": True, "eos_token_id": 1,
}
PRESETS["tiny-qwen35-moe-test"] = dict(PRESETS["tiny-qwen35-test"], architectures=["Qwen3_5MoeForCausalLM"],
                                      num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
                                      shared_expert_intermediate_size=128, norm_topk_prob=True)
PRESETS["tiny-qwen3-test"] = dict(PRESETS["tiny-llama-test"], architectures=["Qwen3ForCausalLM"], model_type="qwen3",
                                  head_dim=64)
PRESETS["tiny-qwen2vl-test"] = dict(PRESETS["tiny-llama-test"], architectures=["Qwen2VLForConditionalGeneration"],
                                    model_type="qwen2_vl", attention_bias=True,
                                    vision_config={"patch_size": 14, "embed_dim": 64, "depth": 2, "num_heads": 2,
                                                   "spatial_merge_size": 2, "temporal_patch_size": 2, "mlp_ratio": 2,
                                                   "min_pixels": 28 * 28, "max_pixels": 28 * 28 * 16},
                                    rope_scaling={"type": "mrope", "mrope_section": [16, 8, 8]})


def get_preset(name: str) -> dict:
    key = name.lower()
    if key not in PRESETS:
        raise KeyError(f"unknown synthetic preset {name!r}; known: {sorted(PRESETS)}")
    return copy.deepcopy(PRESETS[key])
