"""DeepSeek-V4-Flash building blocks: quantisation-aware round trips, the lightning indexer, the
shared-latent (K = V) attention with sinks over sliding-window and compressed rows, the KV compressor
state machine, manifold hyper-connections and the hash / sqrt-softplus routers.  Batched PyTorch
implementations (the CPU path and the oracle) with native kernels for the per-token hot pieces.
``model.py`` assembles them into ``DeepseekV4FlashForCausalLM``, a model that owns its per-request rows and
returns token ids (``executors.py`` adapts it to the engine).  The serving benchmark's MLA + MoE GGUF
configuration runs on ``models/deepseek_mla.py``.
Reference: vllm/model_executor/models/deepseek_v4_flash/ (attention.py, ops.py, moe.py,
hyper_connection.py, compressed_kv.py) and vllm/kernels/triton/deepseek_v4_flash/."""
from .attention import (CompressorState, compressed_row_attention, compressor_step, indexer_scores, indexer_topk,
                        shared_kv_attention, update_latent_cache)
from .hyper_connection import HyperConnectionState, hyper_connection_post, hyper_connection_pre, sinkhorn
from .model import DeepseekV4FlashForCausalLM, V4Config
from .moe import hash_routed_expert_ids, sqrt_softplus_router
from .ops import e2m1_roundtrip, fp8_kv_qat, hadamard128, indexer_qat, q8_k_roundtrip

__all__ = ["CompressorState", "compressed_row_attention", "compressor_step", "indexer_scores", "indexer_topk",
           "shared_kv_attention", "update_latent_cache", "HyperConnectionState", "hyper_connection_post",
           "hyper_connection_pre", "sinkhorn", "hash_routed_expert_ids", "sqrt_softplus_router", "e2m1_roundtrip",
           "fp8_kv_qat", "hadamard128", "indexer_qat", "q8_k_roundtrip", "DeepseekV4FlashForCausalLM", "V4Config"]
