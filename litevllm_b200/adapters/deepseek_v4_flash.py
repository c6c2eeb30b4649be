"""DeepSeek-V4-Flash adapter: the model owns its data plane (per-request latent, compressed and indexer
rows), so the adapter swaps in token-returning executors, frees the model's rows when a request is
released, and narrows what a request may ask for: greedy decoding only, no LoRA, no images, and an admission
cap derived from a byte budget for the per-request rows.
Reference: vllm/adapters/deepseek_v4_flash.py:24-193."""
from __future__ import annotations

import os

from ..engine.custom_runtime_components import CustomRuntimeComponents
from ..engine.errors import InvalidRequestError
from .base import ModelAdapter, ModelCapabilities, RuntimeModelPolicy


def _row_bytes_per_request(v4: dict, max_len: int) -> int:
    """Upper bound of one request's rows at ``max_len`` tokens (fp32 rows): a window per layer, one compressed
    row per ``ratio`` tokens on the compressed layers, plus a 128-wide indexer row on the ratio-4 layers."""
    from ..models.deepseek_v4_flash.model import V4Config
    layers, D = int(v4.get("num_hidden_layers", 1)), int(v4.get("head_dim", 512))
    window = int(v4.get("sliding_window", 128))
    ratios = v4.get("layer_compress_ratios") or V4Config.default_ratios(layers, int(v4.get("compress_ratio_coarse", 128)))
    total = layers * window * D * 4
    for r in ratios:
        if r > 0:
            total += (max_len // int(r)) * (D + (128 if int(r) == 4 else 0)) * 4
    return total


class DeepSeekV4FlashAdapter(ModelAdapter):
    name = "deepseek_v4_flash"

    @classmethod
    def matches(cls, arch) -> bool:
        return arch.family == "deepseek_v4_flash"

    def runtime_policy(self, runtime_config) -> RuntimeModelPolicy:
        budget = float(os.environ.get("FI_V4_ROWS_BUDGET_GB", "8")) * 2 ** 30
        hf = self.arch.extra.get("v4_rows", {})
        max_len = int(getattr(runtime_config, "max_model_len", 0) or self.arch.max_position)
        per_req = max(1, _row_bytes_per_request(hf, max_len))
        cap = max(1, int(budget // per_req))
        return RuntimeModelPolicy(prefill_chunk_size=512, admission_cap=cap,
                                  model_policy={"model_owned_data_plane": True, "rows_budget_bytes": int(budget),
                                                "rows_bytes_per_request": per_req})

    def detect(self, model) -> ModelCapabilities:
        return ModelCapabilities(supports_lora=False, supports_multimodal=False, supports_prefix_cache=False,
                                 supports_sampling=False, supports_cuda_graph=False)

    def validate_request(self, sampling_params, prompt_len, lora_request=None, multi_modal_data=None) -> None:
        if lora_request is not None:
            raise InvalidRequestError("DeepSeek-V4-Flash does not support LoRA adapters")
        if multi_modal_data:
            raise InvalidRequestError("DeepSeek-V4-Flash is text only")
        sp = sampling_params
        if sp is not None:
            if getattr(sp, "temperature", 0.0) not in (0, 0.0) or getattr(sp, "n", 1) != 1:
                raise InvalidRequestError("DeepSeek-V4-Flash decodes greedily: temperature must be 0 and n must be 1")
            if getattr(sp, "logprobs", None) or getattr(sp, "logits_processors", None):
                raise InvalidRequestError("DeepSeek-V4-Flash returns token ids only: no logprobs or logits processors")

    def build_executors(self, engine) -> CustomRuntimeComponents:
        from ..models.deepseek_v4_flash.executors import V4FlashDecodeExecutor, V4FlashPrefillExecutor
        model = engine.model
        stock_release = engine._on_release

        def release(st) -> None:
            if model.release_request(st.request_id):
                hook = getattr(engine.observer, "on_model_event", None)
                if callable(hook):
                    hook("rows_released", request_id=st.request_id, **model.kv_stats())
            stock_release(st)

        engine._on_release = release
        return CustomRuntimeComponents(V4FlashPrefillExecutor(model, engine.observer),
                                       V4FlashDecodeExecutor(model, engine.observer), None)
