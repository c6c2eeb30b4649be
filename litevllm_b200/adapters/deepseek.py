"""DeepSeek adapter (MLA + MoE, GGUF): the generic MLA model runs through the ordinary executors, so only the
LoRA / multimodal restrictions apply.  The V4-Flash checkpoint family, whose model owns its data plane, has
its own adapter (``adapters/deepseek_v4_flash.py``)."""
from ..engine.errors import InvalidRequestError
from .base import ModelAdapter, ModelCapabilities, RuntimeModelPolicy


class DeepSeekAdapter(ModelAdapter):
    name = "deepseek"

    @classmethod
    def matches(cls, arch) -> bool:
        return arch.family == "deepseek_mla"

    def runtime_policy(self, runtime_config) -> RuntimeModelPolicy:
        return RuntimeModelPolicy(prefill_chunk_size=512, model_policy={"mla": True, "moe": bool(self.arch.moe.num_experts)})

    def detect(self, model) -> ModelCapabilities:
        return ModelCapabilities(supports_lora=False, supports_multimodal=False)

    def validate_request(self, sampling_params, prompt_len, lora_request=None, multi_modal_data=None) -> None:
        if lora_request is not None:
            raise InvalidRequestError("DeepSeek models do not support LoRA adapters")
        if multi_modal_data:
            raise InvalidRequestError("DeepSeek models are text only")
