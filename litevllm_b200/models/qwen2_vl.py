"""Qwen2-VL style model: the Llama/Qwen2 text decoder of this engine plus a ViT image tower; image
soft tokens replace the ``<image>`` placeholder embeddings.  Rotary positions use the multimodal
(t, h, w) scheme; for text tokens the three streams coincide, image tokens advance h/w inside their
grid (``freq_stream`` of the rotary kernel selects the stream per frequency).
Reference: vllm/model_executor/models/qwen2_vl.py:16-251 (experimental image input)."""
from __future__ import annotations

import torch

from .gemma4_vision import Gemma4VisionTower
from .llama import LlamaForCausalLM


class Qwen2VLForConditionalGeneration(LlamaForCausalLM):
    supports_multimodal = True
    supports_lora = False

    def __init__(self, vllm_config):
        super().__init__(vllm_config)
        arch = vllm_config.model_config.arch
        if arch.vision is None:
            arch.vision = {"patch_size": 14, "hidden_size": 256, "num_hidden_layers": 2, "tokens_per_image": 16}
        self.vision_tower = Gemma4VisionTower(arch, vllm_config.model_config.dtype)
        self.mrope_section = arch.extra.get("mrope_section")

    def get_multimodal_embeddings(self, **mm_inputs):
        return self.vision_tower(mm_inputs["pixel_patches"], mm_inputs["position_ids"], mm_inputs["patches_per_image"])
