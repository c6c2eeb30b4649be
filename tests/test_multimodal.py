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
    # 84 x 56 pixels -> 6 x 4 patches of 14 -> 3 x 2 merged tokens
    red = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": {"image": [_png_url(84, 56, (255, 0, 0))]}}], sp)
    blue = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": {"image": [_png_url(84, 56, (0, 0, 255))]}}], sp)
    assert len(red[0].prompt_token_ids) == 4 + 6
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


def test_qwen2vl_image_processor_and_mrope_positions():
    from litevllm_b200.models.qwen2_vl import Qwen2VLImageProcessor, mrope_positions, smart_resize
    assert smart_resize(30, 40, 28, 28 * 28, 28 * 28 * 16) == (28, 28)
    h, w = smart_resize(1000, 3000, 28, 56 * 56, 14 * 14 * 4 * 1280)
    assert h % 28 == 0 and w % 28 == 0 and h * w <= 14 * 14 * 4 * 1280 and abs(w / h - 3.0) < 0.25
    ip = Qwen2VLImageProcessor(min_pixels=28 * 28, max_pixels=28 * 28 * 16)
    img = decode_image(_png_url(84, 56, (10, 200, 30)))
    pv, grid = ip(img)
    assert grid == (1, 4, 6) and pv.shape == (24, 3 * 2 * 14 * 14) and ip.num_tokens(grid) == 6
    # CLIP normalisation of a constant image: every patch holds the same three channel values
    want = (torch.tensor([10, 200, 30]) / 255.0 - torch.tensor([0.48145466, 0.4578275, 0.40821073])) / \
        torch.tensor([0.26862954, 0.26130258, 0.27577711])
    got = pv.view(24, 3, 2, 14, 14)
    assert torch.allclose(got[:, :, 0, 0, 0], want.expand(24, 3), atol=2e-2)
    # positions: text, a 3 x 2 merged-grid image, text
    IMG = 99
    ids = [5, 6] + [IMG] * 6 + [7, 8]
    pos, delta = mrope_positions(ids, IMG, [grid])
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 2:8].tolist() == [2] * 6                               # one time step
    assert pos[1, 2:8].tolist() == [2, 2, 2, 3, 3, 3]                     # rows of the 2 x 3 merged grid
    assert pos[2, 2:8].tolist() == [2, 3, 4, 2, 3, 4]                     # columns
    assert pos[:, 8:].tolist() == [[5, 6]] * 3 and delta == 7 - 10
    with pytest.raises(ValueError):
        mrope_positions([5, IMG, IMG], IMG, [grid])


def test_qwen2vl_tower_shapes_and_image_confinement():
    from litevllm_b200.models.qwen2_vl import Qwen2VisionTransformer
    torch.manual_seed(0)
    vt = Qwen2VisionTransformer({"patch_size": 14, "embed_dim": 32, "depth": 2, "num_heads": 2, "mlp_ratio": 2}, 48,
                                torch.float32)
    a, b = torch.randn(16, vt.in_features), torch.randn(24, vt.in_features)
    both = vt(torch.cat([a, b]), [(1, 4, 4), (1, 4, 6)])
    alone = vt(a, [(1, 4, 4)])
    assert both.shape == (4 + 6, 48)
    assert torch.allclose(both[:4], alone, atol=1e-5)                    # attention does not cross images
    # HF checkpoint names load (conv patch embedding flattened, mlp / merger renamed)
    sd = {"visual.patch_embed.proj.weight": torch.randn(32, 3, 2, 14, 14),
          "visual.blocks.0.mlp.fc1.weight": torch.randn(64, 32), "visual.merger.mlp.2.bias": torch.randn(48)}
    used = vt.load_weights(sd.items())
    assert used == set(sd) and torch.equal(vt.blocks[0].fc1.weight, sd["visual.blocks.0.mlp.fc1.weight"])


def test_qwen2vl_decode_positions_continue_the_multimodal_streams():
    """Tokens decoded after an image prompt (position = index + delta on all three streams) must be what a
    fresh prefill of prompt + generated prefix (full three-stream positions) predicts."""
    from litevllm_b200 import LLM, SamplingParams
    llm = LLM("synthetic:tiny-qwen2vl-test", dtype="float32", device="cpu", max_num_seqs=2, max_model_len=128)
    ph = llm.engine.multimodal.image_token_id
    url = _png_url(84, 56, (30, 90, 200))
    first = llm.generate([{"prompt_token_ids": [5, 6, ph, 7, 8], "multi_modal_data": {"image": [url]}}],
                         SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))[0]
    full, gen = list(first.prompt_token_ids), list(first.outputs[0].token_ids)
    assert len(full) == 10
    one = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    for n in range(1, 4):
        nxt = llm.generate([{"prompt_token_ids": full + gen[:n], "multi_modal_data": {"image": [url]}}], one)[0]
        assert nxt.outputs[0].token_ids[0] == gen[n], (n, nxt.outputs[0].token_ids, gen)


def test_chat_request_with_image_blocks_over_http():
    """OpenAI message content as blocks: `image_url` data URLs reach the engine as images (placeholder expanded),
    a remote URL and an image for a text-only model are 400."""
    from fastapi.testclient import TestClient
    from litevllm_b200.entrypoints.openai import api_server as srv
    client = TestClient(srv.app)
    saved = (srv.engine, srv.served_model, srv.debug_endpoints_enabled)

    def body(url, model="vl"):
        return {"model": model, "temperature": 0, "max_tokens": 3,
                "messages": [{"role": "user", "content": [{"type": "text", "text": "what is this"},
                                                          {"type": "image_url", "image_url": {"url": url}}]}]}
    try:
        srv.engine = srv.build_engine("synthetic:tiny-qwen2vl-test", dtype="float32", device="cpu", max_num_seqs=2,
                                      max_model_len=256)
        srv.served_model = "vl"
        r = client.post("/v1/chat/completions", json=body(_png_url(84, 56)))
        assert r.status_code == 200, r.text
        assert r.json()["usage"]["completion_tokens"] == 3 and r.json()["usage"]["prompt_tokens"] > 6   # 6 image tokens + text
        assert srv.engine.stats()["multimodal"]["images"] == 1
        assert client.post("/v1/chat/completions", json=body("http://example.com/cat.png")).status_code == 400
        assert client.post("/v1/chat/completions", json=body("data:image/gif;base64,AAAA")).status_code == 400
        srv.engine.shutdown()
        srv.engine = srv.build_engine("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=2,
                                      max_model_len=128)
        srv.served_model = "txt"
        assert client.post("/v1/chat/completions", json=body(_png_url(), model="txt")).status_code == 400
    finally:
        if srv.engine is not None:
            srv.engine.shutdown()
        srv.engine, srv.served_model, srv.debug_endpoints_enabled = saved


def test_image_and_text_requests_share_steps_without_interfering():
    """Requests with and without images in the same steps (chunked prefill, one abort): a request's tokens are the
    ones it generates alone - placeholder expansion, embedding merge and the per-request rotary offset stay with
    their request."""
    import random
    from litevllm_b200 import LLM, SamplingParams
    cfg = {"profile": "balanced", "tuning_keyvals": {"FASTINFERENCE_LITE_PREFILL_CHUNK": "16", "FASTINFERENCE_MIN_PREFILL_CHUNK": "16",
                                                     "FASTINFERENCE_MAX_PREFILL_CHUNK": "16"}}
    llm = LLM("synthetic:tiny-qwen2vl-test", dtype="float32", device="cpu", max_num_seqs=3, max_model_len=160,
              fastinference_config=cfg)
    eng = llm.engine
    try:
        ph = eng.multimodal.image_token_id
        rng = random.Random(2)
        sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
        reqs = {}
        for i in range(7):
            ids = [rng.randint(5, 300) for _ in range(rng.randint(3, 12))]
            if i % 2 == 0:
                ids.insert(rng.randint(0, len(ids)), ph)
                color = (rng.randint(0, 255), rng.randint(0, 255), rng.randint(0, 255))
                reqs[f"m{i}"] = {"prompt_token_ids": ids, "multi_modal_data": {"image": [_png_url(84, 56, color)]}}
            else:
                reqs[f"m{i}"] = {"prompt_token_ids": ids}
        alone = {rid: llm.generate([p], sp)[0].outputs[0].token_ids for rid, p in reqs.items()}
        pending, finished = list(reqs), {}
        aborted = False
        while pending or eng.has_unfinished_requests():
            if pending and rng.random() < 0.7:
                rid = pending.pop()
                eng.add_request(rid, reqs[rid], sp)
            if not aborted and "m2" not in pending and "m2" not in finished and rng.random() < 0.3:
                aborted = eng.abort_request("m2")
            for o in eng.step():
                if o is not None and o.finished:
                    finished[o.request_id] = o.outputs[0].token_ids
        assert len(finished) >= 6 and all(finished[r] == alone[r] for r in finished)
        assert eng.kv_manager.allocator.num_free == eng.plan.num_total_blocks - 1
    finally:
        llm.shutdown()
