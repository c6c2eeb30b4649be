"""DeepSeek-V4-Flash through the engine: the model owns its per-request rows and returns token ids; the
adapter swaps the executors, caps admission and narrows requests to greedy decoding.
Reference behaviour: vllm/model_executor/models/deepseek_v4_flash/model.py (prefill_request /
decode_tokens_batch), vllm/adapters/deepseek_v4_flash.py."""
import pytest
import torch

from litevllm_b200 import LLM, SamplingParams
from litevllm_b200.engine.errors import InvalidRequestError

PRESET = "synthetic:tiny-deepseek-v4-flash-test"
PROMPTS = [[(7 * i + 3) % 500 + 2 for i in range(30)], [(11 * i + 5) % 500 + 2 for i in range(21)]]


def _greedy(n):
    return SamplingParams(max_tokens=n, temperature=0.0, ignore_eos=True)


@pytest.fixture(scope="module")
def llm():
    return LLM(PRESET, device="cpu", max_model_len=128, dtype="float32")


def _tokens(llm, prompts, n):
    return [list(o.outputs[0].token_ids) for o in llm.generate([{"prompt_token_ids": p} for p in prompts], _greedy(n))]


def test_adapter_and_executors_selected(llm):
    from litevllm_b200.adapters.deepseek_v4_flash import DeepSeekV4FlashAdapter
    from litevllm_b200.models.deepseek_v4_flash.executors import V4FlashDecodeExecutor, V4FlashPrefillExecutor
    eng = llm.engine
    assert isinstance(eng.adapter, DeepSeekV4FlashAdapter)
    assert isinstance(eng.backend.prefill_executor, V4FlashPrefillExecutor)
    assert isinstance(eng.backend.decode_executor, V4FlashDecodeExecutor)
    assert eng.model_policy.admission_cap >= 1
    assert not eng.capabilities.supports_sampling and not eng.capabilities.supports_lora


def test_decode_continues_like_a_longer_prefill(llm):
    """Tokens 7..12 of a generation equal the first 6 tokens generated from prompt + tokens 1..6: the rows a
    decode step appends (window ring, compressor state, emitted rows, indexer rows) are the rows a prefill of
    the longer prompt builds."""
    first = _tokens(llm, PROMPTS[:1], 12)[0]
    again = _tokens(llm, [PROMPTS[0] + first[:6]], 6)[0]
    assert again == first[6:]
    assert len(set(first)) > 4                       # not a degenerate repetition


def test_batched_decode_equals_single_requests(llm):
    together = _tokens(llm, PROMPTS, 10)
    alone = [_tokens(llm, [p], 10)[0] for p in PROMPTS]
    assert together == alone


def test_chunked_prefill_equals_one_chunk(llm):
    model = llm.engine.model
    one = model.prefill_request("a", PROMPTS[0], 0, True)
    assert model.prefill_request("b", PROMPTS[0][:13], 0, False) is None
    two = model.prefill_request("b", PROMPTS[0][13:], 13, True)
    assert one == two
    ra, rb = model.requests["a"], model.requests["b"]
    assert (ra.layers[0].window - rb.layers[0].window).abs().gt(1e-4).float().mean() < 0.002
    assert ra.pos == rb.pos == len(PROMPTS[0])
    for la, lb in zip(ra.layers, rb.layers):
        # the fp8 round trip may flip a rounding step where the two GEMM shapes differ in the last bit, and a
        # flipped step moves the later layers by a little
        assert (la.window - lb.window).abs().mean() < 5e-3
        assert len(la.compressed) == len(lb.compressed)
    # compressed layers emitted one row per `ratio` tokens, more than the indexer keeps
    cfg = model.cfg
    assert cfg.ratios == (0, 0, 4, 8)
    assert len(ra.layers[2].compressed) == len(ra.layers[2].index_rows) == len(PROMPTS[0]) // 4 > cfg.indexer_topk
    assert len(ra.layers[3].compressed) == len(PROMPTS[0]) // 8 and not ra.layers[3].index_rows
    assert not ra.layers[0].compressed and not ra.layers[1].compressed
    with pytest.raises(RuntimeError):
        model.prefill_request("b", [5, 6], 3, True)   # a chunk that does not continue where the rows end
    assert model.release_request("a") and model.release_request("b") and not model.release_request("a")


def test_rows_are_released_with_the_request(llm):
    model = llm.engine.model
    _tokens(llm, PROMPTS, 3)
    assert model.requests == {} and model.request_bytes() == 0


def test_requests_are_narrowed_to_greedy(llm):
    with pytest.raises(InvalidRequestError):
        llm.generate([{"prompt_token_ids": PROMPTS[1]}], SamplingParams(max_tokens=2, temperature=0.8))
    assert llm.engine.model.requests == {}


def test_admission_cap_follows_the_row_budget(monkeypatch):
    from litevllm_b200.adapters.deepseek_v4_flash import DeepSeekV4FlashAdapter, _row_bytes_per_request
    from litevllm_b200.models.arch import arch_from_hf_config
    from litevllm_b200.models.presets import PRESETS
    arch = arch_from_hf_config(PRESETS["tiny-deepseek-v4-flash-test"])
    assert arch.family == "deepseek_v4_flash"
    per = _row_bytes_per_request(arch.extra["v4_rows"], 512)
    monkeypatch.setenv("FI_V4_ROWS_BUDGET_GB", str(3.5 * per / 2 ** 30))

    class RC:
        max_model_len = 512
    assert DeepSeekV4FlashAdapter(arch).runtime_policy(RC()).admission_cap == 3


@pytest.mark.gpu
def test_gpu_tokens_match_cpu(llm):
    """fp32 on both sides: the GPU side runs the native shared-latent attention, indexer and QAT kernels."""
    want = _tokens(llm, PROMPTS, 8)
    gpu = LLM(PRESET, device="cuda", max_model_len=128, dtype="float32")
    got = _tokens(gpu, PROMPTS, 8)
    agree = sum(a == b for w, g in zip(want, got) for a, b in zip(w, g)) / sum(len(w) for w in want)
    assert got[0][0] == want[0][0] and got[1][0] == want[1][0]
    assert agree >= 0.75, (want, got)


def test_checkpoint_tensor_names_map_to_parameters(llm):
    """GGUF names of the checkpoint family land in the matching parameters, with layout adaptation."""
    model = llm.engine.model
    cls = type(model)
    assert cls.param_name("blk.2.indexer.attn_q_b.weight") == "layers.2.idx_q"
    assert cls.param_name("blk.3.attn_compressor_ape.weight") == "layers.3.comp_ape"
    assert cls.param_name("output_hc_fn.weight") == "out_hc_fn"
    names = {n for n, _ in model.named_parameters()} | {n for n, _ in model.named_buffers()}
    every = [f"blk.{i}.{s}" for i in range(model.cfg.layers) for s in cls._GGUF_LAYER] + list(cls._GGUF_TOP)
    mapped = {cls.param_name(n) for n in every}
    assert names <= mapped                                   # every parameter has a checkpoint name
    keep = model.layers[3].comp_ape.clone()
    try:
        new = torch.arange(keep.numel(), dtype=torch.float32).reshape(keep.shape)
        consumed = model.load_weights([("blk.3.attn_compressor_ape.weight", new.t().contiguous()),
                                       ("blk.9.unknown.weight", torch.zeros(1))])
        assert consumed == {"blk.3.attn_compressor_ape.weight"}
        torch.testing.assert_close(model.layers[3].comp_ape.float(), new)
        with pytest.raises(ValueError):
            model.load_weights([("output_norm.weight", torch.zeros(3))])
    finally:
        model.layers[3].comp_ape.data.copy_(keep)
