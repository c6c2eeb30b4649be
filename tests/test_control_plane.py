"""Control-plane units with hand-rolled fakes (no GPU, no model)."""
import asyncio
import time
from types import SimpleNamespace

import pytest
import torch

from litevllm_b200.config.runtime_policy import SchedulerRuntimePolicy
from litevllm_b200.engine.block_allocator import BlockAllocator
from litevllm_b200.engine.errors import InvalidRequestError, RequestRejectedError
from litevllm_b200.engine.kv_block_manager import KVBlockManager
from litevllm_b200.engine.kv_cache import FlatKVCache, KVLayerSpec
from litevllm_b200.engine.planners import AdmissionPlanner, BudgetComputer, DecodePrefillPlanner
from litevllm_b200.engine.prefix_cache import PrefixCache
from litevllm_b200.engine.request_scheduler import RequestScheduler
from litevllm_b200.engine.request_state import RequestState
from litevllm_b200.engine.step_plan import PrefillItem, StepPlan
from litevllm_b200.engine.step_scheduler import StepScheduler
from litevllm_b200.sampling_params import SamplingParams


def _req(rid, n_prompt=10, **kw):
    return RequestState(request_id=rid, prompt=None, prompt_token_ids=list(range(1, n_prompt + 1)),
                        sampling_params=SamplingParams(**kw))


# ----------------------------------------------------------------------------- block allocator
def test_block_allocator_reserves_null_block_and_detects_double_free():
    a = BlockAllocator(5)
    got = a.allocate(4)
    assert sorted(got) == [1, 2, 3, 4] and a.num_free == 0
    with pytest.raises(MemoryError):
        a.allocate(1)
    a.free([2, 0])            # freeing the null block is a no-op
    assert a.num_free == 1
    with pytest.raises(ValueError):
        a.free([2])
    assert a.allocate(1) == [2]


def test_flat_kv_cache_views_do_not_overlap():
    specs = [KVLayerSpec(2, 64), KVLayerSpec(1, 128)]
    kv = FlatKVCache(specs, num_blocks=4, block_size=16, dtype=torch.float32, device=torch.device("cpu"))
    for i, (k, v) in enumerate(kv.layers):
        k.fill_(i + 1)
        v.fill_(-(i + 1))
    for i, (k, v) in enumerate(kv.layers):
        assert float(k.min()) == float(k.max()) == i + 1
        assert float(v.min()) == float(v.max()) == -(i + 1)
    assert kv.layers[0][0].shape == (4, 2, 16, 64) and kv.layers[1][0].shape == (4, 1, 16, 128)


def test_kv_block_manager_grows_and_releases():
    alloc = BlockAllocator(1 + 2 * 4)
    m = KVBlockManager(alloc, 16, max_active=2, blocks_per_seq=4, device=torch.device("cpu"))
    m.register("a", 0)
    assert m.ensure_blocks("a", 1) and len(m.blocks_of("a")) == 1
    assert m.ensure_blocks("a", 16) == []          # still one block
    assert len(m.ensure_blocks("a", 17)) == 1
    m.flush()
    assert m.block_tables[0, :2].tolist() == m.blocks_of("a") and m.block_tables[0, 2:].sum() == 0
    with pytest.raises(ValueError):
        m.ensure_blocks("a", 16 * 4 + 1)
    m.release("a")
    m.release("a")                                  # idempotent
    m.flush()
    assert alloc.num_free == 8 and int(m.block_tables.sum()) == 0


# ----------------------------------------------------------------------------- request scheduler
def test_scheduler_fifo_slots_and_capacity():
    s = RequestScheduler(max_active=2, queue_capacity=3)
    for i in range(3):
        s.enqueue_request(_req(f"r{i}"))
    with pytest.raises(RequestRejectedError):
        s.enqueue_request(_req("r3"))
    with pytest.raises(InvalidRequestError):
        s.enqueue_request(_req("r0"))
    a = s.admit("r0")
    b = s.admit("r1")
    assert {a.slot_idx, b.slot_idx} == {0, 1} and not s.free_slots
    a.is_prefill = False
    pre, dec = s.classify_requests()
    assert [r.request_id for r in pre] == ["r1"] and [r.request_id for r in dec] == ["r0"]
    assert s.release("r0") is not None and s.release("r0") is None
    assert list(s.free_slots) == [0]
    assert s.gauges()["queued"] == 1


def test_scheduler_queue_timeout_expires_oldest_first():
    s = RequestScheduler(max_active=1, queue_timeout_s=10.0)
    old, new = _req("old"), _req("new")
    old.arrival_time -= 11.0
    s.enqueue_request(old)
    s.enqueue_request(new)
    expired = s.expire_queued()
    assert [e.request_id for e in expired] == ["old"] and list(s.queued) == ["new"]


def test_stream_gets_exactly_one_terminal_item():
    async def run():
        s = RequestScheduler(max_active=1)
        loop = asyncio.get_running_loop()
        s.enqueue_request(_req("x"), loop)
        s.publish_output("x", SimpleNamespace(finished=False, n=1))
        s.publish_output("x", SimpleNamespace(finished=True, n=2))
        s.publish_output("x", SimpleNamespace(finished=True, n=3))     # ignored: already terminal
        s.publish_output("x", RuntimeError("late"))                     # ignored too
        got = [o.n async for o in s.get_request_stream("x")]
        return got
    assert asyncio.run(run()) == [1, 2]


def test_stream_raises_published_exception():
    async def run():
        s = RequestScheduler(max_active=1)
        s.enqueue_request(_req("x"), asyncio.get_running_loop())
        s.publish_output("x", RequestRejectedError("nope", "queue_timeout"))
        with pytest.raises(RequestRejectedError):
            async for _ in s.get_request_stream("x"):
                pass
    asyncio.run(run())


# ----------------------------------------------------------------------------- planners
def test_admission_is_fifo_and_capped():
    p = AdmissionPlanner(2)
    assert p.plan(["a", "b", "c"], free_slots=5) == ["a", "b"]
    assert p.plan(["a", "b", "c"], free_slots=1) == ["a"]
    assert p.plan([], free_slots=3) == []


def test_budget_decode_priority_and_catchup():
    b = BudgetComputer(1000, decode_priority=True, catchup_ratio=0.25, reserve_backlog=2, min_chunk=64)
    r = b.compute(n_decode=10, n_prefill=1, backlog=1, force_prefill=False)
    assert r.decode_tokens == 10 and r.prefill_tokens == 250
    r = b.compute(10, 1, backlog=4, force_prefill=False)        # backlog above the reserve: larger share
    assert r.prefill_tokens == 750
    r = b.compute(10, 1, 1, force_prefill=True)
    assert r.prefill_tokens == 990 and r.starvation_override
    r = b.compute(0, 2, 2, False)
    assert r.prefill_tokens == 1000


def test_prefill_plan_is_varlen_and_respects_budget():
    p = DecodePrefillPlanner(chunk_size=64, microbatch=3, min_chunk=16)
    a, b, c = _req("a", 100), _req("b", 30), _req("c", 500)
    a.seq_len = 64                                   # already processed one chunk
    items = p.build_prefill_plan([a, b, c], budget_tokens=90)
    assert [(i.request_id, i.start, i.chunk_len) for i in items] == [("a", 64, 36), ("b", 0, 30), ("c", 0, 24)]
    assert p.build_decode_plan([a, b, c], 2) == ["a", "b"]
    v = DecodePrefillPlanner(64, 2, verified_decode_batch_sizes=(1, 4))
    assert v.build_decode_plan([a, b, c], 10) == ["a"]


def test_step_scheduler_fast_path_and_starvation_guard():
    s = RequestScheduler(max_active=4)
    ss = StepScheduler(step_token_budget=256, prefill_chunk_size=64, prefill_microbatch=1,
                       policy=SchedulerRuntimePolicy(max_decode_streak=2, max_prefill_deferrals=10),
                       catchup_ratio=0.0, min_chunk=1, max_active=4)
    d = _req("d")
    s.enqueue_request(d)
    s.admit("d")
    d.is_prefill = False
    plan = ss.build_plan(s)
    assert plan.fast_path and plan.decodes == ["d"]
    # a long prompt arrives; with a zero catch-up share the prefill only gets min_chunk tokens
    s.enqueue_request(_req("p", 200))
    plan = ss.build_plan(s)
    assert plan.admissions == ["p"] and plan.decodes == ["d"] and plan.prefills[0].chunk_len >= 1
    wire = StepPlan.from_wire(plan.to_wire())
    assert wire.decodes == plan.decodes and wire.prefills[0].chunk_len == plan.prefills[0].chunk_len


# ----------------------------------------------------------------------------- prefix cache
def test_prefix_cache_longest_match_lru_and_budget():
    pc = PrefixCache(max_entries=2, max_bytes=10_000)
    blocks = [(torch.zeros(2, 4), torch.zeros(2, 4))]
    a = _req("a", 48)
    pc.store(a, 32, blocks)
    pc.store(a, 16, blocks)
    hit = pc.lookup(_req("b", 40))
    assert hit is not None and hit.num_tokens == 32
    other = _req("c", 20)
    other.prompt_token_ids = [9] * 20
    assert pc.lookup(other) is None
    pc.store(other, 16, blocks)                      # evicts the least recently used entry
    assert pc.stats()["entries"] == 2 and pc.stats()["evictions"] == 1
    big = PrefixCache(max_entries=4, max_bytes=8)
    big.store(a, 16, blocks)                         # larger than the byte budget: not stored
    assert big.stats()["entries"] == 0
    assert not PrefixCache(0).enabled


def test_prefix_cache_keeps_different_images_apart():
    """Same prompt ids, same placeholder count, images of equal size but different pixels: the two
    requests must not share KV blocks or first-token logits."""
    import base64

    import numpy as np
    from PIL import Image
    pc = PrefixCache(max_entries=8, max_bytes=1 << 20)
    blocks = [(torch.zeros(2, 4), torch.zeros(2, 4))]
    rng = np.random.default_rng(0)
    img_a = Image.fromarray(rng.integers(0, 255, (8, 8, 3), dtype=np.uint8))
    img_b = Image.fromarray(rng.integers(0, 255, (8, 8, 3), dtype=np.uint8))
    a, b, a2 = _req("a", 32), _req("b", 32), _req("a2", 32)
    a.multi_modal_data, b.multi_modal_data = {"image": img_a}, {"image": img_b}
    a2.multi_modal_data = {"image": img_a.copy()}
    pc.store(a, 32, blocks, torch.ones(4))
    assert pc.lookup(b) is None
    assert pc.lookup(a2) is not None                       # byte-identical image: same entry
    # data URLs with a long common head and a different tail
    head = base64.b64encode(bytes(600)).decode()
    u1, u2 = _req("u1", 32), _req("u2", 32)
    u1.multi_modal_data = {"image": ["data:image/jpeg;base64," + head + "AAAA"]}
    u2.multi_modal_data = {"image": ["data:image/jpeg;base64," + head + "BBBB"]}
    pc.store(u1, 32, blocks)
    assert pc.lookup(u2) is None and pc.lookup(u1) is not None
    # content that cannot be identified bypasses the cache in both directions
    odd = _req("odd", 32)
    odd.multi_modal_data = {"image": object()}
    n0 = pc.stats()["entries"]
    pc.store(odd, 32, blocks)
    assert pc.stats()["entries"] == n0 and pc.lookup(odd) is None


def test_generic_moe_activation_layers_and_sniffer_cpu():
    import torch
    from litevllm_b200.debug import ActivationSniffer
    from litevllm_b200.layers.activation import GeluAndMul, Silu, SiluAndMul, get_act_fn
    from litevllm_b200.layers.fused_moe import fused_moe
    g = torch.Generator().manual_seed(3)
    x = torch.randn(5, 16, generator=g)
    assert torch.allclose(Silu()(x), torch.nn.functional.silu(x), atol=1e-6)
    assert torch.allclose(SiluAndMul()(x), torch.nn.functional.silu(x[:, :8]) * x[:, 8:], atol=1e-6)
    assert GeluAndMul()(x).shape == (5, 8) and isinstance(get_act_fn("gelu_pytorch_tanh"), torch.nn.Module)
    E, H, I, k = 4, 16, 8, 2
    w1, w2 = torch.randn(E, 2 * I, H, generator=g) * 0.2, torch.randn(E, H, I, generator=g) * 0.2
    logits = torch.randn(5, E, generator=g)
    got = fused_moe(x, w1, w2, logits, k)
    probs = torch.softmax(logits, -1)
    tw, ti = probs.topk(k, -1)
    tw = tw / tw.sum(-1, keepdim=True)
    want = torch.zeros(5, H)
    for t in range(5):
        for j in range(k):
            e = int(ti[t, j])
            h = x[t] @ w1[e].t()
            want[t] += tw[t, j] * ((torch.nn.functional.silu(h[:I]) * h[I:]) @ w2[e].t())
    assert torch.allclose(got, want, atol=1e-4)
    lin = torch.nn.Sequential(torch.nn.Linear(16, 16), torch.nn.ReLU())
    with ActivationSniffer(lin) as s:
        lin(x)
    assert "0" in s.stats and s.stats["0"].calls == 1 and "absmax" in s.report()


def test_memory_auditor_and_runtime_factory_are_used():
    from litevllm_b200 import LLM
    llm = LLM("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=2, max_model_len=64)
    mem = llm.engine.memory
    assert mem.param_bytes_by_dtype.get("float32", 0) > 0 and mem.kv_cache_bytes == llm.engine.kv_cache.total_bytes
    assert mem.weight_bytes >= mem.param_bytes_by_dtype["float32"]
    from litevllm_b200.engine.runtime_factory import RuntimeComponents
    assert set(RuntimeComponents.__dataclass_fields__) <= set(vars(llm.engine))


def test_span_profiler_accumulates_and_is_free_when_off():
    from litevllm_b200.utils.profiling import SpanProfiler
    p = SpanProfiler()
    with p.span("x"):
        pass
    assert p.summary() == {}
    p.configure(True)
    for _ in range(3):
        with p.span("step"):
            pass
    p.count("tokens", 5)
    s = p.summary()
    assert s["step"]["count"] == 3 and s["counters"]["tokens"] == 5
    p.reset()
    assert p.summary() == {}


def test_tokenizer_helpers_and_incremental_detokenizer():
    from litevllm_b200.tokenizers import IncrementalDetokenizer, TokenizerLike, TokenizerRegistry, get_tokenizer
    from litevllm_b200.transformers_utils.config import build_fallback_hf_config, is_gguf_path

    class ByteTok:
        eos_token_id, bos_token_id = None, None

        def encode(self, text, add_special_tokens=True):
            return list(text.encode())

        def decode(self, ids, skip_special_tokens=True):
            return bytes(ids).decode("utf-8", errors="replace")

        def __len__(self):
            return 256

    tok = ByteTok()
    assert isinstance(tok, TokenizerLike)
    det = IncrementalDetokenizer(tok)
    text = "héllo ✓"
    deltas = [det.push(t) for t in tok.encode(text)]
    assert "".join(deltas) == text and "�" not in "".join(deltas) and "" in deltas   # multi-byte chars wait
    TokenizerRegistry.register("bytes", lambda path, **kw: tok)
    assert get_tokenizer("anything", tokenizer_mode="bytes") is tok
    dummy = get_tokenizer("/nonexistent/path", vocab_size=100)
    assert len(dummy) == 100 and get_tokenizer("/nonexistent/path", vocab_size=100) is dummy   # cached
    flat = build_fallback_hf_config({"architectures": ["Gemma4ForConditionalGeneration"],
                                     "text_config": {"hidden_size": 8, "model_type": "gemma4_text"},
                                     "vision_config": {"patch_size": 16}})
    assert flat["hidden_size"] == 8 and flat["vision_config"]["patch_size"] == 16 and is_gguf_path("a/b.GGUF")


def test_bounds_check_mode_names_the_bad_index():
    """FI_BOUNDS_CHECK mode: index tensors are validated against the buffers they index before an op runs."""
    from litevllm_b200 import ops
    ops.set_bounds_check(True)
    try:
        kc = torch.zeros(9, 2, 16, 8)
        vc = torch.zeros_like(kc)
        q = torch.randn(2, 4 * 8)
        bt = torch.tensor([[1, 2, 0], [3, 99, 0]], dtype=torch.int32)
        with pytest.raises(IndexError, match=r"block_tables: value 99 at position \[1, 1\]"):
            ops.paged_attention_decode(q, kc, vc, bt, torch.tensor([20, 17], dtype=torch.int32), 4, 2, 8, 0.3)
        # the same table is fine while the second sequence stays inside its first block
        ops.paged_attention_decode(q, kc, vc, bt, torch.tensor([20, 16], dtype=torch.int32), 4, 2, 8, 0.3)
        with pytest.raises(IndexError, match="seq_lens"):
            ops.paged_attention_decode(q, kc, vc, bt, torch.tensor([20, 49], dtype=torch.int32), 4, 2, 8, 0.3)
        with pytest.raises(IndexError, match="embedding.ids"):
            ops.embedding(torch.tensor([0, 7, 12]), torch.zeros(12, 4))
        with pytest.raises(IndexError, match="slot_mapping"):
            ops.reshape_and_cache(torch.zeros(1, 2, 8), torch.zeros(1, 2, 8), torch.tensor([9 * 16], dtype=torch.int32), kc, vc)
    finally:
        ops.set_bounds_check(False)


def test_stage_spans_and_attention_metadata_snapshot():
    """Per-stage profile spans of an eager forward, and the paged-attention metadata snapshot: a consistent call
    is described, a block id outside the cache or a sequence longer than its block-table row is refused."""
    import pytest
    import torch
    from litevllm_b200 import LLM, SamplingParams, ops
    from litevllm_b200.utils.profiling import PROFILER
    PROFILER.reset()
    PROFILER.configure(True)
    saved = PROFILER.stages
    PROFILER.stages = True
    try:
        llm = LLM("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=2, max_model_len=64)
        llm.generate([[1, 2, 3, 4, 5]], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))
        summ = PROFILER.summary()
        llm.shutdown()
    finally:
        PROFILER.stages = saved
        PROFILER.configure(False)
    assert summ["layer.attention"]["count"] >= 2 and summ["layer.mlp"]["count"] >= 2
    PROFILER.reset()

    kc = torch.zeros(6, 2, 16, 8)
    q = torch.zeros(3, 4 * 8)
    bt = torch.tensor([[1, 2, 0], [3, 0, 0]], dtype=torch.int32)
    snap = ops.paged_metadata_snapshot(q, kc, bt, torch.tensor([20, 5], dtype=torch.int32),
                                       torch.tensor([0, 2, 3], dtype=torch.int32), scope="layer0")
    assert snap["blocks_needed"] == [2, 1] and snap["block_id_range"] == [1, 3] and snap["new_tokens"] == [2, 1]
    with pytest.raises(IndexError):
        ops.paged_metadata_snapshot(q, kc, torch.tensor([[1, 9, 0], [3, 0, 0]], dtype=torch.int32),
                                    torch.tensor([20, 5], dtype=torch.int32))
    with pytest.raises(IndexError):
        ops.paged_metadata_snapshot(q, kc, bt, torch.tensor([70, 5], dtype=torch.int32))


def test_selective_block_tables_and_engine_cpu():
    """Selective decode attention: the compact table keeps every stride-th block, the leading blocks and the
    last one; with a ratio of 1 the engine generates exactly what it generates without the feature, with a
    small ratio it still runs to completion on a context of many blocks."""
    import torch
    from litevllm_b200 import LLM, SamplingParams, ops
    bt = torch.arange(1, 25, dtype=torch.int32).view(2, 12)
    sl = torch.tensor([16 * 9 + 5, 7], dtype=torch.int32)          # 10 blocks (last partial), 1 block
    tab, lens = ops.select_blocks(bt, sl, 16, 4, 2)
    assert tab[0, :5].tolist() == [1, 2, 5, 9, 10] and tab[0, 5:].tolist() == [0] * 7    # blocks 0,1 | 4 | 8 | 9
    assert lens.tolist() == [4 * 16 + 5, 7] and tab[1, 0].item() == 13
    prompt = [(7 * i) % 500 + 1 for i in range(100)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)

    def run(ratio):
        cfg = {"tuning_keyvals": {"FASTINFERENCE_KV_SELECT_RATIO": str(ratio), "FASTINFERENCE_KV_SELECT_MIN_BLOCKS": "1"}}
        llm = LLM("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=2, max_model_len=160,
                  fastinference_config=cfg if ratio else None)
        out = llm.generate([prompt], sp)[0].outputs[0].token_ids
        llm.shutdown()
        return out
    base = run(0)
    assert run(1.0) == base
    assert len(run(0.25)) == 6


def test_engine_and_weights_are_freed_after_shutdown():
    """The engine parks its objects in the collector's permanent generation while it runs; after ``shutdown`` a
    dropped engine (model, KV pool) must be collectable again, or a second engine in the same process would find
    the first one's memory still in use."""
    import gc
    import weakref
    from litevllm_b200 import LLM, SamplingParams

    def build_and_drop():
        llm = LLM("synthetic:tiny-llama-test", device="cpu", max_model_len=64, dtype="float32")
        llm.generate([{"prompt_token_ids": [3, 4, 5]}], SamplingParams(max_tokens=2, temperature=0.0, ignore_eos=True))
        refs = weakref.ref(llm.engine.model), weakref.ref(llm.engine.kv_cache)
        llm.shutdown()
        return refs

    model_ref, kv_ref = build_and_drop()
    gc.collect()
    assert model_ref() is None and kv_ref() is None
