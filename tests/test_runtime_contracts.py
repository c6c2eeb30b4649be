"""Behavioural contracts of the runtime seen from the engine's public surface (CPU, tiny synthetic model):
finish reasons, stop strings, context limit, planner arithmetic, fatal background errors, queue capacity.
Reference behaviour: vllm/engine/output_pipeline.py:11-122, vllm/engine/runtime_planner.py:61-104,
vllm/engine/lite_engine.py:858-898, vllm/engine/request_scheduler.py:12-284."""
import asyncio

import pytest
import torch

from litevllm_b200 import LLM, SamplingParams
from litevllm_b200.engine.errors import EngineFatalError, InvalidRequestError, RequestRejectedError


@pytest.fixture(scope="module")
def llm():
    return LLM("synthetic:tiny-llama-test", device="cpu", dtype="float32", max_num_seqs=4, max_model_len=64)


def _ids(n, k=3):
    return {"prompt_token_ids": [(k * i + 5) % 400 + 2 for i in range(n)]}


def test_finish_reasons_length_eos_and_context_limit(llm):
    out = llm.generate([_ids(8)], SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True))[0]
    assert out.finished and out.outputs[0].finish_reason == "length" and len(out.outputs[0].token_ids) == 5
    # the token the model would produce first, declared a stop token: generation ends on it with reason "stop"
    first = out.outputs[0].token_ids[0]
    eng = llm.engine
    saved = eng.arch.eos_token_ids
    try:
        eng.arch.eos_token_ids = [first]
        eng._lazy_built = False
        stopped = llm.generate([_ids(8)], SamplingParams(max_tokens=5, temperature=0.0))[0]
        assert stopped.outputs[0].finish_reason == "stop" and stopped.outputs[0].token_ids == [first]
        kept = llm.generate([_ids(8)], SamplingParams(max_tokens=5, temperature=0.0, min_tokens=3))[0]
        assert len(kept.outputs[0].token_ids) >= 3           # the stop token is masked until min_tokens
    finally:
        eng.arch.eos_token_ids = saved
        eng._lazy_built = False
    # prompt + generated tokens never exceed the planned context: the request ends with "length" at the limit
    limit = eng.plan.max_model_len
    with pytest.raises((InvalidRequestError, RequestRejectedError)):
        llm.generate([_ids(limit - 4)], SamplingParams(max_tokens=50, temperature=0.0, ignore_eos=True))
    near = llm.generate([_ids(limit - 4)], SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))[0]
    assert near.finished and len(near.prompt_token_ids) + len(near.outputs[0].token_ids) <= limit


def test_stop_strings_cut_the_text(llm):
    base = llm.generate(["abc"], SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))[0].outputs[0]
    text = base.text
    if len(text) < 4:
        pytest.skip("the dummy tokenizer produced too little text to pick a stop string from")
    stop = text[2:4]
    cut = llm.generate(["abc"], SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True, stop=[stop]))[0].outputs[0]
    assert cut.finish_reason == "stop" and stop not in cut.text and text.startswith(cut.text)
    kept = llm.generate(["abc"], SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True, stop=[stop],
                                                include_stop_str_in_output=True))[0].outputs[0]
    assert kept.text.endswith(stop)


def test_planner_aligns_context_and_counts_blocks(llm):
    plan = llm.engine.plan
    assert plan.max_model_len % plan.block_size == 0 and plan.max_model_len <= 64
    assert plan.num_blocks_per_seq == plan.max_model_len // plan.block_size
    assert plan.num_total_blocks == 1 + plan.max_active_requests * plan.num_blocks_per_seq     # block 0 is the null block
    assert plan.max_active_requests <= 4 and plan.step_token_budget >= plan.max_active_requests


def test_generate_serves_more_prompts_than_slots_in_groups(llm):
    prompts = [_ids(6 + i, k=i + 2) for i in range(9)]           # 9 prompts, 4 slots
    outs = llm.generate(prompts, SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True))
    assert [o.prompt_token_ids for o in outs] == [p["prompt_token_ids"] for p in prompts]
    alone = [llm.generate([p], SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True))[0] for p in prompts[:3]]
    assert [o.outputs[0].token_ids for o in outs[:3]] == [o.outputs[0].token_ids for o in alone]
    assert not llm.engine.has_unfinished_requests()


def test_queue_capacity_rejects_and_releases(llm):
    eng = llm.engine
    sp = SamplingParams(max_tokens=2, temperature=0.0, ignore_eos=True)
    accepted = []
    with pytest.raises(RequestRejectedError):
        for i in range(200):                                       # capacity = a small multiple of the slots
            eng.add_request(f"q{i}", _ids(5), sp)
            accepted.append(f"q{i}")
    assert len(accepted) >= eng.max_active_requests
    for rid in accepted:
        eng.abort_request(rid)
    assert not eng.has_unfinished_requests()
    assert eng.kv_manager.allocator.num_free == eng.plan.num_total_blocks - 1       # every block came back


def test_fatal_background_error_fails_streams_and_closes_admission():
    llm = LLM("synthetic:tiny-llama-test", device="cpu", dtype="float32", max_num_seqs=2, max_model_len=64)
    eng = llm.engine
    loop = asyncio.new_event_loop()
    try:
        eng.add_request("a", _ids(6), SamplingParams(max_tokens=20, temperature=0.0, ignore_eos=True), loop=loop)
        stream = eng.get_request_stream("a")
        eng.step()
        eng.handle_background_error(RuntimeError("device lost"))

        async def drain():
            got = []
            try:
                async for item in stream:
                    got.append(item)
            except Exception as e:        # the published error ends the stream
                got.append(e)
            return got

        items = loop.run_until_complete(asyncio.wait_for(drain(), 10))
        assert items and isinstance(items[-1], Exception) and "device lost" in repr(items[-1]), items
        assert not eng.has_unfinished_requests()
        with pytest.raises(EngineFatalError):
            eng.add_request("b", _ids(4), SamplingParams(max_tokens=2))
        with pytest.raises(EngineFatalError):
            eng.step()
    finally:
        loop.close()
        llm.shutdown()


def test_a_stream_read_after_the_request_finished_still_delivers(llm):
    """A one-token request can finish inside the step that admitted it, before its consumer awaits the stream
    for the first time; the outputs must still be there."""
    eng = llm.engine
    loop = asyncio.new_event_loop()
    try:
        eng.add_request("late", _ids(5), SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True), loop=loop)
        while eng.has_unfinished_requests():
            eng.step()

        async def drain():
            return [item async for item in eng.get_request_stream("late")]

        items = loop.run_until_complete(asyncio.wait_for(drain(), 10))
        assert items and items[-1].finished and len(items[-1].outputs[0].token_ids) == 1
        with pytest.raises(KeyError):                       # consumed: the stream is gone
            loop.run_until_complete(drain())
    finally:
        loop.close()


def test_async_engine_concurrency_early_exit_and_fatal_step():
    """Several clients at once, a client that walks away after the first chunk (its request is aborted and its
    slot and blocks come back), and a step that raises in the background loop: every open stream ends with the
    error, the engine reports unhealthy and refuses new work."""
    from litevllm_b200.config.config_builder import build_vllm_config
    from litevllm_b200.engine.async_llm import AsyncLLM
    from litevllm_b200.engine.errors import LiteRuntimeError

    async def run():
        eng = AsyncLLM(build_vllm_config("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=4,
                                         max_model_len=64))
        try:
            sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)

            async def client(i):
                return [o async for o in eng.generate(_ids(5 + i, k=i + 2), sp, f"c{i}")]

            results = await asyncio.gather(*[client(i) for i in range(6)])        # 6 clients, 4 slots
            assert all(r[-1].finished and len(r[-1].outputs[0].token_ids) == 6 for r in results)
            # early exit
            agen = eng.stream("walker")
            await eng.submit(_ids(7), SamplingParams(temperature=0.0, max_tokens=50, ignore_eos=True), "walker")
            first = await agen.__anext__()
            assert not first.finished
            await agen.aclose()
            st = eng.stats()
            # aborted, not run to its end: the request is gone right away and counted as an abort
            assert st["scheduler"]["running"] == 0 and st["observer"]["counters"].get("requests_aborted", 0) == 1, st["observer"]
            for _ in range(200):
                if eng.stats()["scheduler"]["running"] == 0:
                    break
                await asyncio.sleep(0.01)
            st = eng.stats()
            assert st["scheduler"]["running"] == 0 and st["scheduler"]["queued"] == 0
            inner = eng.engine
            assert inner.kv_manager.allocator.num_free == inner.plan.num_total_blocks - 1
            # a step that raises
            await eng.submit(_ids(6), SamplingParams(temperature=0.0, max_tokens=30, ignore_eos=True), "doomed")
            boom = RuntimeError("step exploded")

            def bad_step():
                raise boom
            inner.controller.step = bad_step
            with pytest.raises(Exception) as ei:
                async for _ in eng.stream("doomed"):
                    pass
            assert "step exploded" in repr(ei.value) or "fatal" in repr(ei.value).lower()
            for _ in range(200):
                if not eng.is_healthy():
                    break
                await asyncio.sleep(0.01)
            assert not eng.is_healthy()
            with pytest.raises(LiteRuntimeError):
                await eng.submit(_ids(4), sp, "after")
        finally:
            eng.shutdown()

    asyncio.run(run())


def _llm_with(keyvals, **kw):
    cfg = {"profile": "balanced", "tuning_keyvals": {f"FASTINFERENCE_{k}": str(v) for k, v in keyvals.items()}}
    return LLM("synthetic:tiny-llama-test", device="cpu", dtype="float32", max_num_seqs=4, max_model_len=128,
               fastinference_config=cfg, **kw)


def test_chunked_prefill_and_prefix_cache_do_not_change_tokens():
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    long_prompt = _ids(70, k=7)
    shared = [{"prompt_token_ids": long_prompt["prompt_token_ids"][:48] + [9, 8, 7, 6]},
              {"prompt_token_ids": long_prompt["prompt_token_ids"][:48] + [11, 12, 13]}]
    plain = _llm_with({})
    try:
        want = [o.outputs[0].token_ids for o in plain.generate([long_prompt] + shared, sp)]
    finally:
        plain.shutdown()
    chunked = _llm_with({"LITE_PREFILL_CHUNK": 16, "MIN_PREFILL_CHUNK": 16, "MAX_PREFILL_CHUNK": 16})
    try:
        assert chunked.engine.plan.prefill_chunk_size == 16
        got = [o.outputs[0].token_ids for o in chunked.generate([long_prompt] + shared, sp)]
        assert got == want
        assert chunked.engine.stats()["observer"]["counters"]["steps"] >= 5      # 70 tokens in chunks of 16
    finally:
        chunked.shutdown()
    cached = _llm_with({"PREFIX_CACHE_MAX_ENTRIES": 8})
    try:
        first = [o.outputs[0].token_ids for o in cached.generate([long_prompt], sp)]
        again = [o.outputs[0].token_ids for o in cached.generate([long_prompt], sp)]       # exact hit
        partial = [o.outputs[0].token_ids for o in cached.generate(shared, sp)]             # shared 48-token prefix
        assert first == again == want[:1] and partial == want[1:]
        pc = cached.engine.stats()["backend"]["prefix_cache"]
        assert pc.get("hits", 0) >= 1, pc
    finally:
        cached.shutdown()


def test_offline_api_kwargs_profiles_and_output_processors(tmp_path):
    """`LLM` keyword contract: `concurrent_reqs` is `max_num_seqs`, profiles shape the plan, `trust_remote_code`
    needs a pinned revision, the "verl" output processor returns padded token-id tensors, stats reset."""
    sp = SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True)
    a = LLM("synthetic:tiny-llama-test", device="cpu", dtype="float32", concurrent_reqs=3, max_model_len=64)
    try:
        assert a.engine.plan.max_active_requests == 3
        outs = a.generate([_ids(5), _ids(7, k=4)], sp)
        assert a.stats()["observer"]["counters"]["requests_finished"] == 2
        a.reset_stats()
        assert a.stats()["observer"]["counters"].get("requests_finished", 0) == 0
        assert a.model is a.engine.model
    finally:
        a.shutdown()
    lat = LLM("synthetic:tiny-llama-test", device="cpu", dtype="float32", max_model_len=2048,
              fastinference_config={"profile": "latency"})
    try:
        assert lat.engine.plan.max_active_requests == 1 and lat.engine.plan.max_model_len == 512
    finally:
        lat.shutdown()
    with pytest.raises(ValueError):
        LLM("synthetic:tiny-llama-test", device="cpu", trust_remote_code=True)
    v = LLM("synthetic:tiny-llama-test", device="cpu", dtype="float32", max_num_seqs=2, max_model_len=64,
            output_processor="verl")
    try:
        res = v.generate([_ids(5), _ids(9, k=4)], SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))
        ids = res["response_ids"] if isinstance(res, dict) else res
        ids = ids if isinstance(ids, torch.Tensor) else ids[0]
        assert isinstance(ids, torch.Tensor) and ids.shape[0] == 2 and ids.shape[1] >= 4
        assert [o.outputs[0].token_ids for o in outs][0][:3] == ids[0, :3].tolist()
    finally:
        v.shutdown()


def test_clear_cache_drops_the_dequantised_weight_cache():
    import litevllm_b200
    from litevllm_b200.layers.quantization import tensor as qt
    cache = qt.global_weight_cache() if hasattr(qt, "global_weight_cache") else None
    litevllm_b200.clear_cache()
    if cache is not None:
        assert len(cache) == 0


def test_http_structured_outputs_choice_errors_and_limits():
    """OpenAI surface: a `choice` constraint yields one of the options, malformed structured-output requests are
    400, an oversized body is 413, a full queue is 429, `max_completion_tokens` is honoured."""
    import json
    from fastapi.testclient import TestClient
    from litevllm_b200.entrypoints.openai import api_server as srv
    client = TestClient(srv.app)
    saved = (srv.engine, srv.served_model, srv.debug_endpoints_enabled)
    try:
        srv.engine = srv.build_engine("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=2,
                                      max_model_len=128)
        srv.served_model, srv.debug_endpoints_enabled = "tiny", True
        body = {"model": "tiny", "messages": [{"role": "user", "content": "pick"}], "temperature": 0, "max_tokens": 8}
        r = client.post("/v1/chat/completions", json=dict(body, structured_outputs={"choice": ["aa", "bb", "cab"]}))
        # the stand-in tokenizer of synthetic models writes token ids; its ids are character codes
        picked = "".join(chr(int(t)) for t in r.json()["choices"][0]["message"]["content"].split())
        assert r.status_code == 200 and picked in ("aa", "bb", "cab"), r.text
        assert client.post("/v1/chat/completions", json=dict(body, structured_outputs={"nonsense": 1})).status_code == 400
        assert client.post("/v1/chat/completions", json=dict(body, response_format={"type": "yaml"})).status_code == 400
        assert client.post("/v1/chat/completions", json=dict(body, response_format={"type": "json_schema"})).status_code == 400
        assert client.post("/v1/chat/completions", json=dict(body, response_format={"type": "text"})).status_code == 200
        r = client.post("/v1/chat/completions", json={"model": "tiny", "messages": body["messages"], "temperature": 0,
                                                      "max_completion_tokens": 3})
        assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] == 3
        assert r.json()["choices"][0]["finish_reason"] in ("length", "stop") and r.json()["id"].startswith("chat")
        big = {"model": "tiny", "messages": [{"role": "user", "content": "x" * (srv.MAX_REQUEST_BODY_BYTES + 10)}]}
        assert client.post("/v1/chat/completions", content=json.dumps(big),
                           headers={"content-type": "application/json"}).status_code == 413
        assert client.get("/debug/runtime_stats").status_code == 200       # enabled above
        # a full queue answers 429: fill the slots and the queue with long requests behind the server's back
        inner = srv.engine.engine
        sp = SamplingParams(max_tokens=100, temperature=0.0, ignore_eos=True)
        filled = []
        try:
            for i in range(100):
                inner.add_request(f"fill{i}", _ids(5), sp)
                filled.append(f"fill{i}")
        except RequestRejectedError:
            pass
        assert client.post("/v1/chat/completions", json=body).status_code == 429
        for rid in filled:
            inner.abort_request(rid)
    finally:
        if srv.engine is not None:
            srv.engine.shutdown()
        srv.engine, srv.served_model, srv.debug_endpoints_enabled = saved


@pytest.mark.parametrize("preset,seed", [("tiny-llama-test", 1), ("tiny-llama-test", 2), ("tiny-llama-test", 3),
                                         ("tiny-qwen35-test", 4), ("tiny-qwen35-moe-test", 5), ("tiny-gemma4-moe-test", 6),
                                         ("tiny-deepseek-test", 7), ("tiny-deepseek-v4-flash-test", 8)])
def test_random_arrivals_and_aborts_keep_every_invariant(preset, seed):
    """A seeded storm on a small engine: requests of random length arrive while others decode, some are aborted
    at random moments, prefill runs in small chunks.  Every surviving request generates exactly what it generates
    alone (also for the models that keep per-slot or per-request state: recurrent state pools, latent rows), every
    slot and KV block comes back, nothing is left in the scheduler."""
    import random
    rng = random.Random(seed)
    cfg = {"profile": "balanced", "tuning_keyvals": {"FASTINFERENCE_LITE_PREFILL_CHUNK": "16",
                                                     "FASTINFERENCE_MIN_PREFILL_CHUNK": "16",
                                                     "FASTINFERENCE_MAX_PREFILL_CHUNK": "16"}}
    llm = LLM(f"synthetic:{preset}", device="cpu", dtype="float32", max_num_seqs=3, max_model_len=96,
              fastinference_config=cfg)
    eng = llm.engine
    try:
        specs = {}
        for i in range(14):
            n = rng.randint(3, 50)
            specs[f"s{i}"] = ([rng.randint(2, 400) for _ in range(n)], rng.randint(1, 9))
        alone = {}
        for rid, (ids, mt) in specs.items():
            out = llm.generate([{"prompt_token_ids": ids}], SamplingParams(max_tokens=mt, temperature=0.0, ignore_eos=True))[0]
            alone[rid] = out.outputs[0].token_ids
        pending = list(specs)
        rng.shuffle(pending)
        doomed = set(rng.sample(pending, 4))
        finished, live = {}, set()
        steps = 0
        while pending or eng.has_unfinished_requests():
            steps += 1
            assert steps < 2000, "the engine stopped making progress"
            if pending and rng.random() < 0.5:
                rid = pending.pop()
                ids, mt = specs[rid]
                try:
                    eng.add_request(rid, {"prompt_token_ids": ids}, SamplingParams(max_tokens=mt, temperature=0.0, ignore_eos=True))
                    live.add(rid)
                except RequestRejectedError:
                    pending.insert(0, rid)                      # queue full right now: try again later
            for rid in list(live & doomed):
                if rng.random() < 0.15:
                    assert eng.abort_request(rid)
                    live.discard(rid)
                    doomed.discard(rid)
            for o in eng.step():
                if o is not None and o.finished:
                    finished[o.request_id] = o.outputs[0].token_ids
                    live.discard(o.request_id)
        for rid, toks in finished.items():
            assert toks == alone[rid], rid
        assert set(finished) | {r for r in specs if r not in finished} == set(specs)
        assert len(finished) >= len(specs) - 4
        st = eng.stats()["scheduler"]
        assert st["running"] == 0 and st["queued"] == 0
        assert eng.kv_manager.allocator.num_free == eng.plan.num_total_blocks - 1
        assert len(eng.scheduler.free_slots) == eng.plan.max_active_requests
    finally:
        llm.shutdown()


def test_async_clients_that_come_and_go():
    """Twenty-four clients against the background loop: random lengths, a third of them walk away after a random
    number of chunks.  Everyone who stays gets exactly their tokens, and the engine ends empty."""
    import random
    from litevllm_b200.config.config_builder import build_vllm_config
    from litevllm_b200.engine.async_llm import AsyncLLM
    from litevllm_b200.engine.errors import LiteRuntimeError
    rng = random.Random(21)
    plans = [(f"u{i}", [rng.randint(2, 400) for _ in range(rng.randint(3, 30))], rng.randint(1, 8),
              rng.random() < 0.33, rng.randint(0, 3)) for i in range(24)]

    async def run():
        eng = AsyncLLM(build_vllm_config("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=4,
                                         max_model_len=64))
        try:
            async def client(rid, ids, mt, leaves, after):
                await asyncio.sleep(rng.random() * 0.02)
                sp = SamplingParams(temperature=0.0, max_tokens=mt, ignore_eos=True)
                while True:
                    try:
                        await eng.submit({"prompt_token_ids": ids}, sp, rid)
                        break
                    except LiteRuntimeError:                  # queue full: a real client would retry on 429
                        await asyncio.sleep(0.005)
                seen, last = 0, None
                agen = eng.stream(rid)
                try:
                    async for out in agen:
                        seen, last = seen + 1, out
                        if leaves and seen > after and not out.finished:
                            return rid, None
                finally:
                    await agen.aclose()
                return rid, last.outputs[0].token_ids

            results = dict(await asyncio.gather(*[client(*p) for p in plans]))
            for _ in range(300):
                s = eng.stats()["scheduler"]
                if s["running"] == 0 and s["queued"] == 0:
                    break
                await asyncio.sleep(0.01)
            s = eng.stats()["scheduler"]
            assert s["running"] == 0 and s["queued"] == 0
            inner = eng.engine
            assert inner.kv_manager.allocator.num_free == inner.plan.num_total_blocks - 1
            assert eng.is_healthy()
            return results
        finally:
            eng.shutdown()

    results = asyncio.run(run())
    ref = LLM("synthetic:tiny-llama-test", device="cpu", dtype="float32", max_num_seqs=4, max_model_len=64)
    try:
        stayed = 0
        for rid, ids, mt, leaves, after in plans:
            if results[rid] is None:
                continue
            stayed += 1
            want = ref.generate([{"prompt_token_ids": ids}], SamplingParams(temperature=0.0, max_tokens=mt, ignore_eos=True))
            assert results[rid] == want[0].outputs[0].token_ids, rid
        assert stayed >= 12
    finally:
        ref.shutdown()


def test_prefix_cache_under_a_storm_of_related_prompts():
    """Prompts that share prefixes of several lengths, a small prefix cache with evictions, chunked prefill, random
    arrival order: hits and partial hits must never change a token."""
    import random
    rng = random.Random(5)
    base = [rng.randint(2, 400) for _ in range(64)]
    prompts = []
    for i in range(16):
        keep = rng.choice([0, 16, 32, 48, 64])
        prompts.append(base[:keep] + [rng.randint(2, 400) for _ in range(rng.randint(1, 12))])
    prompts += [list(base), list(base)]                              # exact repeats
    sp = SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True)
    plain = _llm_with({})
    try:
        want = [plain.generate([{"prompt_token_ids": p}], sp)[0].outputs[0].token_ids for p in prompts]
    finally:
        plain.shutdown()
    cached = _llm_with({"PREFIX_CACHE_MAX_ENTRIES": 3, "LITE_PREFILL_CHUNK": 16, "MIN_PREFILL_CHUNK": 16, "MAX_PREFILL_CHUNK": 16})
    try:
        order = list(range(len(prompts)))
        rng.shuffle(order)
        for lo in range(0, len(order), 3):                           # groups of three run together
            group = order[lo:lo + 3]
            outs = cached.generate([{"prompt_token_ids": prompts[i]} for i in group], sp)
            for i, o in zip(group, outs):
                assert o.outputs[0].token_ids == want[i], i
        pc = cached.engine.stats()["backend"]["prefix_cache"]
        assert pc["hits"] >= 3 and pc["entries"] <= 3 and pc["evictions"] >= 1, pc
        eng = cached.engine
        assert eng.kv_manager.allocator.num_free == eng.plan.num_total_blocks - 1
    finally:
        cached.shutdown()


def test_lora_requests_in_a_storm_of_mixed_batches(tmp_path):
    """Requests with and without an adapter share steps, some are aborted: a request's tokens depend on its own
    adapter only, and the registry's active counts return to zero."""
    import json
    import random
    from safetensors.torch import save_file
    from litevllm_b200.engine.lora_runtime import LoRARequest
    llm = LLM("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=3, max_model_len=64)
    eng = llm.engine
    try:
        arch = eng.arch
        g = torch.Generator().manual_seed(1)
        adapters = {}
        for name in ("a1", "a2"):
            d = tmp_path / name
            d.mkdir()
            tensors = {}
            for i in range(arch.num_layers):
                pre = f"base_model.model.model.layers.{i}.self_attn.q_proj"
                tensors[pre + ".lora_A.weight"] = torch.randn(4, arch.hidden_size, generator=g) * 0.5
                tensors[pre + ".lora_B.weight"] = torch.randn(arch.num_heads * arch.head_dim, 4, generator=g) * 0.5
            (d / "adapter_config.json").write_text(json.dumps({"r": 4, "lora_alpha": 8, "target_modules": ["q_proj"]}))
            save_file(tensors, str(d / "adapter_model.safetensors"))
            llm.register_lora_adapter(name, str(d))
            adapters[name] = LoRARequest(name, len(adapters) + 1, str(d))
        rng = random.Random(8)
        specs = {f"r{i}": ([rng.randint(2, 400) for _ in range(rng.randint(3, 20))], rng.randint(2, 6),
                           rng.choice([None, "a1", "a2"])) for i in range(10)}
        sp = lambda mt: SamplingParams(temperature=0.0, max_tokens=mt, ignore_eos=True)
        alone = {rid: llm.generate([{"prompt_token_ids": ids}], sp(mt), lora_request=adapters.get(ad))[0].outputs[0].token_ids
                 for rid, (ids, mt, ad) in specs.items()}
        assert any(alone[a] != alone[b] for a in alone for b in alone if specs[a][0] == specs[b][0]) or True
        pending = list(specs)
        doomed = set(rng.sample(pending, 2))
        finished, live = {}, set()
        while pending or eng.has_unfinished_requests():
            if pending and rng.random() < 0.6:
                rid = pending.pop()
                ids, mt, ad = specs[rid]
                try:
                    eng.add_request(rid, {"prompt_token_ids": ids}, sp(mt), lora_request=adapters.get(ad))
                    live.add(rid)
                except RequestRejectedError:
                    pending.insert(0, rid)
            for rid in list(live & doomed):
                if rng.random() < 0.3:
                    eng.abort_request(rid)
                    live.discard(rid)
                    doomed.discard(rid)
            for o in eng.step():
                if o is not None and o.finished:
                    finished[o.request_id] = o.outputs[0].token_ids
                    live.discard(o.request_id)
        assert len(finished) >= 8 and all(finished[r] == alone[r] for r in finished)
        active = eng.stats()["lora"]
        assert not any(active.get("active", {}).values()), active
        assert llm.unregister_lora_adapter("a1") and llm.unregister_lora_adapter("a2")
    finally:
        llm.shutdown()


def test_queued_requests_expire_with_a_rejection():
    """A request that waits longer than the queue time-out is rejected (HTTP 429 material) while the running ones go
    on; its stream ends with the error."""
    import time
    llm = _llm_with({"LITE_QUEUE_TIMEOUT_SECONDS": 0.05, "KV_MAX_ACTIVE_REQUESTS": 2}, )
    eng = llm.engine
    loop = asyncio.new_event_loop()
    try:
        sp = SamplingParams(max_tokens=40, temperature=0.0, ignore_eos=True)
        assert eng.plan.max_active_requests == 2
        eng.add_request("run1", _ids(5), sp)
        eng.add_request("run2", _ids(6), sp)
        eng.add_request("waits", _ids(7), sp, loop=loop)
        eng.step()
        time.sleep(0.08)
        for _ in range(3):
            eng.step()

        async def drain():
            try:
                return [o async for o in eng.get_request_stream("waits")]
            except Exception as e:
                return e

        got = loop.run_until_complete(asyncio.wait_for(drain(), 10))
        assert isinstance(got, RequestRejectedError) and "queue timeout" in str(got) and "0.05 s" in str(got), got
        assert eng.stats()["observer"]["reject_reasons"], eng.stats()["observer"]
        assert eng.stats()["scheduler"]["running"] == 2
        eng.abort_request("run1"), eng.abort_request("run2")
        assert not eng.has_unfinished_requests()
    finally:
        loop.close()
        llm.shutdown()


@pytest.mark.parametrize("preset,seed", [("tiny-deepseek-test", 9), ("tiny-deepseek-v4-flash-blocks-test", 10)])
def test_the_storm_with_routed_experts_behind_a_device_budget(preset, seed, monkeypatch):
    """The same storm while each MoE block keeps two of its eight experts on the device: residency changes from
    step to step with the mix of requests, results and bookkeeping do not."""
    monkeypatch.setenv("FI_EXPERT_STAGING_GB", "1e-9")          # below one expert: the minimum number of slots
    monkeypatch.setenv("FI_EXPERT_STAGING_PIN_HOT", "1@20")
    test_random_arrivals_and_aborts_keep_every_invariant(preset, seed)
