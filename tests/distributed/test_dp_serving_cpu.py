"""Data-parallel serving as gloo ranks on the CPU: rank 0 answers HTTP requests through FastAPI's TestClient
and routes them to the replica with the fewest requests in flight; rank 1 serves what it is sent and streams
the outputs back.  Greedy completions must equal what a single engine produces, some requests must have run
on the remote replica, and a streamed request must arrive chunk by chunk."""
import json
import os
import tempfile

from litevllm_b200.parallel.launcher import spawn

BODY = {"model": "tiny", "max_tokens": 6, "temperature": 0}
PROMPTS = ["hello there", "second question", "a third one", "and the fourth"]


def _dp_worker(rank, world, out_dir):
    from litevllm_b200.entrypoints.openai import api_server as srv
    eng = srv.build_engine("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=4, max_model_len=128,
                           data_parallel_size=world)
    served = []
    if eng.is_worker_rank:
        steps = eng.serve_as_worker(lambda outs: served.extend(o.request_id for o in outs if o is not None and o.finished))
        with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
            json.dump({"served": served, "steps": steps}, f)
        eng.shutdown()
        return
    import concurrent.futures

    from fastapi.testclient import TestClient
    srv.engine, srv.served_model = eng, "tiny"
    client = TestClient(srv.app)
    assert client.get("/readyz").status_code == 200

    def ask(text):
        r = client.post("/v1/chat/completions", json=dict(BODY, messages=[{"role": "user", "content": text}]))
        assert r.status_code == 200, r.text
        return r.json()["choices"][0]["message"]["content"], r.json()["usage"]["completion_tokens"]

    with concurrent.futures.ThreadPoolExecutor(4) as pool:        # concurrent, so the router has a choice to make
        answers = list(pool.map(ask, PROMPTS))
    with client.stream("POST", "/v1/chat/completions",
                       json=dict(BODY, stream=True, max_tokens=4, messages=[{"role": "user", "content": PROMPTS[0]}])) as s:
        lines = [ln for ln in s.iter_lines() if ln.startswith("data:")]
    stats = eng.stats().get("data_parallel")
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump({"answers": answers, "stream_tail": lines[-1], "stream_chunks": len(lines), "stats": stats}, f)
    eng.shutdown()


def test_two_replica_server_routes_and_streams():
    from fastapi.testclient import TestClient

    from litevllm_b200.entrypoints.openai import api_server as srv
    single = srv.build_engine("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=4, max_model_len=128)
    srv.engine, srv.served_model = single, "tiny"
    client = TestClient(srv.app)
    want = []
    for text in PROMPTS:
        r = client.post("/v1/chat/completions", json=dict(BODY, messages=[{"role": "user", "content": text}]))
        want.append(r.json()["choices"][0]["message"]["content"])
    single.shutdown()
    with tempfile.TemporaryDirectory() as d:
        spawn(_dp_worker, 2, args=(d,), port=29591)
        r0 = json.load(open(os.path.join(d, "rank0.json")))
        r1 = json.load(open(os.path.join(d, "rank1.json")))
    assert [a[0] for a in r0["answers"]] == want and all(a[1] == 6 for a in r0["answers"])
    assert r0["stream_tail"] == "data: [DONE]" and r0["stream_chunks"] >= 3
    assert len(r1["served"]) >= 1, "no request reached the second replica"
    assert r0["stats"]["replicas"] == 2 and sum(r0["stats"]["inflight"]) == 0


def _dp_storm_worker(rank, world, out_dir):
    import asyncio
    import random

    from litevllm_b200 import SamplingParams
    from litevllm_b200.engine.errors import LiteRuntimeError
    from litevllm_b200.entrypoints.openai import api_server as srv
    eng = srv.build_engine("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=3, max_model_len=96,
                           data_parallel_size=world)
    if eng.is_worker_rank:
        steps = eng.serve_as_worker(None)
        inner = eng.engine
        with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
            json.dump({"steps": steps, "running": inner.stats()["scheduler"]["running"],
                       "free": inner.kv_manager.allocator.num_free, "total": inner.plan.num_total_blocks}, f)
        eng.shutdown()
        return
    rng = random.Random(44)
    plans = [(f"u{i}", [rng.randint(2, 400) for _ in range(rng.randint(3, 30))], rng.randint(1, 8),
              rng.random() < 0.35, rng.randint(0, 2)) for i in range(18)]

    async def client(rid, ids, mt, leaves, after):
        await asyncio.sleep(rng.random() * 0.05)
        sp = SamplingParams(temperature=0.0, max_tokens=mt, ignore_eos=True)
        while True:
            try:
                await eng.submit({"prompt_token_ids": ids}, sp, rid)
                break
            except LiteRuntimeError:
                await asyncio.sleep(0.01)
        seen, last = 0, None
        agen = eng.stream(rid)
        try:
            async for out in agen:
                seen, last = seen + 1, out
                if leaves and seen > after and not out.finished:
                    return rid, None
        finally:
            await agen.aclose()
        return rid, list(last.outputs[0].token_ids)

    async def run():
        res = dict(await asyncio.gather(*[client(*p) for p in plans]))
        for _ in range(500):
            if sum(eng.stats()["data_parallel"]["inflight"]) == 0 and eng.stats()["scheduler"]["running"] == 0:
                break
            await asyncio.sleep(0.01)
        return res

    results = asyncio.run(run())
    stats = eng.stats()
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        r = eng.dp_router
        json.dump({"results": results, "plans": [(p[0], p[1], p[2]) for p in plans], "inflight": stats["data_parallel"]["inflight"],
                   "running": stats["scheduler"]["running"], "owner": dict(r.owner), "done": list(r._done),
                   "leavers": [p[0] for p in plans if p[3]]}, f)
    eng.shutdown()


def test_replicas_serve_a_storm_of_clients():
    """Eighteen clients, a third disconnecting mid-stream, routed over two replicas: whoever stays gets the tokens a
    single engine produces, nothing stays in flight, the remote replica ends with every block free."""
    from litevllm_b200 import LLM, SamplingParams
    with tempfile.TemporaryDirectory() as d:
        spawn(_dp_storm_worker, 2, args=(d,), port=29592)
        r0 = json.load(open(os.path.join(d, "rank0.json")))
        r1 = json.load(open(os.path.join(d, "rank1.json")))
    assert r0["inflight"] == [0, 0] and r0["running"] == 0
    assert r1["running"] == 0 and r1["free"] == r1["total"] - 1 and r1["steps"] > 0
    ref = LLM("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=3, max_model_len=96)
    stayed = 0
    for rid, ids, mt in r0["plans"]:
        got = r0["results"][rid]
        if got is None:
            continue
        stayed += 1
        want = ref.generate([{"prompt_token_ids": ids}], SamplingParams(temperature=0.0, max_tokens=mt, ignore_eos=True))
        assert got == want[0].outputs[0].token_ids, rid
    ref.shutdown()
    assert stayed >= 9
