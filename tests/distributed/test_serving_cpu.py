"""Multi-rank serving as gloo ranks on the CPU: rank 0 answers ``POST /v1/chat/completions`` through
FastAPI's TestClient while rank 1 mirrors its engine through the control channel; both ranks must
have generated the same tokens (tensor parallel, so every step needs both of them)."""
import json
import os
import tempfile

from litevllm_b200.parallel.launcher import spawn


def _serve_worker(rank, world, out_dir):
    from litevllm_b200.entrypoints.openai import api_server as srv
    eng = srv.build_engine("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=4, max_model_len=128,
                           tensor_parallel_size=world, comm_backend="nccl")
    produced: dict = {}

    def on_step(outs):
        for o in outs:
            if o is not None and o.finished:
                produced[o.request_id] = list(o.outputs[0].token_ids)

    if eng.is_worker_rank:
        steps = eng.serve_as_worker(on_step)
        with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
            json.dump({"tokens": sorted(produced.values()), "steps": steps}, f)
        eng.shutdown()
        return
    from fastapi.testclient import TestClient
    orig_step = eng.engine.step

    def recording_step():
        outs = orig_step()
        on_step(outs)
        return outs
    eng.engine.step = recording_step
    srv.engine, srv.served_model = eng, "tiny"
    client = TestClient(srv.app)
    assert client.get("/readyz").status_code == 200
    results = []
    body = {"model": "tiny", "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 6, "temperature": 0}
    r = client.post("/v1/chat/completions", json=body)
    assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] == 6
    results.append(r.json()["choices"][0]["message"]["content"])
    # a sampled request: rank 0 assigns the seed, the worker must draw the same tokens
    r2 = client.post("/v1/chat/completions", json=dict(body, temperature=0.9, top_p=0.9, max_tokens=5,
                                                       messages=[{"role": "user", "content": "second"}]))
    assert r2.status_code == 200
    # a streamed request
    with client.stream("POST", "/v1/chat/completions", json=dict(body, stream=True, max_tokens=4)) as s:
        lines = [l for l in s.iter_lines() if l.startswith("data:")]
    assert lines[-1] == "data: [DONE]"
    # rank 0's own record of what each finished request produced
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump({"ok": True, "messages": eng.coordinator.messages, "tokens": sorted(produced.values())}, f)
    eng.shutdown()          # publishes the shutdown message; the worker leaves its loop


def test_two_rank_server_mirrors_requests():
    with tempfile.TemporaryDirectory() as d:
        spawn(_serve_worker, 2, args=(d,), port=29561)
        r0 = json.load(open(os.path.join(d, "rank0.json")))
        r1 = json.load(open(os.path.join(d, "rank1.json")))
    assert r0["ok"] and r0["messages"] >= 3
    assert len(r1["tokens"]) == 3 and sorted(len(t) for t in r1["tokens"]) == [4, 5, 6]
    assert r1["steps"] > 0
    assert r0["tokens"] == r1["tokens"], "the worker rank generated different tokens than rank 0"


def _serve_storm_worker(rank, world, out_dir):
    import asyncio
    import random

    from litevllm_b200 import SamplingParams
    from litevllm_b200.entrypoints.openai import api_server as srv
    from litevllm_b200.engine.errors import LiteRuntimeError
    eng = srv.build_engine("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=3, max_model_len=96,
                           tensor_parallel_size=world, comm_backend="nccl")
    produced: dict = {}

    def on_step(outs):
        for o in outs:
            if o is not None and o.finished:
                produced[o.request_id] = list(o.outputs[0].token_ids)

    if eng.is_worker_rank:
        steps = eng.serve_as_worker(on_step)
        inner = eng.engine
        with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
            json.dump({"tokens": produced, "steps": steps, "running": inner.stats()["scheduler"]["running"],
                       "free": inner.kv_manager.allocator.num_free, "total": inner.plan.num_total_blocks}, f)
        eng.shutdown()
        return
    orig_step = eng.engine.step

    def recording_step():
        outs = orig_step()
        on_step(outs)
        return outs
    eng.engine.step = recording_step
    rng = random.Random(33)
    plans = [(f"u{i}", [rng.randint(2, 400) for _ in range(rng.randint(3, 30))], rng.randint(1, 8),
              rng.random() < 0.35, rng.randint(0, 2)) for i in range(16)]

    async def client(rid, ids, mt, leaves, after):
        await asyncio.sleep(rng.random() * 0.05)
        sp = SamplingParams(temperature=0.0, max_tokens=mt, ignore_eos=True)
        while True:
            try:
                await eng.submit({"prompt_token_ids": ids}, sp, rid)
                break
            except LiteRuntimeError:
                await asyncio.sleep(0.01)
        seen = 0
        agen = eng.stream(rid)
        try:
            async for out in agen:
                seen += 1
                if leaves and seen > after and not out.finished:
                    return rid, False
        finally:
            await agen.aclose()
        return rid, True

    async def run():
        res = dict(await asyncio.gather(*[client(*p) for p in plans]))
        for _ in range(500):
            s = eng.stats()["scheduler"]
            if s["running"] == 0 and s["queued"] == 0:
                break
            await asyncio.sleep(0.01)
        return res

    stayed = asyncio.run(run())
    inner = eng.engine
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump({"tokens": produced, "stayed": stayed, "running": inner.stats()["scheduler"]["running"],
                   "free": inner.kv_manager.allocator.num_free, "total": inner.plan.num_total_blocks}, f)
    eng.shutdown()


def test_mirrored_worker_follows_a_storm_of_clients():
    """Sixteen clients of rank 0's server, a third of them disconnect mid-stream: the worker rank, which only sees
    the admissions and aborts rank 0 publishes before each step, finishes the same requests with the same tokens
    and ends with every block free."""
    with tempfile.TemporaryDirectory() as d:
        spawn(_serve_storm_worker, 2, args=(d,), port=29565)
        r0 = json.load(open(os.path.join(d, "rank0.json")))
        r1 = json.load(open(os.path.join(d, "rank1.json")))
    assert r0["tokens"] == r1["tokens"], "the worker rank generated different tokens than rank 0"
    finished_all = [rid for rid, ok in r0["stayed"].items() if ok]
    assert len(finished_all) >= 8 and all(rid in r0["tokens"] for rid in finished_all)
    for r in (r0, r1):
        assert r["running"] == 0 and r["free"] == r["total"] - 1
