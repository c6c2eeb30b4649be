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
