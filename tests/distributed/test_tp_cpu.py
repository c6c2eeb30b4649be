"""Tensor-parallel sharding and the library-collective path, run as gloo ranks on the CPU."""
import json
import os
import tempfile

import pytest
import torch

from litevllm_b200.parallel.launcher import spawn


def _prompts():
    g = torch.Generator().manual_seed(5)
    return [torch.randint(0, 512, (n,), generator=g).tolist() for n in (9, 40, 23)]


def _tp_worker(rank, world, out_dir, preset):
    from litevllm_b200 import LLM, SamplingParams
    llm = LLM(f"synthetic:{preset}", dtype="float32", device="cpu", max_num_seqs=4, max_model_len=128,
              tensor_parallel_size=world, comm_backend="nccl")
    outs = llm.generate(_prompts(), SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump([o.outputs[0].token_ids for o in outs], f)
    llm.shutdown()


@pytest.mark.parametrize("preset", ["tiny-llama-test", "tiny-llama-awq-test"])
def test_tp2_matches_single_rank(preset):
    from litevllm_b200 import LLM, SamplingParams
    ref = LLM(f"synthetic:{preset}", dtype="float32", device="cpu", max_num_seqs=4, max_model_len=128)
    want = [o.outputs[0].token_ids for o in
            ref.generate(_prompts(), SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))]
    with tempfile.TemporaryDirectory() as d:
        spawn(_tp_worker, 2, args=(d, preset), port=29541 if "awq" in preset else 29542)
        got = [json.load(open(os.path.join(d, f"rank{r}.json"))) for r in range(2)]
    assert got[0] == got[1], "ranks diverged"
    assert got[0] == want


def _ep_worker(rank, world, out_dir, preset):
    from litevllm_b200 import LLM, SamplingParams
    llm = LLM(f"synthetic:{preset}", dtype="float32", device="cpu", max_num_seqs=4, max_model_len=128,
              expert_parallel_size=world, comm_backend="nccl")
    outs = llm.generate(_prompts(), SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump([o.outputs[0].token_ids for o in outs], f)
    llm.shutdown()


@pytest.mark.parametrize("preset", ["tiny-gemma4-moe-test", "tiny-deepseek-test"])
def test_ep2_matches_single_rank(preset):
    """Expert parallelism: experts split over two ranks, partial outputs summed; same tokens as one rank."""
    from litevllm_b200 import LLM, SamplingParams
    ref = LLM(f"synthetic:{preset}", dtype="float32", device="cpu", max_num_seqs=4, max_model_len=128)
    want = [o.outputs[0].token_ids for o in
            ref.generate(_prompts(), SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))]
    with tempfile.TemporaryDirectory() as d:
        spawn(_ep_worker, 2, args=(d, preset), port=29543 if "gemma" in preset else 29544)
        got = [json.load(open(os.path.join(d, f"rank{r}.json"))) for r in range(2)]
    assert got[0] == got[1], "ranks diverged"
    assert got[0] == want


def _staged_ep_worker(rank, world, out_dir, preset, budget_gb):
    os.environ["FI_EXPERT_STAGING_GB"] = budget_gb
    from litevllm_b200 import LLM, SamplingParams
    llm = LLM(f"synthetic:{preset}", dtype="float32", device="cpu", max_num_seqs=4, max_model_len=128,
              expert_parallel_size=world, comm_backend="nccl")
    outs = llm.generate(_prompts(), SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump({"tokens": [o.outputs[0].token_ids for o in outs], "staging": llm.engine.stats()["expert_staging"]}, f)
    llm.shutdown()


def test_ep2_with_staged_experts_matches_single_rank():
    """Each rank owns four of the eight experts and keeps two of them on the device at a time."""
    from litevllm_b200 import LLM, SamplingParams
    from litevllm_b200.models.deepseek_mla import RoutedExperts
    preset = "tiny-deepseek-test"
    ref = LLM(f"synthetic:{preset}", dtype="float32", device="cpu", max_num_seqs=4, max_model_len=128)
    want = [o.outputs[0].token_ids for o in
            ref.generate(_prompts(), SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))]
    blocks = [m for m in ref.engine.model.modules() if isinstance(m, RoutedExperts)]
    per_expert = sum(int(t[0].numel()) * t.element_size() for t in blocks[0].raw.values())
    ref.shutdown()
    budget = repr(2.5 * per_expert * len(blocks) / 2 ** 30)
    with tempfile.TemporaryDirectory() as d:
        spawn(_staged_ep_worker, 2, args=(d, preset, budget), port=29548)
        got = [json.load(open(os.path.join(d, f"rank{r}.json"))) for r in range(2)]
    assert got[0]["tokens"] == got[1]["tokens"] == want
    for g in got:
        assert g["staging"]["slots_per_block"] == 2 and g["staging"]["experts_per_block"] == 4
        assert g["staging"]["evictions"] > 0


def _tpep_worker(rank, world, out_dir, preset):
    from litevllm_b200 import LLM, SamplingParams
    llm = LLM(f"synthetic:{preset}", dtype="float32", device="cpu", max_num_seqs=4, max_model_len=128,
              tensor_parallel_size=world, expert_parallel_size=world, comm_backend="nccl")
    outs = llm.generate(_prompts(), SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump([o.outputs[0].token_ids for o in outs], f)
    llm.shutdown()


@pytest.mark.parametrize("preset", ["tiny-gemma4-moe-test", "tiny-deepseek-test"])
def test_tp2_with_ep2_matches_single_rank(preset):
    """Both at once on the same two ranks: attention and dense layers tensor parallel, experts sharded."""
    from litevllm_b200 import LLM, SamplingParams
    ref = LLM(f"synthetic:{preset}", dtype="float32", device="cpu", max_num_seqs=4, max_model_len=128)
    want = [o.outputs[0].token_ids for o in
            ref.generate(_prompts(), SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))]
    with tempfile.TemporaryDirectory() as d:
        spawn(_tpep_worker, 2, args=(d, preset), port=29545 if "gemma" in preset else 29546)
        got = [json.load(open(os.path.join(d, f"rank{r}.json"))) for r in range(2)]
    assert got[0] == got[1], "ranks diverged"
    assert got[0] == want


def _a2a_unit_worker(rank, world, out_dir):
    import torch
    from litevllm_b200.parallel import ep_alltoall, state as pstate
    pstate.init_parallel(tp=1, ep=world, comm_backend="nccl", backend="gloo")
    g = torch.Generator().manual_seed(5)
    T, K, H, per = 7, 2, 8, 4
    E = per * world
    x = torch.randn(T, H, generator=g)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)])
    w = torch.rand(T, K, generator=g)
    gain = torch.arange(1, E + 1, dtype=torch.float32)
    seen = []

    def run(rows, expert_ids):
        seen.append(expert_ids.clone())
        return rows * gain[expert_ids].unsqueeze(-1)

    out = ep_alltoall.sharded_moe(x, ids, w, per, run)
    want = (x.unsqueeze(1) * gain[ids].unsqueeze(-1) * w.unsqueeze(-1)).sum(1)
    mine_only = all(bool(((s // per) == rank).all()) for s in seen)
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump({"err": float((out - want).abs().max()), "mine_only": mine_only}, f)


@pytest.mark.parametrize("world", [2, 3])
def test_alltoall_dispatch_combine_matches_replicated_sum(world):
    """Routes reach only the rank that owns their expert, results come back to the token's rank, and after the
    all-gather every rank holds what the replicated computation gives (7 tokens: uneven slices)."""
    with tempfile.TemporaryDirectory() as d:
        spawn(_a2a_unit_worker, world, args=(d,), port=29547 + world)
        got = [json.load(open(os.path.join(d, f"rank{r}.json"))) for r in range(world)]
    assert all(g["err"] < 1e-5 and g["mine_only"] for g in got), got


def _ep_alltoall_worker(rank, world, out_dir, preset):
    from litevllm_b200.parallel import ep_alltoall
    assert ep_alltoall.ENABLED, "the switch did not reach the rank process"
    calls = []
    inner = ep_alltoall.dispatch_combine
    ep_alltoall.dispatch_combine = lambda *a, **k: (calls.append(1), inner(*a, **k))[1]
    _ep_worker(rank, world, out_dir, preset)
    assert calls, "the all-to-all path was not taken"


@pytest.mark.parametrize("preset", ["tiny-gemma4-moe-test", "tiny-deepseek-test"])
def test_ep2_alltoall_path_matches_single_rank(preset, monkeypatch):
    """``FI_EP_ALLTOALL=1``: the MoE blocks shard the step's tokens over the ranks and exchange routes by
    all-to-all; tokens equal the single-rank run."""
    from litevllm_b200 import LLM, SamplingParams
    ref = LLM(f"synthetic:{preset}", dtype="float32", device="cpu", max_num_seqs=4, max_model_len=128)
    want = [o.outputs[0].token_ids for o in
            ref.generate(_prompts(), SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))]
    monkeypatch.setenv("FI_EP_ALLTOALL", "1")
    with tempfile.TemporaryDirectory() as d:
        spawn(_ep_alltoall_worker, 2, args=(d, preset), port=29551 if "gemma" in preset else 29552)
        got = [json.load(open(os.path.join(d, f"rank{r}.json"))) for r in range(2)]
    assert got[0] == got[1] == want


def _storm(llm, seed, n_requests=9):
    """Random arrivals and aborts driven through the engine; returns {request id: tokens} of what finished."""
    import random

    from litevllm_b200 import SamplingParams
    from litevllm_b200.engine.errors import RequestRejectedError
    rng = random.Random(seed)
    eng = llm.engine
    specs = {f"s{i}": ([rng.randint(2, 400) for _ in range(rng.randint(3, 40))], rng.randint(1, 7)) for i in range(n_requests)}
    pending = list(specs)
    rng.shuffle(pending)
    doomed = set(rng.sample(pending, 2))
    finished, live, steps = {}, set(), 0
    while pending or eng.has_unfinished_requests():
        steps += 1
        assert steps < 2000
        if pending and rng.random() < 0.5:
            rid = pending.pop()
            ids, mt = specs[rid]
            try:
                eng.add_request(rid, {"prompt_token_ids": ids}, SamplingParams(max_tokens=mt, temperature=0.0, ignore_eos=True))
                live.add(rid)
            except RequestRejectedError:
                pending.insert(0, rid)
        for rid in list(live & doomed):
            if rng.random() < 0.2:
                eng.abort_request(rid)
                live.discard(rid)
                doomed.discard(rid)
        for o in eng.step():
            if o is not None and o.finished:
                finished[o.request_id] = o.outputs[0].token_ids
                live.discard(o.request_id)
    assert eng.kv_manager.allocator.num_free == eng.plan.num_total_blocks - 1
    return finished


def _storm_worker(rank, world, out_dir, preset, mode):
    from litevllm_b200 import LLM
    kw = {"tensor_parallel_size": world} if mode == "tp" else {"expert_parallel_size": world}
    llm = LLM(f"synthetic:{preset}", dtype="float32", device="cpu", max_num_seqs=3, max_model_len=96,
              comm_backend="nccl", **kw)
    got = _storm(llm, seed=11)
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump(got, f)
    llm.shutdown()


@pytest.mark.parametrize("preset,mode", [("tiny-llama-test", "tp"), ("tiny-gemma4-moe-test", "ep")])
def test_ranks_stay_in_step_through_random_arrivals_and_aborts(preset, mode):
    """Every rank runs the same seeded storm (the control plane is deterministic, so no plan is exchanged): the
    ranks must finish the same requests with the same tokens as one rank alone."""
    from litevllm_b200 import LLM
    ref = LLM(f"synthetic:{preset}", dtype="float32", device="cpu", max_num_seqs=3, max_model_len=96)
    want = _storm(ref, seed=11)
    ref.shutdown()
    with tempfile.TemporaryDirectory() as d:
        spawn(_storm_worker, 2, args=(d, preset, mode), port=29563 if mode == "tp" else 29564)
        got = [json.load(open(os.path.join(d, f"rank{r}.json"))) for r in range(2)]
    assert got[0] == got[1] == want
