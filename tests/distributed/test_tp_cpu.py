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
