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
