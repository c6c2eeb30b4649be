"""Sampling stages and structured-output constraints on the CPU."""
import torch

from litevllm_b200.engine.request_state import RequestState
from litevllm_b200.engine.sampling.penalty_encoder import PenaltyEncoder
from litevllm_b200.engine.sampling.sampler import Sampler
from litevllm_b200.engine.structured_constraints import (ChoiceTrieConstraint, JsonPrefixConstraint,
                                                         _is_json_prefix, build_constraint)
from litevllm_b200.sampling_params import SamplingParams, StructuredOutputsParams


def _req(**kw):
    gen = kw.pop("generated", [])
    st = RequestState("r", None, [1, 2, 3], SamplingParams(**kw))
    st.generated_ids = list(gen)
    return st


def test_greedy_is_argmax_and_seeded_sampling_repeats():
    logits = torch.randn(3, 50)
    s = Sampler()
    greedy = [_req(temperature=0.0) for _ in range(3)]
    assert s.sample(logits.clone(), greedy).tolist() == logits.argmax(-1).tolist()

    def draw():
        reqs = [_req(temperature=0.9, top_k=10, top_p=0.8, seed=7) for _ in range(3)]
        for r in reqs:
            r.rng = torch.Generator().manual_seed(7)
        return s.sample(logits.clone(), reqs).tolist()
    assert draw() == draw()


def test_top_k_one_and_tiny_top_p_reduce_to_argmax():
    logits = torch.randn(4, 100)
    s = Sampler()
    for kw in (dict(top_k=1), dict(top_p=1e-6)):
        reqs = [_req(temperature=1.0, **kw) for _ in range(4)]
        for r in reqs:
            r.rng = torch.Generator().manual_seed(0)
        assert s.sample(logits.clone(), reqs).tolist() == logits.argmax(-1).tolist()


def test_min_p_masks_unlikely_tokens():
    logits = torch.full((1, 10), -10.0)
    logits[0, 3] = 5.0
    logits[0, 4] = 4.9
    r = _req(temperature=1.0, min_p=0.5)
    r.rng = torch.Generator().manual_seed(1)
    picks = {int(Sampler().sample(logits.clone(), [r])[0]) for _ in range(50)}
    assert picks <= {3, 4}


def test_penalties_apply_to_generated_tokens_only():
    enc = PenaltyEncoder(20)
    logits = torch.ones(1, 20)
    r = _req(temperature=0.0, repetition_penalty=2.0, frequency_penalty=0.5, presence_penalty=0.25, generated=[5, 5, 7])
    out = enc.encode(logits.clone(), [r])
    assert torch.isclose(out[0, 5], torch.tensor(1 / 2.0 - 0.5 * 2 - 0.25))
    assert torch.isclose(out[0, 7], torch.tensor(1 / 2.0 - 0.5 * 1 - 0.25))
    assert float(out[0, 1]) == 1.0 and float(out[0, 2]) == 1.0      # prompt tokens untouched


def test_eos_masked_until_min_tokens_and_logit_bias():
    enc = PenaltyEncoder(10)
    r = _req(temperature=0.0, min_tokens=3, logit_bias={4: 2.5}, generated=[1])
    r.eos_token_ids = frozenset({9})
    out = enc.encode(torch.zeros(1, 10), [r])
    assert out[0, 9] == float("-inf") and float(out[0, 4]) == 2.5
    r.generated_ids = [1, 2, 3]
    assert not PenaltyEncoder.needs_encoding([_req(temperature=0.0)])
    out = enc.encode(torch.zeros(1, 10), [r])
    assert float(out[0, 9]) == 0.0


class _CharTok:
    """One token per character; id = ord."""
    def encode(self, text, add_special_tokens=True):
        return [ord(c) for c in text]

    def decode(self, ids, **kw):
        return "".join(chr(i) for i in ids)


def test_choice_trie_constraint_walks_one_option():
    c = ChoiceTrieConstraint(["yes", "no"], _CharTok(), 128)
    row = torch.zeros(128)
    row[ord("n")] = 1.0
    c.apply_mask(row)
    assert set(torch.nonzero(torch.isfinite(row)).flatten().tolist()) == {ord("y"), ord("n")}
    c.on_token(ord("n"))
    row = torch.zeros(128)
    c.apply_mask(row)
    assert torch.nonzero(torch.isfinite(row)).flatten().tolist() == [ord("o")]
    c.on_token(ord("o"))
    assert c.should_finish()


def test_json_prefix_constraint():
    assert _is_json_prefix('{"a": [1, 2') and not _is_json_prefix('{"a": ]') and not _is_json_prefix("}")
    c = JsonPrefixConstraint(_CharTok(), top_n=128)
    row = torch.zeros(128)
    c.apply_mask(row)
    ok = set(torch.nonzero(torch.isfinite(row)).flatten().tolist())
    assert ord("{") in ok and ord("}") not in ok and ord("x") not in ok
    for ch in '{"k":1}':
        c.on_token(ord(ch))
    assert c.should_finish()


def test_build_constraint_falls_back_without_a_real_vocabulary():
    c = build_constraint(StructuredOutputsParams(choice=["a", "b"]), _CharTok(), 128)
    assert isinstance(c, ChoiceTrieConstraint)
    assert build_constraint(StructuredOutputsParams(), _CharTok(), 128) is None
