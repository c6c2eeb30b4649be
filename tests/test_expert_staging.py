"""Routed experts behind a device budget: slot bookkeeping of the stager, and models whose experts are staged
produce what the fully resident models produce."""
import random

import pytest
import torch

from litevllm_b200.layers.expert_stager import ExpertStager, budget_bytes_from_env


def _host(E=8, rows=4, width=16):
    g = torch.Generator().manual_seed(0)
    return {"gate": torch.randint(0, 255, (E, rows, width), generator=g, dtype=torch.uint8),
            "down": torch.randint(0, 255, (E, 2, width), generator=g, dtype=torch.uint8)}


def _check_slab(st: ExpertStager):
    for e in st.resident():
        for k in st.names:
            assert torch.equal(st.slab[k][st.slot_of(e)], st.host[k][e])
    slots = [st.slot_of(e) for e in st.resident()]
    assert len(set(slots)) == len(slots) and all(0 <= s < st.slots for s in slots)


def test_budget_sets_the_slot_count():
    host = _host()
    per = 4 * 16 + 2 * 16
    assert ExpertStager(host, "cpu", 3 * per + 5).slots == 3
    assert ExpertStager(host, "cpu", 0).slots == 1                      # never fewer than the minimum
    assert ExpertStager(host, "cpu", 0, min_slots=2).slots == 2
    assert ExpertStager(host, "cpu", 10 ** 9).slots == 8                # never more than there are experts
    st = ExpertStager(host, "cpu", 3 * per)
    assert st.bytes_per_expert == per and st.device_bytes == 3 * per
    with pytest.raises(ValueError):
        ExpertStager({"a": torch.zeros(3, 2), "b": torch.zeros(4, 2)}, "cpu", 100)


def test_least_recently_used_expert_is_evicted_first():
    st = ExpertStager(_host(), "cpu", 3 * 96)
    st.stage([0]); st.stage([1]); st.stage([2])
    assert st.resident() == [0, 1, 2] and st.stats["misses"] == 3 and st.stats["evictions"] == 0
    st.stage([0])                                   # refresh 0: 1 is now the oldest
    st.stage([5])
    assert st.resident() == [0, 2, 5] and st.stats["evictions"] == 1 and st.stats["hits"] == 1
    st.stage([2, 7])                                # 2 stays although it is older than 5: the wave needs it
    assert st.resident() == [2, 5, 7]
    _check_slab(st)
    assert st.stats["bytes_staged"] == 5 * 96


def test_pinned_experts_survive_any_traffic():
    st = ExpertStager(_host(), "cpu", 3 * 96)
    st.pin([4, 6])
    for e in (0, 1, 2, 3, 5, 7, 0, 1):
        st.stage([e])
        assert {4, 6} <= set(st.resident())
    _check_slab(st)
    with pytest.raises(ValueError):
        st.pin([0])                                 # would leave no evictable slot
    st.unpin([4])
    st.stage([1]); st.stage([2])
    assert 6 in st.resident() and 4 not in st.resident()
    with pytest.raises(IndexError):
        st.stage([8])


def test_hot_experts_are_chosen_by_use():
    st = ExpertStager(_host(), "cpu", 4 * 96)
    for e in (3, 3, 3, 5, 5, 1, 0, 2, 6):
        st.stage([e])
    assert st.pin_hot(2) == [3, 5] and st.pinned() == [3, 5]
    assert st.pin_hot(10) == [3, 5, 0]              # capped so that a slot stays evictable; ties by number
    _check_slab(st)


def test_a_step_with_more_experts_than_slots_runs_in_waves():
    st = ExpertStager(_host(), "cpu", 3 * 96)
    st.pin([7])
    st.stage([2])
    waves = st.waves([0, 1, 2, 3, 7, 7, 2])
    assert waves[0][0] == 7 and waves[0][1] == 2    # pinned and resident experts lead
    assert sorted(e for w in waves for e in w) == [0, 1, 2, 3, 7]
    assert all(len(set(w) | {7}) <= st.slots for w in waves)
    assert st.waves([]) == [] and st.waves([7]) == [[7]]
    ids = torch.tensor([[0, 7], [3, 2], [9, 1]])    # 9: another rank's expert
    seen = torch.zeros_like(ids)
    for w in waves:
        placed = st.stage(w)
        slots = st.slot_ids(ids, placed)
        assert slots.dtype == ids.dtype
        for (t, k), s in zip([(t, k) for t in range(3) for k in range(2)], slots.flatten().tolist()):
            e = int(ids[t, k])
            if s >= 0:
                assert e in placed and placed[e] == s
                seen[t, k] += 1
            else:
                assert e not in placed
        _check_slab(st)
    assert seen.tolist() == [[1, 1], [1, 1], [0, 1]]          # every local route in exactly one wave
    shifted = st.slot_ids(ids + 16, st.stage([0]), e_lo=16)
    assert shifted[0, 0] == st.slot_of(0) and int((shifted >= 0).sum()) == 1


def test_random_traffic_keeps_the_books_straight():
    rng = random.Random(3)
    st = ExpertStager(_host(E=16), "cpu", 5 * 96)
    st.pin([rng.randrange(16)])
    for step in range(200):
        need = rng.sample(range(16), rng.randint(1, 9))
        for w in st.waves(need):
            placed = st.stage(w)
            assert set(placed) == set(w)
            _check_slab(st)
        if step % 50 == 49:
            st.pin_hot(2)
    snap = st.snapshot()
    assert snap["hits"] + snap["misses"] >= 200 and 0 < snap["hit_rate"] < 1 and snap["resident"] <= 5
    assert snap["device_bytes"] == 5 * 96 and snap["host_bytes"] == 16 * 96


def test_budget_from_the_environment(monkeypatch):
    monkeypatch.delenv("FI_EXPERT_STAGING_GB", raising=False)
    assert budget_bytes_from_env() is None
    monkeypatch.setenv("FI_EXPERT_STAGING_GB", "0.5")
    assert budget_bytes_from_env() == 2 ** 29
    monkeypatch.setenv("FI_EXPERT_STAGING_GB", "-1")
    with pytest.raises(ValueError):
        budget_bytes_from_env()


def _generate(name, **kw):
    from litevllm_b200 import LLM, SamplingParams
    llm = LLM(f"synthetic:{name}", dtype="float32", device="cpu", max_num_seqs=4, max_model_len=128, **kw)
    prompts = [{"prompt_token_ids": [(7 * i + 3 * j) % 500 + 2 for i in range(20 + 5 * j)]} for j in range(3)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    tokens = [o.outputs[0].token_ids for o in outs]
    return llm, tokens


def _experts(llm):
    from litevllm_b200.models.deepseek_mla import RoutedExperts
    return [m for m in llm.engine.model.modules() if isinstance(m, RoutedExperts)] or \
        [l.routed for l in getattr(llm.engine.model, "layers", []) if getattr(l, "routed", None) is not None]


@pytest.mark.parametrize("name", ["tiny-deepseek-test"])
def test_staged_experts_generate_what_resident_experts_generate(name, monkeypatch):
    monkeypatch.delenv("FI_EXPERT_STAGING_GB", raising=False)
    ref, want = _generate(name)
    assert all(e.stager is None and e.raw for e in _experts(ref))
    ref.shutdown()
    # 8 experts per block; a budget of three experts per block: prefill steps name more experts than slots
    blocks = _experts(ref)
    per_expert = sum(int(t[0].numel()) * t.element_size() for t in blocks[0].raw.values())
    monkeypatch.setenv("FI_EXPERT_STAGING_GB", repr(3.2 * per_expert * len(blocks) / 2 ** 30))
    llm, got = _generate(name)
    assert got == want
    staged = _experts(llm)
    assert staged and all(e.stager is not None and not e.raw for e in staged)
    for e in staged:
        snap = e.stager.snapshot()
        assert snap["slots"] == 3 and snap["waves"] > snap["steps"] > 0 and snap["evictions"] > 0
        assert snap["device_bytes"] < snap["host_bytes"]
    assert llm.engine.model.supports_cuda_graph is False
    from litevllm_b200.layers import expert_stager
    total = llm.engine.stats()["expert_staging"]
    assert total["blocks"] == len(staged) and total["slots_per_block"] == 3 and 0 < total["hit_rate"] < 1
    assert total["bytes_staged"] == sum(e.stager.stats["bytes_staged"] for e in staged)
    assert expert_stager.pin_hot_experts(llm.engine.model, 2) == 2 * len(staged) and \
        llm.engine.stats()["expert_staging"]["pinned"] == 2 * len(staged)
    again = [o.outputs[0].token_ids for o in llm.generate(
        [{"prompt_token_ids": [(7 * i + 3 * j) % 500 + 2 for i in range(20 + 5 * j)]} for j in range(3)],
        __import__("litevllm_b200").SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))]
    assert again == want                           # pinned experts change residency, not results
    llm.shutdown()


def test_a_budget_that_holds_everything_turns_staging_off(monkeypatch):
    monkeypatch.setenv("FI_EXPERT_STAGING_GB", "1")
    llm, got = _generate("tiny-deepseek-test")
    monkeypatch.delenv("FI_EXPERT_STAGING_GB")
    assert all(e.stager is None and e.raw and not e.host for e in _experts(llm))
    llm.shutdown()
    ref, want = _generate("tiny-deepseek-test")
    ref.shutdown()
    assert got == want


def test_hot_experts_are_pinned_automatically_after_the_configured_steps(monkeypatch):
    from litevllm_b200.layers.expert_stager import auto_pin_from_env
    monkeypatch.delenv("FI_EXPERT_STAGING_PIN_HOT", raising=False)
    assert auto_pin_from_env() == (0, 0)
    monkeypatch.setenv("FI_EXPERT_STAGING_PIN_HOT", "2")
    assert auto_pin_from_env() == (2, 64)
    monkeypatch.setenv("FI_EXPERT_STAGING_PIN_HOT", "2@3")
    st = ExpertStager(_host(), "cpu", 4 * 96)
    for need in ([1, 5], [5, 6], [5, 1]):
        st.begin_step()
        st.stage(need)
        assert st.pinned() == []
    st.begin_step()                                  # the fourth step: three steps of traffic decide
    assert st.pinned() == [1, 5]
    for e in (0, 2, 3, 4, 6, 7):
        st.begin_step()
        st.stage([e])
    assert {1, 5} <= set(st.resident()) and st.pinned() == [1, 5]
    monkeypatch.setenv("FI_EXPERT_STAGING_PIN_HOT", "-1")
    with pytest.raises(ValueError):
        auto_pin_from_env()


@pytest.mark.parametrize("name", ["tiny-deepseek-test", "tiny-deepseek-v4-flash-blocks-test"])
def test_the_budget_can_come_with_the_model_configuration(name, monkeypatch):
    monkeypatch.delenv("FI_EXPERT_STAGING_GB", raising=False)
    ref, want = _generate(name)
    ref.shutdown()
    llm, got = _generate(name, hf_overrides={"expert_staging_gb": 1e-9})
    assert got == want
    st = llm.engine.stats()["expert_staging"]
    assert st["blocks"] >= 1 and st["slots_per_block"] == 2 and st["evictions"] > 0
    llm.shutdown()
