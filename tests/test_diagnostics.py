"""The maintained diagnostics run end to end on the CPU and keep their contracts: gates fail the exit status,
the GGUF inspection reads headers only, drift reports name the first layer over the threshold, the grid
interleaves its points."""
import json

import pytest
import torch

from litevllm_b200.diagnostics import gguf_inspect, layer_drift, perf_grid, smoke

CPU = ["--device", "cpu", "--dtype", "float32"]


def _json_line(capsys):
    return json.loads([l for l in capsys.readouterr().out.splitlines() if l.startswith("{")][-1])


def test_smoke_reports_steady_state_and_applies_gates(capsys, tmp_path):
    prof = tmp_path / "p.json"
    args = ["--model", "synthetic:tiny-llama-test", *CPU, "--prompt-length", "12", "--max-tokens", "10", "--batch", "2",
            "--repeat", "2", "--warmup-tokens", "2", "--profile-json", str(prof)]
    assert smoke.main(args) == 0
    res = _json_line(capsys)
    assert [r["cold"] for r in res["repeats"]] == [True, False]
    for r in res["repeats"]:
        assert r["generated_tokens"] == 20 and 0 < r["first_token_s"] <= r["total_s"]
        assert r["steady_tokens"] == 20 - 2 - 2 * 2          # minus the first tokens and two warm-up decode steps
        assert r["steady_decode_tps"] > 0
    assert res["failures"] == [] and res["expert_staging"] == {}
    saved = json.loads(prof.read_text())
    assert saved["result"]["steady_decode_tps"] == res["steady_decode_tps"] and "observer" in saved["engine"]
    assert smoke.main(args[:-2] + ["--min-steady-decode-tps", "1e12"]) == 1
    assert "steady decode" in _json_line(capsys)["failures"][0]
    with pytest.raises(SystemExit):
        smoke.main(args + ["--full-resident", "--staging-budget-gb", "1"])


def test_smoke_with_a_staging_budget_reports_the_slots(capsys, monkeypatch):
    monkeypatch.delenv("FI_EXPERT_STAGING_GB", raising=False)
    try:
        assert smoke.main(["--model", "synthetic:tiny-deepseek-test", *CPU, "--prompt-length", "16", "--max-tokens", "4",
                           "--repeat", "1", "--staging-budget-gb", "0.0005"]) == 0
    finally:
        monkeypatch.delenv("FI_EXPERT_STAGING_GB", raising=False)
    st = _json_line(capsys)["expert_staging"]
    assert st["blocks"] >= 1 and st["slots_per_block"] < st["experts_per_block"] and st["misses"] > 0


def test_gguf_inspection_reads_the_header(tmp_path, capsys):
    from litevllm_b200.loaders.gguf import GGUFTensor, write_gguf
    from litevllm_b200.ops import gguf_quant as gq
    E, I, H = 4, 64, 256
    experts = GGUFTensor(gq.quantize_q8_0(torch.randn(E * I, H)).view(E, I, -1), 8, (E, I, H))
    path = tmp_path / "x.gguf"
    write_gguf(path, {"general.architecture": "llama", "llama.block_count": 1},
               {"blk.0.ffn_gate_exps.weight": experts, "blk.0.ffn_up_exps.weight": experts,
                "blk.0.attn_norm.weight": torch.ones(H), "token_embd.weight": torch.zeros(8, H)})
    info = gguf_inspect.inspect(str(path), pattern=r"attn_norm")
    assert info["architecture"] == "llama" and info["tensors"] == 4 and info["layers"] == 1
    per = I * (H // 32) * 34
    assert [e["bytes_per_expert"] for e in info["expert_tensors"]] == [per, per]
    assert info["expert_bytes_per_slot_per_block"] == 2 * per and info["expert_bytes_total"] == 2 * per * E
    assert info["by_type"]["Q8_0"]["bits_per_weight"] == 8.5 and info["by_type"]["F32"]["tensors"] == 2
    assert [t["name"] for t in info["listed"]] == ["blk.0.attn_norm.weight"] and info["unsupported"] == []
    text = gguf_inspect.render(info, show_metadata=True)
    assert "Q8_0" in text and "routed experts" in text and "general.architecture" in text
    budget = 3.5 * 2 * per / 2 ** 30
    assert gguf_inspect.slots_for_budget(info, budget) == {"blocks": 1, "slots_per_block": 3, "experts_per_block": 4,
                                                           "resident_share": 0.75}
    assert gguf_inspect.slots_for_budget(info, 1.0)["slots_per_block"] == 4
    gguf_inspect.main([str(path), "--device-budget-gb", repr(budget)])
    assert "holds 3 of 4 experts in each of 1 blocks" in capsys.readouterr().out
    assert gguf_inspect.main([str(tmp_path / "missing.gguf")]) == 2
    assert "error" in capsys.readouterr().err


def test_layer_drift_names_the_first_layer_over_the_threshold(capsys):
    b = json.dumps({"device": "cpu", "dtype": "float32", "fastinference_config": {"kv_type": "turbo_int4"}})
    args = ["--model", "synthetic:tiny-llama-test", "--b", b, "--prompt-length", "20", "--decode-steps", "1", "--json"]
    assert layer_drift.main(args + ["--threshold", "1e-4"]) == 1
    rep = _json_line(capsys)
    assert rep["first_over_threshold"]["layer"] == "layers.0" and rep["first_over_threshold"]["step"] == 0
    assert len(rep["rows"]) == 2 * 2 and len({(r["step"], r["layer"]) for r in rep["rows"]}) == 4
    assert rep["rows"][0]["rel_l2"] != rep["rows"][1]["rel_l2"]          # rows are copies, not views of one stream
    assert all(0.9 < r["cosine"] <= 1.0 and r["finite"] for r in rep["rows"])
    same = json.dumps({"device": "cpu", "dtype": "float32"})
    assert layer_drift.main(args[:2] + ["--b", same, "--prompt-length", "20", "--decode-steps", "1", "--json"]) == 0
    rep = _json_line(capsys)
    assert rep["worst"]["rel_l2"] == 0.0 and rep["tokens_agree"] == 2 and rep["tokens_a"] == rep["tokens_b"]


def test_grid_points_and_engine_arguments():
    pts = perf_grid.grid(["max_num_seqs=2,4"], ["FASTINFERENCE_LITE_PREFILL_CHUNK=16,64"], [])
    assert len(pts) == 4 and pts[0]["set"] == {"max_num_seqs": 2} and pts[3]["tuning"] == {"FASTINFERENCE_LITE_PREFILL_CHUNK": "64"}
    assert perf_grid.grid([], [], [])[0]["label"] == "base"
    a = type("A", (), {"batch": 3, "prompt_length": 40, "max_tokens": 8})
    kw = perf_grid.engine_kwargs({"device": "cpu", "fastinference_config": {"kv_type": "fp8"}}, pts[3], a)
    assert kw["max_num_seqs"] == 4 and kw["max_model_len"] == 64
    assert kw["fastinference_config"] == {"kv_type": "fp8", "tuning_keyvals": {"FASTINFERENCE_LITE_PREFILL_CHUNK": "64"}}
    with pytest.raises(SystemExit):
        perf_grid.grid(["broken"], [], [])


def test_grid_runs_interleaved_rounds_in_process(capsys):
    assert perf_grid.main(["--model", "synthetic:tiny-llama-test", "--base", json.dumps({"device": "cpu", "dtype": "float32"}),
                           "--set", "max_num_seqs=1,3", "--batch", "3", "--prompt-length", "24", "--max-tokens", "6",
                           "--rounds", "2", "--warmup-rounds", "1", "--json"]) == 0
    rep = _json_line(capsys)
    assert rep["child_processes"] is False and [p["samples"] for p in rep["points"]] == [2, 2]
    assert rep["points"][0]["vs_first"] == 1.0 and rep["best"] in [p["label"] for p in rep["points"]]
    assert all(p["min_tps"] <= p["median_tps"] <= p["max_tps"] for p in rep["points"])


def test_grid_with_an_environment_axis_runs_child_processes(capsys):
    assert perf_grid.main(["--model", "synthetic:tiny-llama-test", "--base", json.dumps({"device": "cpu", "dtype": "float32"}),
                           "--env", "FI_BOUNDS_CHECK=0,1", "--batch", "2", "--prompt-length", "16", "--max-tokens", "4",
                           "--rounds", "1", "--warmup-rounds", "0", "--json"]) == 0
    rep = _json_line(capsys)
    assert rep["child_processes"] is True and [p["env"] for p in rep["points"]] == [{"FI_BOUNDS_CHECK": "0"}, {"FI_BOUNDS_CHECK": "1"}]
    assert all(p["median_tps"] > 0 for p in rep["points"])


def test_ngram_replay_counts_what_a_verify_step_would_accept():
    from litevllm_b200.diagnostics import speculative_ngram as sn
    prompt = [1, 2, 3, 4, 5, 6]
    assert sn.propose(prompt + [9, 1, 2], 3, 3) == [3, 4, 5]            # suffix (1, 2) seen in the prompt
    assert sn.propose(prompt + [9], 1, 3) == []                          # too little output for a 2-gram
    assert sn.propose([7, 8, 9, 7, 8], 2, 4) == [9, 7, 8]               # most recent earlier occurrence
    rep = sn.replay(prompt, [1, 2, 3, 4, 5, 6, 1, 2], k=3)
    # steps: 1 | 2 | (draft 3 4 5: all accepted) 3 4 5 6 | (draft 1 2 3: 2 accepted, then the output ends) 1 2
    assert rep == {"tokens": 8, "verify_steps": 4, "steps_with_draft": 2, "proposed": 6, "accepted": 5}
    assert sn.replay(prompt, [], 3)["verify_steps"] == 0
    noisy = sn.replay([1, 2, 3], [9, 8, 7, 6, 5], 3)
    assert noisy["accepted"] == 0 and noisy["verify_steps"] == 5
    s = sn.summarise([rep, noisy], verify_cost=1.5)
    assert s["tokens"] == 13 and s["tokens_per_step"] == round(13 / 9, 4) and s["acceptance"] == round(5 / 6, 4)
    assert s["projected_speedup"] == round(13 / (7 + 1.5 * 2), 4)


def test_ngram_tool_runs_on_a_model(capsys):
    from litevllm_b200.diagnostics import speculative_ngram as sn
    assert sn.main(["--model", "synthetic:tiny-llama-test", "--engine", json.dumps({"device": "cpu", "dtype": "float32",
                    "max_model_len": 128}), "--max-tokens", "24", "-k", "3"]) == 0
    rep = _json_line(capsys)
    assert rep["tokens"] == sum(p["tokens"] for p in rep["per_prompt"]) and rep["tokens"] > 0
    assert 1.0 <= rep["tokens_per_step"] <= 4.0 and 0.0 <= rep["acceptance"] <= 1.0


def test_quality_cases_are_judged_by_their_expectations(tmp_path, capsys):
    from litevllm_b200.diagnostics import quality_spotcheck as qs
    ok = qs.judge_case({"expect_any": ["Paris", "Lyon"], "expect_all": ["france"], "expect_regex": r"capital\s+of",
                        "forbid": ["berlin"]}, "The capital of France is paris.", [1, 2, 3], "stop")
    assert ok == []
    why = qs.judge_case({"expect_any": ["Paris"], "forbid": ["the"]}, "The answer", [1, 2], "abort")
    assert len(why) == 3 and any("finish reason" in w for w in why)
    assert qs.judge_case({}, "", [], "stop") == ["empty answer"]
    assert any("degenerate" in w for w in qs.judge_case({}, "x" * 20, [5] * 15 + [6] * 5, "length"))
    assert qs.judge_case({}, "fine", list(range(20)), "length") == []
    fixtures = tmp_path / "cases.json"
    fixtures.write_text(json.dumps([
        {"name": "anything", "prompt_token_ids": [5, 6, 7, 8], "max_tokens": 6, "expect_regex": "."},
        {"name": "impossible", "prompt_token_ids": [9, 10, 11], "max_tokens": 6, "expect_all": ["no such text ☃"]}]))
    args = ["--model", "synthetic:tiny-llama-test", "--fixtures", str(fixtures),
            "--engine", json.dumps({"device": "cpu", "dtype": "float32", "max_model_len": 64})]
    assert qs.main(args) == 1
    rep = _json_line(capsys)
    assert rep["pass_rate"] == 0.5 and [r["passed"] for r in rep["results"]] == [True, False]
    assert qs.main(args + ["--min-pass-rate", "0.5"]) == 0
    empty = tmp_path / "empty.json"
    empty.write_text("[]")
    assert qs.main(["--model", "synthetic:tiny-llama-test", "--fixtures", str(empty)]) == 2
