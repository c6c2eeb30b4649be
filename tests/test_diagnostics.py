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
