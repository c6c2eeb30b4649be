"""End-to-end engine runs on the GPU checked against the CPU fp32 oracle of the same weights."""
import pytest
import torch

from litevllm_b200 import LLM, SamplingParams, ops

pytestmark = pytest.mark.gpu


def _prompts(vocab, lens, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]


def _agreement(a, b):
    same = sum(int(x == y) for x, y in zip(a, b))
    return same / max(len(a), 1)


@pytest.mark.parametrize("graph", [True, False])
def test_tiny_llama_matches_cpu_oracle(graph):
    lens = (5, 33, 17, 64, 100, 1)
    kw = dict(max_num_seqs=8, max_model_len=256)
    cfg = {"tuning_keyvals": {"FASTINFERENCE_CUDA_GRAPH_DECODE": "1" if graph else "0"}}
    gpu = LLM("synthetic:tiny-llama-test", dtype="bfloat16", device="cuda:0", fastinference_config=cfg, **kw)
    cpu = LLM("synthetic:tiny-llama-test", dtype="float32", device="cpu", **kw)
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    prompts = _prompts(512, lens)
    og = gpu.generate(prompts, sp)
    oc = cpu.generate(prompts, sp)
    ops.check_status(torch.device("cuda:0"))
    # bf16 vs fp32 may flip near-ties; the first token and most of the rest must agree
    first = [a.outputs[0].token_ids[0] == b.outputs[0].token_ids[0] for a, b in zip(og, oc)]
    assert sum(first) >= len(lens) - 1, first
    agree = [_agreement(a.outputs[0].token_ids, b.outputs[0].token_ids) for a, b in zip(og, oc)]
    assert sum(agree) / len(agree) > 0.6, agree
    if graph:
        assert gpu.engine.decode_executor.graph_replays > 0


def test_logits_close_to_oracle():
    """Prefill logits of the GPU model vs the CPU fp32 model on identical weights."""
    kw = dict(max_num_seqs=4, max_model_len=128)
    gpu = LLM("synthetic:tiny-llama-test", dtype="bfloat16", device="cuda:0", **kw)
    cpu = LLM("synthetic:tiny-llama-test", dtype="float32", device="cpu", **kw)
    outs = {}
    for name, llm in (("gpu", gpu), ("cpu", cpu)):
        eng = llm.engine
        eng._build_lazy()
        for i, p in enumerate(_prompts(512, (40, 7, 64))):
            eng.add_request(f"r{i}", p, SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
        plan = eng.step_scheduler.build_plan(eng.scheduler)
        eng.controller._admit(plan)
        eng.backend.ensure_kv_blocks(plan)
        res = eng.prefill_executor.execute(plan.prefills, eng.scheduler.requests)
        outs[name] = res.logits.float().cpu()
    cos = torch.nn.functional.cosine_similarity(outs["gpu"], outs["cpu"], dim=-1)
    assert float(cos.min()) > 0.995, cos


def test_chunked_prefill_equals_single_shot():
    """A prompt processed in 3 chunks must give the same tokens as one chunk."""
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    p = _prompts(512, (150,), seed=3)
    a = LLM("synthetic:tiny-llama-test", dtype="bfloat16", device="cuda:0", max_num_seqs=2, max_model_len=256)
    cfg = {"tuning_keyvals": {"FASTINFERENCE_LITE_PREFILL_CHUNK": "64", "FASTINFERENCE_MIN_PREFILL_CHUNK": "16"}}
    b = LLM("synthetic:tiny-llama-test", dtype="bfloat16", device="cuda:0", max_num_seqs=2, max_model_len=256,
            fastinference_config=cfg)
    ta = a.generate(p, sp)[0].outputs[0].token_ids
    tb = b.generate(p, sp)[0].outputs[0].token_ids
    assert ta[0] == tb[0]
    assert _agreement(ta, tb) >= 0.5


def test_sampling_with_seed_is_reproducible():
    llm = LLM("synthetic:tiny-llama-test", dtype="bfloat16", device="cuda:0", max_num_seqs=4, max_model_len=128)
    sp = SamplingParams(temperature=0.8, top_k=20, top_p=0.9, max_tokens=8, seed=123, ignore_eos=True,
                        repetition_penalty=1.1, presence_penalty=0.1)
    p = _prompts(512, (9, 21))
    a = [o.outputs[0].token_ids for o in llm.generate(p, sp)]
    b = [o.outputs[0].token_ids for o in llm.generate(p, sp)]
    assert a == b


def _prefill_logits(llm, prompts):
    eng = llm.engine
    eng._build_lazy()
    for i, p in enumerate(prompts):
        eng.add_request(f"lg{i}", p, SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
    plan = eng.step_scheduler.build_plan(eng.scheduler)
    eng.controller._admit(plan)
    eng.backend.ensure_kv_blocks(plan)
    with torch.inference_mode():
        res = eng.prefill_executor.execute(plan.prefills, eng.scheduler.requests)
    return res.logits.float().cpu()


@pytest.mark.parametrize("preset,min_cos", [("tiny-gemma4-moe-test", 0.96), ("tiny-llama-awq-test", 0.99),
                                             ("tiny-llama-ct-test", 0.99), ("tiny-deepseek-test", 0.97),
                                             ("tiny-qwen35-test", 0.97), ("tiny-qwen35-moe-test", 0.95), ("tiny-qwen2vl-test", 0.99), ("tiny-qwen3-test", 0.99)])
def test_quantised_models_match_cpu_oracle(preset, min_cos):
    """int4 weights (+ fp8 KV, MoE routing for Gemma4): GPU kernels vs the CPU fp32 path on the same
    synthetic checkpoint."""
    kw = dict(max_num_seqs=4, max_model_len=128)
    prompts = _prompts(512, (40, 7, 64))
    gpu = LLM(f"synthetic:{preset}", dtype="bfloat16", device="cuda:0", **kw)
    cpu = LLM(f"synthetic:{preset}", dtype="float32", device="cpu", **kw)
    a, b = _prefill_logits(gpu, prompts), _prefill_logits(cpu, prompts)
    cos = torch.nn.functional.cosine_similarity(a, b, dim=-1)
    assert float(cos.min()) > min_cos, cos
    outs = gpu.generate(_prompts(512, (9, 33)), SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    assert all(len(o.outputs[0].token_ids) == 8 for o in outs)
    ops.check_status(torch.device("cuda:0"))


def test_int4_repack_cache_round_trip(tmp_path, monkeypatch):
    """An AWQ checkpoint directory loaded twice with FASTINFERENCE_REPACK_CACHE_DIR set: the first start
    writes the repacked layouts, the second attaches them (no packed tensor is read) and generates the same
    tokens; a touched checkpoint file changes the fingerprint and the cache is not used."""
    import json
    import os

    from safetensors.torch import save_file

    from litevllm_b200 import LLM, SamplingParams
    from litevllm_b200.loaders import repack_cache, synth
    from litevllm_b200.models.arch import arch_from_hf_config
    from litevllm_b200.models.presets import get_preset
    preset = get_preset("tiny-llama-awq-test")
    ckpt = tmp_path / "ckpt"
    ckpt.mkdir()
    (ckpt / "config.json").write_text(json.dumps(preset))
    arch = arch_from_hf_config(preset)
    tensors = {n: t.contiguous().cpu() for n, t in synth.iter_llama_weights(arch, 0, torch.float32, "cpu")}
    save_file(tensors, str(ckpt / "model.safetensors"))
    monkeypatch.setenv("FASTINFERENCE_REPACK_CACHE_DIR", str(tmp_path / "cache"))
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    prompts = [[3, 9, 27, 81], [5, 6, 7]]

    def run():
        llm = LLM(str(ckpt), dtype="bfloat16", device="cuda:0", max_num_seqs=2, max_model_len=64)
        cached = [getattr(m, "_repack_cached", False) for m in llm.engine.model.modules() if hasattr(m, "int4")]
        toks = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        llm.shutdown()
        return toks, cached

    first, cached1 = run()
    files = list((tmp_path / "cache").glob("*.pt"))
    assert len(files) == 1 and not any(cached1)
    second, cached2 = run()
    assert cached2 and all(cached2) and second == first
    st = os.stat(ckpt / "model.safetensors")
    os.utime(ckpt / "model.safetensors", ns=(st.st_atime_ns, st.st_mtime_ns + 10 ** 9))
    assert repack_cache.fingerprint(ckpt) not in files[0].name
    third, cached3 = run()
    assert not any(cached3) and third == first


def test_mla_absorbed_matches_materialised():
    """Multi-head latent attention: the absorbed form (one 576-value cache row per token, attention in latent
    space, per-head projections before and after) against the materialised per-head K/V form on the same GPU
    and weights: prefill logits of prompts spanning several 64-row chunks, and decode steps after them."""
    import litevllm_b200.models.deepseek_mla as dm
    kw = dict(max_num_seqs=4, max_model_len=320)
    prompts = _prompts(512, (200, 7, 130))
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    res = {}
    saved = dm._ABSORBED
    try:
        for mode in (True, False):
            dm._ABSORBED = mode
            llm = LLM("synthetic:tiny-deepseek-mla512-test", dtype="bfloat16", device="cuda:0", **kw)
            assert llm.engine.model.layers[0].self_attn.absorbed == mode
            width = llm.engine.kv_cache.layers[0][0].shape[-1]
            assert width == (576 if mode else 256)
            logits = _prefill_logits(llm, prompts)
            toks = [o.outputs[0].token_ids for o in llm.generate(_prompts(512, (150, 20)), sp)]
            res[mode] = (logits, toks)
            llm.shutdown()
    finally:
        dm._ABSORBED = saved
    ops.check_status(torch.device("cuda:0"))
    cos = torch.nn.functional.cosine_similarity(res[True][0], res[False][0], dim=-1)
    assert float(cos.min()) > 0.995, cos
    assert all(len(t) == 12 for t in res[True][1])          # (random-init logits are too flat to compare tokens)
