"""DeepSeek-V4-Flash through the engine: the model owns its per-request rows and returns token ids; the
adapter swaps the executors, caps admission and narrows requests to greedy decoding.
Reference behaviour: vllm/model_executor/models/deepseek_v4_flash/model.py (prefill_request /
decode_tokens_batch), vllm/adapters/deepseek_v4_flash.py."""
import pytest
import torch

from litevllm_b200 import LLM, SamplingParams
from litevllm_b200.engine.errors import InvalidRequestError

PRESET = "synthetic:tiny-deepseek-v4-flash-test"
PROMPTS = [[(7 * i + 3) % 500 + 2 for i in range(30)], [(11 * i + 5) % 500 + 2 for i in range(21)]]


def _greedy(n):
    return SamplingParams(max_tokens=n, temperature=0.0, ignore_eos=True)


@pytest.fixture(scope="module")
def llm():
    return LLM(PRESET, device="cpu", max_model_len=128, dtype="float32")


def _tokens(llm, prompts, n):
    return [list(o.outputs[0].token_ids) for o in llm.generate([{"prompt_token_ids": p} for p in prompts], _greedy(n))]


def test_adapter_and_executors_selected(llm):
    from litevllm_b200.adapters.deepseek_v4_flash import DeepSeekV4FlashAdapter
    from litevllm_b200.models.deepseek_v4_flash.executors import V4FlashDecodeExecutor, V4FlashPrefillExecutor
    eng = llm.engine
    assert isinstance(eng.adapter, DeepSeekV4FlashAdapter)
    assert isinstance(eng.backend.prefill_executor, V4FlashPrefillExecutor)
    assert isinstance(eng.backend.decode_executor, V4FlashDecodeExecutor)
    assert eng.model_policy.admission_cap >= 1
    assert not eng.capabilities.supports_sampling and not eng.capabilities.supports_lora


def test_decode_continues_like_a_longer_prefill(llm):
    """Tokens 7..12 of a generation equal the first 6 tokens generated from prompt + tokens 1..6: the rows a
    decode step appends (window ring, compressor state, emitted rows, indexer rows) are the rows a prefill of
    the longer prompt builds."""
    first = _tokens(llm, PROMPTS[:1], 12)[0]
    again = _tokens(llm, [PROMPTS[0] + first[:6]], 6)[0]
    assert again == first[6:]
    assert len(set(first)) > 4                       # not a degenerate repetition


def test_batched_decode_equals_single_requests(llm):
    together = _tokens(llm, PROMPTS, 10)
    alone = [_tokens(llm, [p], 10)[0] for p in PROMPTS]
    assert together == alone


def test_chunked_prefill_equals_one_chunk(llm):
    model = llm.engine.model
    one = model.prefill_request("a", PROMPTS[0], 0, True)
    assert model.prefill_request("b", PROMPTS[0][:13], 0, False) is None
    two = model.prefill_request("b", PROMPTS[0][13:], 13, True)
    assert one == two
    ra, rb = model.requests["a"], model.requests["b"]
    assert (ra.layers[0].pool - rb.layers[0].pool).abs().gt(1e-4).float().mean() < 0.002
    assert ra.pos == rb.pos == len(PROMPTS[0])
    for la, lb in zip(ra.layers, rb.layers):
        # the fp8 round trip may flip a rounding step where the two GEMM shapes differ in the last bit, and a
        # flipped step moves the later layers by a little
        assert (la.pool[: la.window] - lb.pool[: lb.window]).abs().mean() < 5e-3
        assert la.n_comp == lb.n_comp
    # compressed layers emitted one row per `ratio` tokens, more than the indexer keeps
    cfg = model.cfg
    assert cfg.ratios == (0, 0, 4, 8)
    assert ra.layers[2].n_comp == len(ra.layers[2].index_rows) == len(PROMPTS[0]) // 4 > cfg.indexer_topk
    assert ra.layers[3].n_comp == len(PROMPTS[0]) // 8 and ra.layers[3].index_pool is None
    assert ra.layers[0].n_comp == ra.layers[1].n_comp == 0
    with pytest.raises(RuntimeError):
        model.prefill_request("b", [5, 6], 3, True)   # a chunk that does not continue where the rows end
    assert model.release_request("a") and model.release_request("b") and not model.release_request("a")


def test_rows_are_released_with_the_request(llm):
    model = llm.engine.model
    _tokens(llm, PROMPTS, 3)
    assert model.requests == {} and model.request_bytes() == 0


def test_requests_are_narrowed_to_greedy(llm):
    with pytest.raises(InvalidRequestError):
        llm.generate([{"prompt_token_ids": PROMPTS[1]}], SamplingParams(max_tokens=2, temperature=0.8))
    assert llm.engine.model.requests == {}


def test_admission_cap_follows_the_row_budget(monkeypatch):
    from litevllm_b200.adapters.deepseek_v4_flash import DeepSeekV4FlashAdapter, _row_bytes_per_request
    from litevllm_b200.models.arch import arch_from_hf_config
    from litevllm_b200.models.presets import PRESETS
    arch = arch_from_hf_config(PRESETS["tiny-deepseek-v4-flash-test"])
    assert arch.family == "deepseek_v4_flash"
    per = _row_bytes_per_request(arch.extra["v4_rows"], 512)
    monkeypatch.setenv("FI_V4_ROWS_BUDGET_GB", str(3.5 * per / 2 ** 30))

    class RC:
        max_model_len = 512
    assert DeepSeekV4FlashAdapter(arch).runtime_policy(RC()).admission_cap == 3


def _prefill_logits(model, prompt):
    rows = model._new_request(model.embed.device)
    hidden = model.forward_tokens([(rows, t) for t in prompt])[-1]
    w = model.lm_head.dense() if hasattr(model.lm_head, "dense") else model.lm_head
    return hidden.float().cpu(), (w.float() @ hidden.float()).cpu()


@pytest.mark.gpu
def test_gpu_tokens_match_cpu(llm):
    """fp32 on both sides: the GPU side runs the native shared-latent attention, indexer, QAT and fused token
    kernels.  Random weights leave some first tokens on a knife edge (a rounding step of the fp8 round trip or a
    routing tie flips them), so the token comparison uses the prompts whose CPU logits have the clearest winner,
    and every prompt's final hidden vector has to point the same way."""
    gpu = LLM(PRESET, device="cuda", max_model_len=128, dtype="float32")
    g = torch.Generator().manual_seed(3)
    cands = [torch.randint(2, 500, (int(n),), generator=g).tolist() for n in (30, 21, 26, 17, 33, 24)]
    cpu_m, gpu_m = llm.engine.model, gpu.engine.model
    margins, cosines = [], []
    for p in cands:
        h_c, l_c = _prefill_logits(cpu_m, p)
        h_g, l_g = _prefill_logits(gpu_m, p)
        top = torch.topk(l_c, 2).values
        margins.append(float(top[0] - top[1]))
        cosines.append(float(torch.nn.functional.cosine_similarity(h_c, h_g, dim=0)))
    assert sorted(cosines)[len(cosines) // 2] > 0.98 and min(cosines) > 0.8, cosines
    best = sorted(range(len(cands)), key=lambda i: -margins[i])[:2]
    prompts = [cands[i] for i in best]
    want, got = _tokens(llm, prompts, 8), _tokens(gpu, prompts, 8)
    assert [w[0] for w in want] == [x[0] for x in got], (want, got, margins)

    def common_prefix(a, b):
        n = 0
        while n < len(a) and a[n] == b[n]:
            n += 1
        return n

    # once one token differs everything after it differs: count how far the two sides walk together
    assert all(common_prefix(w, x) >= 2 for w, x in zip(want, got)), (want, got)
    # the decode batch (one launch per step for all requests) against each request decoded alone
    alone = [_tokens(gpu, [p], 8)[0] for p in prompts]
    assert all(common_prefix(w, x) >= 3 for w, x in zip(alone, got)), (alone, got)
    assert gpu.engine.model.requests == {}


def test_checkpoint_tensor_names_map_to_parameters(llm):
    """GGUF names of the checkpoint family land in the matching parameters, with layout adaptation."""
    model = llm.engine.model
    cls = type(model)
    assert cls.param_name("blk.2.indexer.attn_q_b.weight") == "layers.2.idx_q"
    assert cls.param_name("blk.3.attn_compressor_ape.weight") == "layers.3.comp_ape"
    assert cls.param_name("output_hc_fn.weight") == "out_hc_fn"
    names = {n for n, _ in model.named_parameters()} | {n for n, _ in model.named_buffers() if "inv_freq" not in n}
    every = [f"blk.{i}.{s}" for i in range(model.cfg.layers) for s in cls._GGUF_LAYER] + list(cls._GGUF_TOP)
    mapped = {cls.param_name(n) for n in every}
    assert names <= mapped                                   # every parameter has a checkpoint name
    keep = model.layers[3].comp_ape.clone()
    try:
        new = torch.arange(keep.numel(), dtype=torch.float32).reshape(keep.shape)
        consumed = model.load_weights([("blk.3.attn_compressor_ape.weight", new.t().contiguous()),
                                       ("blk.9.unknown.weight", torch.zeros(1))], strict=False)
        assert consumed == {"blk.3.attn_compressor_ape.weight"}
        torch.testing.assert_close(model.layers[3].comp_ape.float(), new)
        with pytest.raises(ValueError):
            model.load_weights([("output_norm.weight", torch.zeros(3))], strict=False)
        with pytest.raises(ValueError, match="unbound"):       # a checkpoint delivers every tensor or none
            model.load_weights([("blk.3.attn_compressor_ape.weight", new)])
    finally:
        model.layers[3].comp_ape.data.copy_(keep)


def _write_v4_gguf(src, path, two_bit_experts: bool = False):
    """The synthetic model as a `deepseek4` GGUF file: projections as Q8_0 blocks, routed experts as Q8_0 blocks
    of the model's weights or as random IQ2_XXS (gate, up) / Q2_K (down) blocks, the rest F32."""
    from litevllm_b200.loaders.gguf import GGUFTensor, write_gguf
    from litevllm_b200.ops import gguf_quant as gq
    c = src.cfg
    cls = type(src)
    back = {v: k for k, v in cls._GGUF_TOP.items()}
    layer_back = {v: k for k, v in cls._GGUF_LAYER.items()}

    def q8(t):
        rows = t.float().reshape(-1, t.shape[-1])
        return GGUFTensor(gq.quantize_q8_0(rows).view(*t.shape[:-1], -1), 8, tuple(t.shape))

    tensors = {}
    named = dict(src.named_parameters())
    named.update({n: b for n, b in src.named_buffers() if "inv_freq" not in n})
    for name, p in named.items():
        if name.startswith("layers."):
            _, idx, attr = name.split(".", 2)
            gname = f"blk.{idx}.{layer_back[attr]}"
        else:
            idx, attr, gname = "0", name, back[name]
        t = p.detach().cpu()
        if two_bit_experts and attr in ("w_gate", "w_up", "w_down"):
            ty = 10 if attr == "w_down" else 16
            E, R, K = t.shape
            raw = gq.random_blocks(ty, E * R, K, seed=17 * int(idx) + len(attr), scale=0.05)
            tensors[gname] = GGUFTensor(raw.view(E, R, -1), ty, (E, R, K))
        elif attr in ("w_gate", "w_up", "w_down", "q_b", "s_gate", "s_up", "s_down", "lm_head"):
            tensors[gname] = q8(t)
        elif attr == "o_a":
            tensors[gname] = t.float().reshape(-1, t.shape[-1]).contiguous()       # groups flattened, as on disk
        elif attr == "hash_table":
            tensors[gname] = t.to(torch.int32).t().contiguous()                    # [vocab, top_k]
        else:
            tensors[gname] = t.float().contiguous()
    meta = {"general.architecture": "deepseek4", "deepseek4.block_count": c.layers,
            "deepseek4.embedding_length": c.hidden, "deepseek4.attention.head_count": c.heads,
            "deepseek4.attention.head_count_kv": 1, "deepseek4.attention.key_length": c.head_dim,
            "deepseek4.attention.sliding_window": c.window, "deepseek4.attention.indexer.head_count": c.indexer_heads,
            "deepseek4.attention.indexer.key_length": 128, "deepseek4.attention.indexer.top_k": c.indexer_topk,
            "deepseek4.expert_count": c.experts, "deepseek4.expert_used_count": c.top_k,
            "deepseek4.vocab_size": c.vocab, "deepseek4.context_length": 512,
            "deepseek4.attention.compress_ratio_coarse": 8, "deepseek4.swiglu_clamp": 0.0,
            "deepseek4.attention.layer_norm_rms_epsilon": 1e-6}
    write_gguf(path, meta, tensors)


def test_gguf_checkpoint_round_trip(llm, tmp_path):
    """A `deepseek4` GGUF file written from the synthetic model loads through the ordinary entry point: geometry
    from metadata and tensor shapes, block tensors kept in block format, and the same first token as the
    source model."""
    from litevllm_b200.loaders.gguf import hf_config_from_gguf
    from litevllm_b200.models.deepseek_v4_flash.model import BlockMatrix
    src = llm.engine.model
    c = src.cfg
    path = tmp_path / "tiny-v4.gguf"
    _write_v4_gguf(src, path)
    hf = hf_config_from_gguf(path)
    assert hf["architectures"] == ["DeepseekV4FlashForCausalLM"]
    assert (hf["q_lora_rank"], hf["o_groups"], hf["o_lora_rank"], hf["hc_mult"]) == (c.q_lora, c.o_groups, c.o_lora, c.hc)
    assert (hf["moe_intermediate_size"], hf["num_hash_layers"], hf["index_topk"]) == (c.expert_inter, c.hash_layers, c.indexer_topk)
    loaded = LLM(str(path), device="cpu", max_model_len=128, dtype="float32")
    m = loaded.engine.model
    assert m.cfg.ratios == c.ratios
    assert isinstance(m.layers[0].q_b, BlockMatrix) and isinstance(m.lm_head, BlockMatrix)
    assert m.layers[2].routed is not None and m.layers[2].w_gate is None
    torch.testing.assert_close(m.layers[1].o_a.float(), src.layers[1].o_a.float())
    assert torch.equal(m.layers[0].hash_table, src.layers[0].hash_table)
    torch.testing.assert_close(m.layers[3].comp_ape.float(), src.layers[3].comp_ape.float())
    want = _tokens(llm, PROMPTS[:1], 4)[0]
    got = _tokens(loaded, PROMPTS[:1], 10)
    assert got[0][0] == want[0]
    # the loaded model is consistent with itself: decode continues like a longer prefill
    assert _tokens(loaded, [PROMPTS[0] + got[0][:5]], 5)[0] == got[0][5:]


@pytest.mark.gpu
def test_gguf_checkpoint_on_gpu_matches_cpu(llm, tmp_path, monkeypatch):
    """The checkpoint formats of the full-size model (Q8_0 projections, IQ2_XXS / Q2_K routed experts) stay in
    block format on the GPU and run through the GGUF GEMV and expert kernels; tokens follow the CPU model that
    dequantises the same file."""
    path = tmp_path / "tiny-v4-2bit.gguf"
    _write_v4_gguf(llm.engine.model, path, two_bit_experts=True)
    cpu = LLM(str(path), device="cpu", max_model_len=128, dtype="float32")
    gpu = LLM(str(path), device="cuda", max_model_len=128, dtype="bfloat16")
    assert gpu.engine.model.layers[2].routed.types == {"gate": 16, "up": 16, "down": 10}
    want, got = _tokens(cpu, PROMPTS, 6), _tokens(gpu, PROMPTS, 6)
    agree = sum(a == b for w, g in zip(want, got) for a, b in zip(w, g)) / sum(len(w) for w in want)
    assert got[0][0] == want[0][0] and agree >= 0.3, (want, got)
    # decode steps replay CUDA graphs of their static stretches; the same steps launched one by one walk the same way
    from litevllm_b200.models.deepseek_v4_flash import model as v4_model
    assert gpu.engine.model._dgraphs, "the decode graphs were not used"
    monkeypatch.setattr(v4_model, "_DECODE_GRAPHS", False)
    eager = _tokens(gpu, PROMPTS, 6)
    assert all(a[:3] == b[:3] for a, b in zip(eager, got)), (eager, got)


@pytest.mark.gpu
def test_fused_token_kernels_match_their_pytorch_forms():
    """Every fused per-token kernel against the PyTorch formulation it replaces (fp32 on the CPU)."""
    from litevllm_b200.models.deepseek_v4_flash import native as nv
    from litevllm_b200.models.deepseek_v4_flash.attention import CompressorState
    from litevllm_b200.models.deepseek_v4_flash.model import V4Config
    from litevllm_b200.models.presets import PRESETS
    g = torch.Generator().manual_seed(11)
    T, hc, H = 5, 4, 512
    n_mix = 2 * hc + hc * hc

    def both(fn, *args):
        cpu = fn(*args)
        gpu = fn(*[a.cuda() if isinstance(a, torch.Tensor) else a for a in args])
        return cpu, gpu

    def close(a, b, tol=2e-4, what=""):
        torch.testing.assert_close(b.cpu(), a, rtol=tol, atol=tol, msg=lambda m: f"{what}: {m}")

    streams = torch.randn(T, hc, H, generator=g)
    fn_w = torch.randn(hc * H, n_mix, generator=g) / 30
    base, scale = torch.randn(n_mix, generator=g) * 0.3, torch.tensor([0.7, 1.3, 0.9])
    s_cpu, s_gpu = both(lambda *a: nv.hc_pre(*a, 1e-6), streams, fn_w, base, scale)
    close(s_cpu.mixed, s_gpu.mixed, what="hc_pre mixed")
    close(s_cpu.post, s_gpu.post, what="hc_pre post")
    close(s_cpu.combine, s_gpu.combine, what="hc_pre combine")
    assert (s_gpu.combine.sum(-1) - 1).abs().max() < 1e-3 and (s_gpu.combine.sum(-2) - 1).abs().max() < 1e-3
    out = torch.randn(T, H, generator=g)
    n_cpu = nv.hc_post(out, streams, s_cpu)
    n_gpu = nv.hc_post(out.cuda(), streams.cuda(), s_gpu)
    close(n_cpu, n_gpu, what="hc_post")
    ofn, obase, oscale = torch.randn(hc, hc * H, generator=g) / 30, torch.randn(hc, generator=g), torch.tensor([0.8])
    c_cpu, c_gpu = both(lambda *a: nv.hc_collapse(*a, 1e-6), streams, ofn, obase, oscale)
    close(c_cpu, c_gpu, what="hc_collapse")

    cfg = V4Config.from_hf(PRESETS["tiny-deepseek-v4-flash-test"])
    pos = torch.tensor([0, 3, 17, 200, 4001])
    for compressed in (False, True):
        freq = cfg.rope_inv_freq(compressed)
        x = torch.randn(T, 3, 512, generator=g) * 2
        w = torch.rand(512, generator=g) + 0.5
        for kw in (dict(norm=True), dict(norm=False, inverse=True), dict(norm=True, fp8=True)):
            wt = None if kw.get("inverse") else w
            a, b = both(lambda xx, ww, ff, pp: nv.norm_rope(xx, ww, ff, pp, 1e-6, **kw), x, wt, freq, pos)
            if kw.get("fp8"):       # a rounding step may flip where the two sides differ in the last bit
                assert ((a - b.cpu()).abs() > 1e-3 * a.abs().clamp_min(1e-2)).float().mean() < 0.002
            else:
                close(a, b, tol=2e-3, what=f"norm_rope {kw} compressed={compressed}")   # fp32 angles on the CPU side
    a, b = both(lambda xx, ww: nv.norm_rope(xx, ww, None, None, 1e-6), torch.randn(7, 256, generator=g), torch.rand(256, generator=g))
    close(a, b, what="plain norm")

    for ratio, D in ((4, 512), (8, 512), (4, 128)):
        width = (2 if ratio == 4 else 1) * D
        ape = torch.randn(ratio, width, generator=g)
        st_c, st_g = CompressorState.empty(D, ratio, "cpu"), CompressorState.empty(D, ratio, "cuda")
        for tok in range(3 * ratio + 1):
            kv, sc = torch.randn(width, generator=g), torch.randn(width, generator=g)
            e_c = nv.compressor_step_(st_c, kv, sc, ape, tok, D, ratio)
            e_g = nv.compressor_step_(st_g, kv.cuda(), sc.cuda(), ape.cuda(), tok, D, ratio)
            assert (e_c is None) == (e_g is None) == ((tok + 1) % ratio != 0)
            if e_c is not None:
                close(e_c, e_g, what=f"compressor ratio {ratio} token {tok}")
        close(st_c.kv, st_g.kv, what="compressor state")

    x = torch.randn(6, 512, generator=g)
    x[2, :256] = 0
    a, b = both(nv.q8k, x)
    close(a, b, tol=1e-6, what="q8k")

    # a run of tokens in one launch: window spans of a linear buffer plus a prefix / a selection of compressed rows
    from litevllm_b200.models.deepseek_v4_flash.attention import shared_kv_attention_run
    n, heads, D = 9, 3, 256
    q = torch.randn(n, heads, D, generator=g)
    lin, comp = torch.randn(14, D, generator=g), torch.randn(12, D, generator=g)
    sinks = torch.randn(heads, generator=g)
    a0 = [max(0, j + 6 - 8) for j in range(n)]
    na = [j + 6 - s0 for j, s0 in enumerate(a0)]
    nb = [min(12, 3 + j) for j in range(n)]
    spans = torch.tensor([a0, na, nb], dtype=torch.int32)
    a, b = both(lambda *t: shared_kv_attention_run(t[0], t[1], t[2], t[3], None, t[4], 0.07), q, lin, comp, spans, sinks)
    close(a, b, what="attention run, prefix rows")
    sel = torch.stack([torch.randperm(12, generator=g)[:5] for _ in range(n)]).to(torch.int32)
    spans[2] = torch.tensor([min(5, v) for v in nb], dtype=torch.int32)
    a, b = both(lambda *t: shared_kv_attention_run(t[0], t[1], t[2], t[3], t[4], t[5], 0.07), q, lin, comp, spans, sel, sinks)
    close(a, b, what="attention run, selected rows")


def test_abort_releases_the_rows(llm):
    eng = llm.engine
    eng.add_request("abort-me", {"prompt_token_ids": PROMPTS[0]}, _greedy(50))
    for _ in range(3):
        eng.step()
    assert "abort-me" in eng.model.requests and eng.model.request_bytes() > 0
    assert eng.abort_request("abort-me")
    assert eng.model.requests == {}
    assert not eng.has_unfinished_requests()


def test_served_over_http_greedy_only():
    """The OpenAI server in front of the model-owned data plane: greedy chat completions stream and finish, a
    sampling temperature is refused with 400, and the rows are gone afterwards."""
    import json
    from fastapi.testclient import TestClient
    from litevllm_b200.entrypoints.openai import api_server as srv
    client = TestClient(srv.app)
    saved = (srv.engine, srv.served_model, srv.debug_endpoints_enabled)
    try:
        srv.engine = srv.build_engine(PRESET, dtype="float32", device="cpu", max_num_seqs=2, max_model_len=128)
        srv.served_model, srv.debug_endpoints_enabled = "v4", False
        body = {"model": "v4", "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 5, "temperature": 0}
        r = client.post("/v1/chat/completions", json=body)
        assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] == 5
        assert client.post("/v1/chat/completions", json=dict(body, temperature=0.7)).status_code == 400
        with client.stream("POST", "/v1/chat/completions", json=dict(body, stream=True)) as s:
            lines = [l for l in s.iter_lines() if l.startswith("data:")]
        assert lines[-1] == "data: [DONE]" and len(lines) >= 3
        assert json.loads(lines[0][5:])["choices"][0]["delta"] == {"role": "assistant"}
        assert srv.engine.engine.model.requests == {}
    finally:
        if srv.engine is not None:
            srv.engine.shutdown()
        srv.engine, srv.served_model, srv.debug_endpoints_enabled = saved


def test_deepseek4_files_are_validated(tmp_path):
    from litevllm_b200.loaders.gguf import hf_config_from_gguf, write_gguf
    f = tmp_path / "bad.gguf"
    write_gguf(f, {"general.architecture": "deepseek4", "deepseek4.embedding_length": 256},
               {"token_embd.weight": torch.zeros(8, 256)})
    with pytest.raises(ValueError, match="block_count"):
        hf_config_from_gguf(f)
    write_gguf(f, {"general.architecture": "deepseek4", "deepseek4.embedding_length": 256, "deepseek4.block_count": 2,
                   "deepseek4.attention.head_count": 4}, {"token_embd.weight": torch.zeros(8, 256)})
    with pytest.raises(ValueError, match="attn_q_a"):
        hf_config_from_gguf(f)


def test_model_events_reach_the_observer(llm):
    eng = llm.engine
    eng.observer.reset()
    _tokens(llm, PROMPTS, 4)
    ev = eng.stats()["observer"]["model_events"]
    assert ev["counts"]["rows_allocated"] == 2 and ev["counts"]["rows_released"] == 2
    assert ev["counts"]["decode_batch"] >= 3 and ev["last"]["decode_batch"]["batch_size"] >= 1
    assert ev["last"]["rows_released"]["active_requests"] == 0
    assert ev["last"]["rows_allocated"]["active_requests_high_water"] >= 1


def test_engine_chunked_prefill_matches_one_shot(llm):
    """The engine feeds a long prompt in chunks (`start` advances, the last chunk returns the first token)."""
    cfg = {"profile": "balanced", "tuning_keyvals": {"FASTINFERENCE_LITE_PREFILL_CHUNK": "16", "FASTINFERENCE_MIN_PREFILL_CHUNK": "16",
                                                     "FASTINFERENCE_MAX_PREFILL_CHUNK": "16"}}
    chunked = LLM(PRESET, device="cpu", max_model_len=128, dtype="float32", fastinference_config=cfg)
    try:
        assert chunked.engine.plan.prefill_chunk_size == 16
        long_prompt = [(13 * i + 7) % 500 + 2 for i in range(57)]
        want = _tokens(llm, [long_prompt], 5)
        got = _tokens(chunked, [long_prompt], 5)
        assert got[0][:2] == want[0][:2], (got, want)          # same model, same rows: the walk starts the same
        assert chunked.engine.model.requests == {}
    finally:
        chunked.shutdown()


def test_async_clients_leave_no_rows_behind():
    """Clients of the background loop that finish or walk away: every request's rows are released either way."""
    import asyncio
    import random
    from litevllm_b200.config.config_builder import build_vllm_config
    from litevllm_b200.engine.async_llm import AsyncLLM
    from litevllm_b200.engine.errors import LiteRuntimeError
    rng = random.Random(3)
    plans = [(f"c{i}", [rng.randint(2, 500) for _ in range(rng.randint(4, 40))], rng.randint(1, 6), i % 3 == 0) for i in range(9)]

    async def run():
        eng = AsyncLLM(build_vllm_config(PRESET, dtype="float32", device="cpu", max_num_seqs=3, max_model_len=128))
        try:
            async def client(rid, ids, mt, leaves):
                sp = SamplingParams(temperature=0.0, max_tokens=mt if not leaves else 30, ignore_eos=True)
                while True:
                    try:
                        await eng.submit({"prompt_token_ids": ids}, sp, rid)
                        break
                    except LiteRuntimeError:
                        await asyncio.sleep(0.01)
                agen = eng.stream(rid)
                try:
                    async for out in agen:
                        if leaves and not out.finished:
                            return False
                finally:
                    await agen.aclose()
                return True

            done = await asyncio.gather(*[client(*p) for p in plans])
            for _ in range(300):
                if eng.stats()["scheduler"]["running"] == 0:
                    break
                await asyncio.sleep(0.01)
            model = eng.engine.model
            ev = eng.stats()["observer"]["model_events"]["counts"]
            return done, dict(model.requests), ev
        finally:
            eng.shutdown()

    done, left, ev = asyncio.run(run())
    assert left == {} and sum(done) >= 6
    assert ev["rows_allocated"] == ev["rows_released"] == 9


def test_staged_experts_of_a_gguf_checkpoint_match_resident_ones(llm, tmp_path, monkeypatch):
    """The two-bit routed experts of a `deepseek4` file behind a device budget of three experts per block: the
    tokens equal those of the fully resident model, and the slots saw hits, misses and evictions."""
    path = tmp_path / "tiny-v4-2bit.gguf"
    _write_v4_gguf(llm.engine.model, path, two_bit_experts=True)
    monkeypatch.delenv("FI_EXPERT_STAGING_GB", raising=False)
    resident = LLM(str(path), device="cpu", max_model_len=128, dtype="float32")
    want = _tokens(resident, PROMPTS[:2], 6)
    blocks = [l.routed for l in resident.engine.model.layers]
    assert all(b is not None and b.stager is None for b in blocks)
    per_expert = sum(int(t[0].numel()) * t.element_size() for t in blocks[0].raw.values())
    resident.shutdown()
    monkeypatch.setenv("FI_EXPERT_STAGING_GB", repr(3.5 * per_expert * len(blocks) / 2 ** 30))
    staged = LLM(str(path), device="cpu", max_model_len=128, dtype="float32")
    assert _tokens(staged, PROMPTS[:2], 6) == want
    for l in staged.engine.model.layers:
        snap = l.routed.stager.snapshot()
        assert snap["slots"] == 3 and snap["misses"] > 0 and snap["hits"] > 0 and snap["evictions"] > 0
        assert not l.routed.raw
    staged.shutdown()
