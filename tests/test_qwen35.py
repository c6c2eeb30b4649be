"""Qwen3.5 hybrid model: the chunked gated delta rule against the token-by-token recurrence, decode
steps on the slot-indexed state pools against one long prefill, and the MoE variant."""
import pytest
import torch

from litevllm_b200 import LLM, SamplingParams
from litevllm_b200.ops import linear_attn as la


@pytest.mark.parametrize("L", [1, 7, 64, 65, 200])
def test_chunked_rule_equals_recurrence(L):
    torch.manual_seed(L)
    H, dk, dv = 3, 16, 24
    q = torch.nn.functional.normalize(torch.randn(L, H, dk), dim=-1) * dk ** -0.5
    k = torch.nn.functional.normalize(torch.randn(L, H, dk), dim=-1)
    v = torch.randn(L, H, dv)
    g = -torch.rand(L, H) * 0.5
    beta = torch.sigmoid(torch.randn(L, H))
    S0 = torch.randn(H, dk, dv) * 0.1
    o1, S1 = la.gated_delta_recurrent(q, k, v, g, beta, S0)
    o2, S2 = la.gated_delta_chunked(q, k, v, g, beta, S0)
    assert float((o1 - o2).abs().max()) < 1e-5 and float((S1 - S2).abs().max()) < 1e-5
    # two halves with the state carried over = one pass
    if L > 1:
        h = L // 2
        oa, Sa = la.gated_delta_chunked(q[:h], k[:h], v[:h], g[:h], beta[:h], S0)
        ob, Sb = la.gated_delta_chunked(q[h:], k[h:], v[h:], g[h:], beta[h:], Sa)
        assert float((torch.cat([oa, ob]) - o1).abs().max()) < 1e-5 and float((Sb - S1).abs().max()) < 1e-5


def test_step_ops_cpu_match_recurrence():
    torch.manual_seed(3)
    B, H, dk, dv, C, kw = 3, 2, 8, 8, 12, 4
    pool = torch.randn(5, H, dk, dv)
    want_pool = pool.clone()
    slots = torch.tensor([4, -1, 1], dtype=torch.int32)
    q, k, v = torch.randn(B, H, dk), torch.randn(B, H, dk), torch.randn(B, H, dv)
    g, beta = -torch.rand(B, H), torch.rand(B, H)
    o = la.gated_delta_step(pool, slots, q, k, v, g, beta)
    for b, s in enumerate(slots.tolist()):
        if s < 0:
            continue
        ow, Sw = la.gated_delta_recurrent(q[b:b + 1], k[b:b + 1], v[b:b + 1], g[b:b + 1], beta[b:b + 1], want_pool[s])
        assert torch.allclose(o[b], ow[0], atol=1e-6) and torch.allclose(pool[s], Sw, atol=1e-6)
    assert torch.equal(pool[0], want_pool[0]) and torch.equal(pool[2], want_pool[2])
    cpool = torch.randn(5, C, kw - 1)
    w = torch.randn(C, kw)
    x = torch.randn(B, C)
    before = cpool.clone()
    y = la.conv1d_step(x, cpool, slots, w)
    win = torch.cat([before[4], x[0][:, None]], dim=1)
    assert torch.allclose(y[0], torch.nn.functional.silu((win * w).sum(-1)), atol=1e-6)
    assert torch.allclose(cpool[4], win[:, 1:]) and torch.equal(cpool[3], before[3])


@pytest.mark.parametrize("preset", ["tiny-qwen35-test", "tiny-qwen35-moe-test"])
def test_decode_steps_agree_with_one_long_prefill_cpu(preset):
    """Greedy tokens produced by prefill + decode steps (state pools, step ops) must be what a fresh
    prefill of prompt + generated prefix predicts next (chunk-wise rule over the whole sequence), also
    when the prompt is fed in several chunks."""
    kw = dict(dtype="float32", device="cpu", max_num_seqs=4, max_model_len=256)
    llm = LLM(f"synthetic:{preset}", **kw)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (70, 9)]
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    outs = llm.generate(prompts, sp)
    gen = [list(o.outputs[0].token_ids) for o in outs]
    one = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    for p, gt in zip(prompts, gen):
        for n in range(1, 5):
            nxt = llm.generate([p + gt[:n]], one)[0].outputs[0].token_ids[0]
            assert nxt == gt[n], (preset, n, nxt, gt)
    # chunked prefill (32-token chunks) gives the same continuation as one chunk
    small = LLM(f"synthetic:{preset}", max_num_batched_tokens=32,
                fastinference_config={"tuning_keyvals": {"FASTINFERENCE_LITE_PREFILL_CHUNK": "32", "FASTINFERENCE_MIN_PREFILL_CHUNK": "16"}}, **kw)
    outs2 = small.generate(prompts, sp)
    assert [list(o.outputs[0].token_ids) for o in outs2] == gen


@pytest.mark.gpu
def test_step_kernels_match_torch_gpu():
    torch.manual_seed(5)
    dev = "cuda"
    B, H, dk, dv, C, kw = 5, 6, 128, 128, 512, 4
    pool = torch.randn(9, H, dk, dv, device=dev)
    ref_pool = pool.cpu().clone()
    slots = torch.tensor([3, -1, 8, 0, 5], dtype=torch.int32, device=dev)
    q = torch.nn.functional.normalize(torch.randn(B, H, dk, device=dev), dim=-1) * dk ** -0.5
    k = torch.nn.functional.normalize(torch.randn(B, H, dk, device=dev), dim=-1)
    v = torch.randn(B, H, dv, device=dev)
    g, beta = -torch.rand(B, H, device=dev), torch.rand(B, H, device=dev)
    for _ in range(2):
        o = la.gated_delta_step(pool, slots, q, k, v, g, beta)
        ow = la.gated_delta_step(ref_pool, slots.cpu(), q.cpu(), k.cpu(), v.cpu(), g.cpu(), beta.cpu())
        live = slots.cpu() >= 0
        assert float((o.cpu()[live] - ow[live]).abs().max()) < 1e-3
        assert float((pool.cpu() - ref_pool).abs().max()) < 1e-3
    cpool = torch.randn(9, C, kw - 1, device=dev).bfloat16()
    rpool = cpool.cpu().clone()
    w = torch.randn(C, kw, device=dev).bfloat16()
    x = torch.randn(B, C, device=dev).bfloat16()
    y = la.conv1d_step(x, cpool, slots, w)
    yw = la.conv1d_step(x.cpu(), rpool, slots.cpu(), w.cpu())
    live = slots.cpu() >= 0
    assert float((y.cpu()[live] - yw[live]).abs().max()) < 2e-2
    assert torch.equal(cpool.cpu(), rpool)


@pytest.mark.parametrize("preset", ["tiny-qwen35-test", "tiny-qwen35-moe-test"])
def test_gguf_file_with_the_exporters_conventions_round_trips(tmp_path, preset):
    """A Qwen3.5 GGUF file stores value heads tiled, RMSNorm gains plus one, the depthwise convolution as
    [kernel, channels] and -exp(A_log); a directory with `config.json` and such a file loads to the same model as
    the HF-layout tensors it was exported from."""
    import json
    import re
    import torch
    from litevllm_b200 import LLM, SamplingParams
    from litevllm_b200.loaders import synth
    from litevllm_b200.loaders.gguf import _QWEN35_LAYER_MAP, grouped_to_tiled, tiled_to_grouped, write_gguf
    from litevllm_b200.models.presets import PRESETS

    x = torch.arange(2 * 3 * 4 * 5, dtype=torch.float32).reshape(2, 3 * 4, 5)
    assert torch.equal(tiled_to_grouped(grouped_to_tiled(x, 1, 3, 4, 1), 1, 3, 4, 1), x)
    assert not torch.equal(grouped_to_tiled(x, 1, 3, 4, 1), x)

    cfg = PRESETS[preset]
    src = LLM(f"synthetic:{preset}", device="cpu", dtype="float32", max_num_seqs=2, max_model_len=96)
    arch = src.engine.arch
    nk, nv, dk, dv = (cfg[k] for k in ("linear_num_key_heads", "linear_num_value_heads", "linear_key_head_dim",
                                       "linear_value_head_dim"))
    per, qk = nv // nk, 2 * nk * dk
    back = {v: k for k, v in _QWEN35_LAYER_MAP.items() if k != "ffn_norm"}
    tensors = {}
    experts: dict = {}
    for name, t in synth.iter_qwen35_weights(arch, 0, torch.float32, "cpu"):
        t = t.float()
        em = re.match(r"model\.layers\.(\d+)\.mlp\.experts\.(\d+)\.(\w+)\.weight", name)
        if em:                                   # the file holds one [experts, rows, cols] tensor per projection
            experts.setdefault((em.group(1), em.group(3)), {})[int(em.group(2))] = t
            continue
        if name == "model.embed_tokens.weight":
            tensors["token_embd.weight"] = t
        elif name == "model.norm.weight":
            tensors["output_norm.weight"] = t + 1.0
        elif name == "lm_head.weight":
            tensors["output.weight"] = t
        else:
            layer, rest = re.match(r"model\.layers\.(\d+)\.(.+)", name).groups()
            if rest == "linear_attn.A_log":
                tensors[f"blk.{layer}.ssm_a"] = grouped_to_tiled((-torch.exp(t)).unsqueeze(-1), 0, nk, per, 1).squeeze(-1)
            elif rest == "linear_attn.dt_bias":
                tensors[f"blk.{layer}.ssm_dt.bias"] = grouped_to_tiled(t.unsqueeze(-1), 0, nk, per, 1).squeeze(-1)
            else:
                mod, suffix = rest.rsplit(".", 1)
                kind = back[mod]
                if kind == "ssm_conv1d":
                    c = t.reshape(t.shape[0], -1)
                    c = torch.cat([c[:qk], grouped_to_tiled(c[qk:], 0, nk, per, dv)])
                    t = c.t().contiguous()                                   # [kernel, channels]
                elif kind.endswith("norm") and kind != "ssm_norm":
                    t = t + 1.0
                elif kind == "attn_qkv":
                    t = torch.cat([t[:qk], grouped_to_tiled(t[qk:], 0, nk, per, dv)])
                elif kind == "attn_gate":
                    t = grouped_to_tiled(t, 0, nk, per, dv)
                elif kind == "ssm_out":
                    t = grouped_to_tiled(t, 1, nk, per, dv)
                elif kind in ("ssm_alpha", "ssm_beta"):
                    t = grouped_to_tiled(t, 0, nk, per, 1)
                tensors[f"blk.{layer}.{kind}.{suffix}"] = t.contiguous()
    for (layer, which), per_expert in experts.items():
        kind = {"gate_proj": "ffn_gate_exps", "up_proj": "ffn_up_exps", "down_proj": "ffn_down_exps"}[which]
        tensors[f"blk.{layer}.{kind}.weight"] = torch.stack([per_expert[e] for e in sorted(per_expert)])
    # the synthetic stream carries no norm gains: give the source model random ones and export them shifted
    gen = torch.Generator().manual_seed(9)
    for pname, p in src.engine.model.named_parameters():
        if not pname.endswith("norm.weight"):
            continue
        p.data.copy_(torch.randn(p.shape, generator=gen) * 0.1)
        if pname == "norm.weight":
            tensors["output_norm.weight"] = p.detach().float() + 1.0
            continue
        layer, mod = re.match(r"layers\.(\d+)\.(.+)\.weight", pname).groups()
        kind = back[mod]
        tensors[f"blk.{layer}.{kind}.weight"] = p.detach().float() + (0.0 if kind == "ssm_norm" else 1.0)
    d = tmp_path / "qwen35-gguf"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    write_gguf(d / "model.gguf", {"general.architecture": "qwen35", "qwen35.block_count": cfg["num_hidden_layers"],
                                  "qwen35.embedding_length": cfg["hidden_size"]}, tensors)
    loaded = LLM(str(d), device="cpu", dtype="float32", max_num_seqs=2, max_model_len=96)
    a, b = dict(src.engine.model.named_parameters()), dict(loaded.engine.model.named_parameters())
    assert a.keys() == b.keys()
    for k in a:
        torch.testing.assert_close(b[k].float(), a[k].float(), rtol=1e-5, atol=1e-5, msg=lambda m, k=k: f"{k}: {m}")
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    prompt = [{"prompt_token_ids": [(5 * i + 3) % 400 + 2 for i in range(20)]}]
    assert loaded.generate(prompt, sp)[0].outputs[0].token_ids == src.generate(prompt, sp)[0].outputs[0].token_ids
