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
