"""KV-cache formats with one scale per (token, head) row: block-scaled e4m3 (``fp8_block``) and packed
int4 (``turbo_int4``).  CPU: quantiser round trips and the engine on every format.  GPU: the quantising
cache write and both attention kernels against the PyTorch reference on the same cache."""
import math

import pytest
import torch

from litevllm_b200 import LLM, SamplingParams, ops
from litevllm_b200.ops import reference as ref


def test_row_quantisers_round_trip():
    torch.manual_seed(0)
    x = torch.randn(5, 3, 64) * torch.tensor([0.01, 1.0, 30.0])[None, :, None]
    q4, s4 = ref.quant_rows(x, 3)
    assert q4.dtype == torch.uint8 and q4.shape == (5, 3, 32) and s4.shape == (5, 3)
    back = ref.dequant_rows(q4, s4, 3)
    assert float(((back - x).abs() / s4[..., None]).max()) <= 0.5 + 1e-3          # half a quantisation step
    assert int(((q4 & 0x0F) == 8).sum() + ((q4 >> 4) == 8).sum()) == 0            # -8 is never produced
    q8, s8 = ref.quant_rows(x, 2)
    back8 = ref.dequant_rows(q8, s8, 2)
    assert float(((back8 - x).abs() / x.abs().amax(-1, keepdim=True)).max()) < 0.07
    tiny = torch.zeros(2, 64)
    q, s = ref.quant_rows(tiny, 3)
    assert float(s.min()) == pytest.approx(1e-4) and int(q.sum()) == 0


def test_engine_runs_on_every_kv_format_cpu():
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (70, 9, 33)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    fmt = {}
    for kv in ("fp16", "fp8", "fp8_block", "turbo_int4"):
        llm = LLM("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=4, max_model_len=128,
                  fastinference_config={"kv_type": kv})
        fmt[kv] = llm.engine.kv_plan.fmt
        outs = llm.generate(prompts, sp)
        assert all(len(o.outputs[0].token_ids) == 6 for o in outs)
        if kv == "turbo_int4":
            k, v = llm.engine.kv_cache.layers[0]
            assert k.dtype == torch.uint8 and k.shape[-1] == 32 and k.fi_scales.shape == k.shape[:3]
            assert llm.engine.kv_plan.bytes_total < 0.4 * 33 * 2 * 2 * 16 * 64 * 2 * 4    # well under the fp32 pool
    assert fmt == {"fp16": 0, "fp8": 1, "fp8_block": 2, "turbo_int4": 3}


def test_prefix_cache_carries_row_scales_cpu():
    llm = LLM("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=2, max_model_len=128,
              fastinference_config={"kv_type": "turbo_int4",
                                    "tuning_keyvals": {"FASTINFERENCE_PREFIX_CACHE_MAX_ENTRIES": "4"}})
    g = torch.Generator().manual_seed(3)
    p = torch.randint(0, 512, (48,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    first = llm.generate([p], sp)[0].outputs[0].token_ids
    again = llm.generate([p + [7, 8]], sp)[0].outputs[0].token_ids            # reuses the cached blocks + scales
    cold = LLM("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=2, max_model_len=128,
               fastinference_config={"kv_type": "turbo_int4"}).generate([p + [7, 8]], sp)[0].outputs[0].token_ids
    assert len(first) == 5 and again == cold


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [2, 3])
@pytest.mark.parametrize("nh,nkv,hd", [(8, 2, 64), (16, 4, 128), (4, 2, 256)])
def test_row_scaled_cache_write_and_attention_gpu(mode, nh, nkv, hd):
    torch.manual_seed(mode * 10 + hd)
    dev = "cuda"
    bs = 16
    lens = [1, 17, 200, 64, 33]
    B = len(lens)
    max_blocks = (max(lens) + bs - 1) // bs + 1
    nb = 1 + B * max_blocks

    def make_cache(device):
        if mode == 3:
            k = torch.zeros(nb, nkv, bs, hd // 2, dtype=torch.uint8, device=device)
        else:
            k = torch.zeros(nb, nkv, bs, hd, device=device).to(torch.float8_e4m3fn)
        v = k.clone()
        for t in (k, v):
            t.fi_scales = torch.zeros(nb, nkv, bs, dtype=torch.float32, device=device)
            t.fi_mode = mode
        return k, v
    kc, vc = make_cache(dev)
    kr, vr = make_cache("cpu")
    bt = torch.zeros(B, max_blocks, dtype=torch.int32)
    perm = torch.randperm(nb - 1) + 1
    used = 0
    for b in range(B):
        n = (lens[b] + bs - 1) // bs
        bt[b, :n] = perm[used:used + n].to(torch.int32)
        used += n
    # fill the caches token by token through the quantising write (all tokens of all sequences at once)
    T = sum(lens)
    k_new = (torch.randn(T, nkv, hd) * torch.rand(T, nkv, 1) * 3).bfloat16()
    v_new = (torch.randn(T, nkv, hd) * torch.rand(T, nkv, 1) * 3).bfloat16()
    slots = torch.cat([bt[b, torch.arange(lens[b]) // bs].long() * bs + torch.arange(lens[b]) % bs for b in range(B)]).int()
    ops.reshape_and_cache(k_new.to(dev), v_new.to(dev), slots.to(dev), kc, vc)
    ref.reshape_and_cache(k_new, v_new, slots, kr, vr)
    torch.cuda.synchronize()
    if mode == 3:
        # nibbles may differ by one step where bf16 rounding of value / scale sits on a boundary
        diff = (ref.dequant_rows(kc.cpu(), kc.fi_scales.cpu(), 3) - ref.dequant_rows(kr, kr.fi_scales, 3)).abs()
        assert float((diff / kr.fi_scales[..., None].clamp_min(1e-4)).max()) <= 1.001
        assert float((kc.cpu() != kr).float().mean()) < 0.01      # bytes differ only at exact .5 boundaries
    else:
        assert float((kc.cpu().float() - kr.float()).abs().max()) <= 32.0          # one e4m3 step at the top of the range
    assert torch.allclose(kc.fi_scales.cpu(), kr.fi_scales, rtol=1e-5, atol=1e-7)
    # attention on the GPU-written cache: kernels vs reference reading the same bytes
    kcpu, vcpu = kc.cpu(), vc.cpu()
    for t, src in ((kcpu, kc), (vcpu, vc)):
        t.fi_scales, t.fi_mode = src.fi_scales.cpu(), mode
    scale = 1.0 / math.sqrt(hd)
    sl = torch.tensor(lens, dtype=torch.int32)
    q = torch.randn(B, nh * hd).bfloat16()
    cu = torch.arange(B + 1, dtype=torch.int32)
    want = ref.paged_attention(q, kcpu, vcpu, bt, sl, cu, nh, nkv, hd, scale, out_dtype=torch.float32)
    for splits in (1, 3):
        got = ops.paged_attention_decode(q.to(dev), kc, vc, bt.to(dev), sl.to(dev), nh, nkv, hd, scale, splits=splits,
                                         max_kv_len=max(lens))
        err = (got.float().cpu() - want).abs()
        assert bool((err <= 3e-2 + 3e-2 * want.abs()).all()), (mode, splits, float(err.max()))
    # prefill: the last min(len, 40) tokens of every sequence are query tokens
    qlens = [min(l, 40) for l in lens]
    cu_q = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32)
    qp = torch.randn(sum(qlens), (nh + 2 * nkv) * hd).bfloat16()
    want_p = ref.paged_attention(qp, kcpu, vcpu, bt, sl, cu_q, nh, nkv, hd, scale, out_dtype=torch.float32)
    got_p = ops.paged_attention_prefill(qp.to(dev), kc, vc, bt.to(dev), sl.to(dev), cu_q.to(dev), max(qlens), nh, nkv,
                                        hd, scale)
    err = (got_p.float().cpu() - want_p).abs()
    assert bool((err <= 3e-2 + 3e-2 * want_p.abs()).all()), (mode, float(err.max()))
    ops.check_status(torch.device(dev, 0))


@pytest.mark.gpu
@pytest.mark.parametrize("kv", ["fp8_block", "turbo_int4"])
def test_engine_row_scaled_kv_gpu(kv):
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (70, 9, 33)]
    llm = LLM("synthetic:tiny-llama-test", dtype="bfloat16", device="cuda:0", max_num_seqs=4, max_model_len=128,
              fastinference_config={"kv_type": kv})
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    assert all(len(o.outputs[0].token_ids) == 8 for o in outs)
    ops.check_status(torch.device("cuda:0"))


@pytest.mark.parametrize("kv_type", ["fp8", "fp8_block", "turbo_int4"])
def test_quantised_caches_keep_batch_invariance_on_the_cpu_path(kv_type):
    """Rows are quantised one (token, head) at a time, so what a request generates cannot depend on who shares the
    step with it or on how its prompt was chunked."""
    import random
    from litevllm_b200 import LLM, SamplingParams
    rng = random.Random(7)
    prompts = [{"prompt_token_ids": [rng.randint(2, 400) for _ in range(rng.randint(5, 45))]} for _ in range(7)]
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    cfg = {"profile": "balanced", "kv_type": kv_type,
           "tuning_keyvals": {"FASTINFERENCE_LITE_PREFILL_CHUNK": "16", "FASTINFERENCE_MIN_PREFILL_CHUNK": "16",
                              "FASTINFERENCE_MAX_PREFILL_CHUNK": "16"}}
    llm = LLM("synthetic:tiny-llama-test", dtype="float32", device="cpu", max_num_seqs=3, max_model_len=96,
              fastinference_config=cfg)
    try:
        together = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        alone = [llm.generate([p], sp)[0].outputs[0].token_ids for p in prompts]
        assert together == alone
    finally:
        llm.shutdown()
