"""CUDA kernels vs the PyTorch fp32 reference of the same op (small and odd shapes)."""
import math

import pytest
import torch

from litevllm_b200 import ops
from litevllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, rtol, atol, what=""):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = err > tol
    assert not bool(bad.any()), (
        f"{what}: {int(bad.sum())}/{bad.numel()} mismatches, max abs err {float(err.max()):.4g}, "
        f"ref absmax {float(b.abs().max()):.4g}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,N,K,splits", [
    (1, 256, 128, 1), (16, 2560, 2048, 0), (32, 2048, 5632, 0), (32, 2048, 5632, 1),
    (7, 384, 512, 0), (100, 384, 520, 2), (300, 1024, 1024, 0), (64, 128, 64, 1),
    (129, 520, 1032, 0), (32, 32000, 2048, 0),
])
def test_dense_gemm(T, N, K, splits, dtype):
    torch.manual_seed(0)
    x = (torch.randn(T, K, device=DEV) * 0.5).to(dtype)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(dtype)
    y = ops.linear(x, w, splits=splits)
    _close(y, ref.linear(x, w, out_dtype=torch.float32), 2e-2, 2e-2, f"gemm {T}x{N}x{K}")
    ops.check_status(x.device)


def test_dense_gemm_epilogues():
    torch.manual_seed(1)
    T, N, K = 48, 1024, 768
    x = (torch.randn(T, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.05).bfloat16()
    bias = torch.randn(N, device=DEV).bfloat16()
    res = torch.randn(T, N, device=DEV).bfloat16()
    y = ops.linear(x, w, bias=bias, residual=res)
    _close(y, ref.linear(x, w, bias, res, out_dtype=torch.float32), 2e-2, 2e-2, "bias+residual")
    y32 = ops.linear(x, w, out_dtype=torch.float32)
    assert y32.dtype == torch.float32
    _close(y32, ref.linear(x, w, out_dtype=torch.float32), 1e-3, 1e-3, "fp32 out")
    # in-place residual accumulate (out aliases residual)
    h = res.clone()
    ops.linear(x, w, residual=h, out=h)
    _close(h, ref.linear(x, w, None, res, out_dtype=torch.float32), 2e-2, 2e-2, "in-place residual")
    # deterministic across runs (cluster split-K has a fixed summation order)
    a = ops.linear(x, w, splits=4)
    b = ops.linear(x, w, splits=4)
    assert torch.equal(a, b)


@pytest.mark.parametrize("T,I,K,act,splits", [(32, 5632, 2048, "silu", 0), (5, 256, 128, "gelu_tanh", 1),
                                              (200, 640, 512, "silu", 0), (16, 1408, 1024, "gelu_tanh", 3)])
def test_gated_gemm(T, I, K, act, splits):
    torch.manual_seed(2)
    x = (torch.randn(T, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(2 * I, K, device=DEV) * 0.05).bfloat16()
    y = ops.gated_linear(x, w, act, splits=splits)
    _close(y, ref.gated_linear(x, w, act, out_dtype=torch.float32), 3e-2, 2e-2, f"gated {T}x{I}x{K}")
    ops.check_status(x.device)


@pytest.mark.parametrize("rows,H", [(5, 2048), (33, 4096), (64, 128), (7, 256), (3, 2816)])
@pytest.mark.parametrize("w_mode", [0, 1, 2])
def test_rmsnorm(rows, H, w_mode):
    torch.manual_seed(3)
    x = torch.randn(rows, H, device=DEV).bfloat16()
    w = (torch.randn(H, device=DEV) * 0.1 + 1).bfloat16()
    y = ops.rmsnorm(x, w, 1e-5, w_mode=w_mode)
    yr, _ = ref.rmsnorm(x, w, 1e-5, w_mode=w_mode)
    _close(y, yr, 1e-2, 1e-2, "rmsnorm")
    res = torch.randn(rows, H, device=DEV).bfloat16()
    res2 = res.clone()
    y = ops.rmsnorm(x, w, 1e-5, residual=res2, w_mode=w_mode)
    yr, rr = ref.rmsnorm(x, w, 1e-5, residual=res, w_mode=w_mode)
    _close(res2, rr, 1e-2, 1e-2, "residual out")
    _close(y, yr, 2e-2, 2e-2, "fused add rmsnorm")


def _make_cache(num_blocks, nkv, bs, hd, dtype, fp8):
    shape = (num_blocks, nkv, bs, hd)
    if fp8:
        return (torch.zeros(shape, device=DEV, dtype=torch.float8_e4m3fn),
                torch.zeros(shape, device=DEV, dtype=torch.float8_e4m3fn))
    return torch.zeros(shape, device=DEV, dtype=dtype), torch.zeros(shape, device=DEV, dtype=dtype)


@pytest.mark.parametrize("nh,nkv,hd,rot,fp8,norm", [(32, 4, 64, 64, False, -1), (8, 2, 128, 64, True, 0),
                                                    (4, 2, 256, 256, True, 1), (2, 1, 128, 128, False, -1)])
def test_rope_cache(nh, nkv, hd, rot, fp8, norm):
    torch.manual_seed(4)
    T, bs, nb = 37, 16, 12
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV).bfloat16()
    pos = torch.randint(0, 500, (T,), device=DEV, dtype=torch.int32)
    cs = ref.build_cos_sin(rot, 512, 10000.0).to(DEV)
    slots = torch.randperm((nb - 1) * bs, device=DEV)[:T].to(torch.int32) + bs
    slots[3] = -1
    qw = (torch.randn(hd, device=DEV) * 0.1 + 1).bfloat16() if norm >= 0 else None
    kw = (torch.randn(hd, device=DEV) * 0.1 + 1).bfloat16() if norm >= 0 else None
    kc, vc = _make_cache(nb, nkv, bs, hd, torch.bfloat16, fp8)
    kcr, vcr = kc.clone(), vc.clone()
    a, b = qkv.clone(), qkv.clone()
    kw_args = dict(q_norm_w=qw, k_norm_w=kw, qk_norm_mode=norm, v_norm=(norm == 1), eps=1e-6,
                   k_scale=0.5, v_scale=0.25)
    ops.rope_and_cache(a, pos, cs, slots, kc, vc, nh, nkv, hd, rot, **kw_args)
    ref.rope_and_cache(b, pos, cs, slots, kcr, vcr, nh, nkv, hd, rot, **kw_args)
    _close(a, b, 2e-2, 2e-2, "rotated qkv")
    _close(kc.float(), kcr.float(), 0.13 if fp8 else 2e-2, 2e-2, "k cache")
    _close(vc.float(), vcr.float(), 0.13 if fp8 else 2e-2, 2e-2, "v cache")


def _fill_paged(B, lens, nkv, hd, bs, fp8, dtype=torch.bfloat16):
    max_blocks = (max(lens) + bs - 1) // bs + 1
    nb = 1 + B * max_blocks
    kc, vc = _make_cache(nb, nkv, bs, hd, dtype, fp8)
    bt = torch.zeros(B, max_blocks, dtype=torch.int32, device=DEV)
    perm = torch.randperm(nb - 1, device=DEV) + 1
    used = 0
    for b in range(B):
        n = (lens[b] + bs - 1) // bs
        bt[b, :n] = perm[used:used + n].to(torch.int32)
        used += n
    k = torch.randn(nb, nkv, bs, hd, device=DEV) * 0.7
    v = torch.randn(nb, nkv, bs, hd, device=DEV) * 0.7
    if fp8:
        kc.copy_(ref.fp8_quant(k, 0.5)); vc.copy_(ref.fp8_quant(v, 0.5))
    else:
        kc.copy_(k.to(dtype)); vc.copy_(v.to(dtype))
    return kc, vc, bt


@pytest.mark.parametrize("nh,nkv,hd", [(32, 4, 64), (32, 8, 128), (16, 8, 256), (4, 4, 64), (40, 2, 128)])
@pytest.mark.parametrize("fp8,window,softcap,splits", [(False, 0, 0.0, 1), (False, 0, 0.0, 0), (True, 100, 50.0, 3),
                                                       (False, 64, 0.0, 2)])
def test_paged_decode(nh, nkv, hd, fp8, window, softcap, splits):
    torch.manual_seed(5)
    lens = [1, 16, 17, 250, 129, 64]
    B, bs = len(lens), 16
    kc, vc, bt = _fill_paged(B, lens, nkv, hd, bs, fp8)
    q = torch.randn(B, nh * hd, device=DEV).bfloat16()
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    ks = vs = 0.5 if fp8 else 1.0
    y = ops.paged_attention_decode(q, kc, vc, bt, sl, nh, nkv, hd, scale, window, softcap, ks, vs,
                                   splits=splits, max_kv_len=max(lens))
    cu = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    yr = ref.paged_attention(q, kc, vc, bt, sl, cu, nh, nkv, hd, scale, window, softcap, ks, vs,
                             out_dtype=torch.float32)
    _close(y, yr, 2e-2, 2e-2, f"decode nh{nh} nkv{nkv} hd{hd}")


@pytest.mark.parametrize("merge", ["cluster", "kernel", "ticket"])
@pytest.mark.parametrize("nh,nkv,hd,fp8,splits", [(32, 4, 64, False, 2), (32, 4, 64, False, 4), (32, 8, 128, True, 8),
                                                  (16, 8, 256, False, 3), (40, 2, 128, False, 5)])
def test_paged_decode_merge_variants(monkeypatch, merge, nh, nkv, hd, fp8, splits):
    """The three ways of merging split-KV partials (thread-block cluster over distributed shared memory,
    separate merge launch, last-CTA ticket) against the fp32 oracle, including splits with no tokens."""
    monkeypatch.setattr(ops, "_DECODE_MERGE", merge)
    torch.manual_seed(7)
    lens = [1, 40, 300, 129, 1000, 64, 17]
    B, bs = len(lens), 16
    kc, vc, bt = _fill_paged(B, lens, nkv, hd, bs, fp8)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    ks = vs = 0.5 if fp8 else 1.0
    cu = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    for rep in range(2):
        q = torch.randn(B, nh * hd, device=DEV).bfloat16()
        y = ops.paged_attention_decode(q, kc, vc, bt, sl, nh, nkv, hd, scale, 0, 0.0, ks, vs, splits=splits,
                                       max_kv_len=max(lens))
        yr = ref.paged_attention(q, kc, vc, bt, sl, cu, nh, nkv, hd, scale, 0, 0.0, ks, vs, out_dtype=torch.float32)
        _close(y, yr, 2e-2, 2e-2, f"{merge} merge rep {rep} nh{nh} nkv{nkv} hd{hd} splits {splits}")


@pytest.mark.parametrize("nh,nkv,hd,fp8", [(8, 2, 64, False), (32, 8, 128, False), (8, 2, 128, True)])
def test_paged_decode_long_context_merges_in_kernel(nh, nkv, hd, fp8):
    """Long splits (>= 1024 tokens each): the last split CTA merges the partials itself; run twice so the
    second call sees the tickets the first one left (they must be zero again)."""
    torch.manual_seed(11)
    import litevllm_b200.ops as O
    saved, O._DECODE_MERGE = O._DECODE_MERGE, "ticket"
    lens = [4096, 2100, 3000, 1]
    B, bs = len(lens), 16
    kc, vc, bt = _fill_paged(B, lens, nkv, hd, bs, fp8)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    ks = vs = 0.5 if fp8 else 1.0
    cu = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    for rep in range(2):
        q = torch.randn(B, nh * hd, device=DEV).bfloat16()
        y = ops.paged_attention_decode(q, kc, vc, bt, sl, nh, nkv, hd, scale, 0, 0.0, ks, vs, splits=3,
                                       max_kv_len=max(lens))
        yr = ref.paged_attention(q, kc, vc, bt, sl, cu, nh, nkv, hd, scale, 0, 0.0, ks, vs, out_dtype=torch.float32)
        _close(y, yr, 2e-2, 2e-2, f"merged decode rep {rep} nh{nh} nkv{nkv} hd{hd}")
    O._DECODE_MERGE = saved
    assert int(ops._merge_tickets(torch.device(DEV, 0)).abs().sum().item()) == 0


@pytest.mark.parametrize("nh,nkv,hd", [(8, 2, 64), (8, 4, 128), (4, 2, 256)])
@pytest.mark.parametrize("fp8,window,softcap", [(False, 0, 0.0), (True, 0, 30.0), (False, 48, 0.0)])
def test_paged_prefill(nh, nkv, hd, fp8, window, softcap):
    torch.manual_seed(6)
    # (q_len, kv_len): fresh prompts, a chunk continuing a cached prefix, single-token rows
    cases = [(70, 70), (1, 1), (130, 200), (16, 16), (33, 97), (1, 50)]
    B, bs = len(cases), 16
    lens = [c[1] for c in cases]
    kc, vc, bt = _fill_paged(B, lens, nkv, hd, bs, fp8)
    T = sum(c[0] for c in cases)
    width = (nh + 2 * nkv) * hd
    qkv = torch.randn(T, width, device=DEV).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor([c[0] for c in cases]).cumsum(0)), dtype=torch.int32, device=DEV)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    ks = vs = 0.5 if fp8 else 1.0
    y = ops.paged_attention_prefill(qkv, kc, vc, bt, sl, cu, max(c[0] for c in cases), nh, nkv, hd, scale,
                                    window, softcap, ks, vs)
    yr = ref.paged_attention(qkv, kc, vc, bt, sl, cu, nh, nkv, hd, scale, window, softcap, ks, vs,
                             out_dtype=torch.float32)
    _close(y, yr, 2e-2, 2e-2, f"prefill nh{nh} nkv{nkv} hd{hd}")


@pytest.mark.parametrize("nh,nkv,hd", [(8, 2, 64), (4, 2, 128), (2, 2, 64)])
@pytest.mark.parametrize("window,softcap,dtype,bs", [(0, 0.0, torch.bfloat16, 16), (300, 0.0, torch.bfloat16, 32),
                                                     (0, 30.0, torch.float16, 64), (128, 20.0, torch.bfloat16, 128)])
def test_paged_prefill_tensor_core(nh, nkv, hd, window, softcap, dtype, bs):
    """The tcgen05 prefill kernel against the fp32 oracle, and against the mma.sync kernel's own result:
    several 128-row query tiles and 128-key tiles per sequence, chunks that continue a cached prefix,
    ragged lengths on both axes, sliding window and soft cap."""
    import litevllm_b200.ops as O
    torch.manual_seed(16)
    cases = [(700, 700), (1, 1), (130, 1500), (128, 128), (257, 900), (5, 1000), (384, 385)]
    B = len(cases)
    lens = [c[1] for c in cases]
    kc, vc, bt = _fill_paged(B, lens, nkv, hd, bs, False, dtype)
    T = sum(c[0] for c in cases)
    width = (nh + 2 * nkv) * hd
    qkv = torch.randn(T, width, device=DEV).to(dtype)
    cu = torch.tensor([0] + list(torch.tensor([c[0] for c in cases]).cumsum(0)), dtype=torch.int32, device=DEV)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    outs = {}
    saved = O._PREFILL_TC
    try:
        for mode in ("on", "off"):
            O._PREFILL_TC = mode
            outs[mode] = ops.paged_attention_prefill(qkv, kc, vc, bt, sl, cu, max(c[0] for c in cases), nh, nkv, hd,
                                                     scale, window, softcap)
    finally:
        O._PREFILL_TC = saved
    torch.cuda.synchronize()
    ops.check_status(torch.device(DEV, 0))
    yr = ref.paged_attention(qkv, kc, vc, bt, sl, cu, nh, nkv, hd, scale, window, softcap, 1.0, 1.0,
                             out_dtype=torch.float32)
    _close(outs["on"], yr, 2e-2, 2e-2, f"tc prefill nh{nh} nkv{nkv} hd{hd} w{window} cap{softcap}")
    _close(outs["on"], outs["off"].float(), 2e-2, 2e-2, "tc prefill vs mma.sync prefill")


def test_paged_prefill_tensor_core_repeated():
    """Many back-to-back launches over long sequences (hundreds of KV tiles per CTA in flight on every SM):
    no bounded wait may run out and every launch must give the same result."""
    import litevllm_b200.ops as O
    torch.manual_seed(17)
    nh, nkv, hd, bs, B, L = 16, 4, 128, 16, 6, 2048
    kc, vc, bt = _fill_paged(B, [L] * B, nkv, hd, bs, False)
    qkv = torch.randn(B * L, (nh + 2 * nkv) * hd, device=DEV).bfloat16()
    cu = torch.arange(B + 1, dtype=torch.int32, device=DEV) * L
    sl = torch.full((B,), L, dtype=torch.int32, device=DEV)
    saved = O._PREFILL_TC
    O._PREFILL_TC = "on"
    try:
        first = ops.paged_attention_prefill(qkv, kc, vc, bt, sl, cu, L, nh, nkv, hd, hd ** -0.5).clone()
        for _ in range(40):
            y = ops.paged_attention_prefill(qkv, kc, vc, bt, sl, cu, L, nh, nkv, hd, hd ** -0.5)
        torch.cuda.synchronize()
    finally:
        O._PREFILL_TC = saved
    ops.check_status(torch.device(DEV, 0))
    assert torch.equal(y, first)


def test_small_ops():
    torch.manual_seed(7)
    table = torch.randn(1000, 256, device=DEV).bfloat16()
    ids = torch.randint(0, 1000, (77,), device=DEV)
    _close(ops.embedding(ids, table, scale=16.0), ref.embedding(ids, table, scale=16.0), 1e-2, 1e-2, "embedding")
    x = torch.randn(9, 2 * 704, device=DEV).bfloat16()
    _close(ops.act_mul(x, "silu"), ref.act_mul(x, "silu"), 2e-2, 1e-2, "silu_mul")
    _close(ops.act_mul(x, "gelu_tanh"), ref.act_mul(x, "gelu_tanh"), 2e-2, 1e-2, "gelu_mul")
    logits = torch.randn(6, 32000, device=DEV)
    logits[2, 100] = logits[2, 5000] = 99.0
    assert torch.equal(ops.argmax(logits), ref.argmax(logits))
    assert torch.equal(ops.argmax(logits.bfloat16()), ref.argmax(logits.bfloat16()))
    bt = torch.randint(1, 50, (4, 8), device=DEV, dtype=torch.int32)
    bt[1, 3] = 0
    pos = torch.tensor([0, 5, 17, 50, 100, 127, 3], device=DEV, dtype=torch.int32)
    seq = torch.tensor([0, 1, 2, 1, 3, 3, -1], device=DEV, dtype=torch.int32)
    assert torch.equal(ops.slot_mapping(pos, seq, bt, 16), ref.slot_mapping(pos, seq, bt, 16))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,N,K,G,zp,splits", [(16, 512, 512, 128, True, 1), (1, 256, 256, 32, False, 0),
                                               (33, 1280, 1024, 128, True, 0), (200, 384, 512, 32, False, 0),
                                               (16, 6144, 4096, 128, True, 0), (7, 200, 320, 64, True, 2)])
def test_int4_gemm(T, N, K, G, zp, splits, dtype):
    from litevllm_b200.ops import awq
    torch.manual_seed(8)
    nib = torch.randint(0, 16, (N, K), device=DEV, dtype=torch.uint8)
    scales = (torch.randn(N, K // G, device=DEV).abs() * 0.01 + 1e-3).to(dtype)
    zeros = torch.randint(0, 16, (N, K // G), device=DEV, dtype=torch.uint8) if zp else None
    w = awq.Int4Weight(nib, scales, zeros, G, dtype, keep_reference=True)
    x = (torch.randn(T, K, device=DEV) * 0.5).to(dtype)
    y = awq.int4_linear(x, w, splits=splits)
    dense = awq.dequantize(nib, scales, zeros, G)
    _close(y, ref.linear(x, dense, out_dtype=torch.float32), 3e-2, 3e-2, f"int4 gemm {T}x{N}x{K} g{G}")
    ops.check_status(x.device)


def test_int4_gated_and_layout_roundtrip():
    from litevllm_b200.ops import awq
    torch.manual_seed(9)
    T, I, K, G = 24, 640, 512, 32
    nib = torch.randint(0, 16, (2 * I, K), device=DEV, dtype=torch.uint8)
    scales = (torch.randn(2 * I, K // G, device=DEV).abs() * 0.01 + 1e-3).bfloat16()
    w = awq.Int4Weight(nib, scales, None, G, torch.bfloat16, keep_reference=True)
    x = (torch.randn(T, K, device=DEV) * 0.5).bfloat16()
    y = awq.int4_linear(x, w, gated_act="gelu_tanh")
    dense = awq.dequantize(nib, scales, None, G)
    _close(y, ref.gated_linear(x, dense, "gelu_tanh", out_dtype=torch.float32), 4e-2, 3e-2, "int4 gated")
    # packing helpers are inverses; AutoAWQ layout converts to the same nibbles
    assert torch.equal(awq.unpack_nibbles(awq.pack_nibbles(nib)), nib)
    order = [0, 2, 4, 6, 1, 3, 5, 7]
    kn = nib.t().contiguous()                                   # [K, N]
    inter = kn.reshape(K, 2 * I // 8, 8)[:, :, order].reshape(K, 2 * I)
    back, s2, _ = awq.autoawq_to_rowmajor(awq.pack_nibbles(inter), scales.t().contiguous(), None)
    assert torch.equal(back, nib) and torch.equal(s2, scales)


def test_fused_collective_wait_is_bounded():
    """World of 2 emulated on one GPU with a peer that never signals: the kernel must give up after
    its cycle budget, report status 4 (peer timeout) and leave the context usable."""
    import ctypes
    from litevllm_b200.ops import _lib
    from litevllm_b200.parallel.symm import FiComm
    T, N, K = 8, 128, 64
    x = torch.randn(T, K, device=DEV).bfloat16()
    w = torch.randn(N, K, device=DEV).bfloat16()
    out = torch.zeros(T, N, device=DEV).bfloat16()
    recv = torch.zeros(2 * 2 * T * N, device=DEV, dtype=torch.float32)
    flags = torch.zeros(8192 * 8 * 8 // 64, device=DEV, dtype=torch.int32)   # tile 0 only is touched
    ready = torch.zeros(64, device=DEV, dtype=torch.int32)
    ctl = torch.zeros(64, device=DEV, dtype=torch.int32)
    c = FiComm()
    c.mode, c.world, c.rank, c.slab_elems = 1, 2, 0, T * N
    for d in range(2):
        c.recv[d], c.flags[d], c.ready[d] = recv.data_ptr(), flags.data_ptr(), ready.data_ptr()
    c.epoch, c.done = ctl.data_ptr(), ctl.data_ptr() + 64
    ops.status_word(x.device).zero_()
    rc = _lib.kernels().fi_dense_gemm_comm(x.data_ptr(), w.data_ptr(), out.data_ptr(), None, None, T, N, K,
                                           K, K, N, 0, 0, 0, 0, 1, 0, ops.status_word(x.device).data_ptr(),
                                           torch.cuda.current_stream().cuda_stream, ctypes.byref(c))
    assert rc == 0
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="status 4"):
        ops.check_status(x.device)
    # the context still works
    y = ops.linear(x, w)
    _close(y, ref.linear(x, w, out_dtype=torch.float32), 3e-2, 3e-2, "gemm after timeout")


@pytest.mark.parametrize("mode,E,K", [("softmax", 128, 8), ("sigmoid", 256, 6), ("sqrt_softplus", 64, 4), ("softmax", 8, 2)])
def test_moe_route(mode, E, K):
    from litevllm_b200.ops import moe
    torch.manual_seed(10)
    logits = torch.randn(37, E, device=DEV)
    bias = torch.randn(E, device=DEV) * 0.1 if mode != "softmax" else None
    scale = torch.rand(E, device=DEV) + 0.5 if mode == "softmax" else None
    ids, w = moe.route(logits, K, mode, bias, scale, True, 1.5)
    ids_r, w_r = moe.route(logits.cpu(), K, mode, None if bias is None else bias.cpu(),
                           None if scale is None else scale.cpu(), True, 1.5)
    assert torch.equal(ids.cpu().sort(-1).values, ids_r.sort(-1).values)
    order = ids.cpu().argsort(-1), ids_r.argsort(-1)
    _close(torch.gather(w.cpu(), 1, order[0]), torch.gather(w_r, 1, order[1]), 1e-4, 1e-5, "router weights")


@pytest.mark.parametrize("T,E,K,H,I,e_lo,e_n", [(1, 16, 4, 256, 128, 0, 16), (32, 16, 4, 512, 192, 0, 16),
                                                (200, 8, 2, 256, 704, 0, 8), (24, 16, 4, 256, 128, 4, 8)])
def test_fused_experts_int4(T, E, K, H, I, e_lo, e_n):
    from litevllm_b200.ops import awq, moe
    torch.manual_seed(11)
    G = 32
    x = (torch.randn(T, H, device=DEV) * 0.5).bfloat16()
    logits = torch.randn(T, E, device=DEV)
    ids, w = moe.route(logits, K, "softmax")

    def mk(rows, cols):
        nib = torch.randint(0, 16, (rows, cols), device=DEV, dtype=torch.uint8)
        sc = (torch.randn(rows, cols // G, device=DEV).abs() * 0.02 + 2e-3).bfloat16()
        return nib, sc
    gu_nib, gu_sc = mk(e_n * 2 * I, H)
    dn_nib, dn_sc = mk(e_n * H, I)
    wg = awq.Int4Weight(gu_nib, gu_sc, None, G, torch.bfloat16, keep_reference=True)
    wd = awq.Int4Weight(dn_nib, dn_sc, None, G, torch.bfloat16, keep_reference=True)
    y = moe.fused_experts(x, wg, wd, ids, w, e_n, e_lo, "gelu_tanh")
    wg_c = awq.Int4Weight(gu_nib.cpu(), gu_sc.cpu(), None, G, torch.bfloat16)
    wd_c = awq.Int4Weight(dn_nib.cpu(), dn_sc.cpu(), None, G, torch.bfloat16)
    yr = moe.fused_experts(x.cpu(), wg_c, wd_c, ids.cpu(), w.cpu(), e_n, e_lo, "gelu_tanh")
    _close(y.cpu(), yr, 5e-2, 5e-2, f"fused experts T{T} E{E}")
    ops.check_status(x.device)


@pytest.mark.parametrize("tname", ["Q8_0", "Q2_K", "IQ2_XXS", "Q4_0", "Q4_K", "Q6_K"])
def test_gguf_dequant_and_gemv(tname):
    from litevllm_b200.ops import gguf_quant as gq
    ty = gq.GGML_TYPES[tname]
    rows, K = 304, 1024
    raw = gq.random_blocks(ty, rows, K, seed=3, scale=0.02).to(DEV)
    want = gq.dequantize(raw.cpu(), ty, K)
    got = gq.dequantize_cuda(raw, ty, K, torch.bfloat16)
    _close(got.cpu(), want, 1e-2, 1e-3, f"dequant {tname}")
    for M in (1, 5, 8, 40):
        x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
        y = gq.gguf_linear(x, raw, ty, K, out_dtype=torch.float32)
        _close(y.cpu(), x.float().cpu() @ want.t(), 3e-2, 3e-2 * float(want.abs().max()) * 8, f"gemv {tname} M{M}")
    # the same bytes behind the weight interface: native path and (high-fidelity prefix) dense path
    from litevllm_b200.layers.quantization import tensor as qt
    w = qt.GGUFWeight(raw, tname, K, prefix="model.layers.0.mlp.down_proj")
    x = (torch.randn(6, K, device=DEV) * 0.5).bfloat16()
    ref_y = x.float().cpu() @ want.t()
    tol = 3e-2 * float(want.abs().max()) * 8
    _close(w.matmul(x, out_dtype=torch.float32).cpu(), ref_y, 3e-2, tol, f"GGUFWeight native {tname}")
    hf = qt.resolve_execution_policy(scope="all", high_fidelity_prefixes=("down_proj",))
    _close(w.matmul(x, policy=hf).float().cpu(), ref_y, 3e-2, tol, f"GGUFWeight dense {tname}")
    qt.clear_global_weight_cache()


def test_q8_0_quantize_roundtrip():
    from litevllm_b200.ops import gguf_quant as gq
    w = torch.randn(16, 256)
    raw = gq.quantize_q8_0(w)
    back = gq.dequantize(raw, 8, 256)
    assert float((back - w).abs().max()) < float(w.abs().max()) / 127 + 1e-3


@pytest.mark.parametrize("T,N,K,splits", [(32, 2560, 2048, 0), (1, 256, 512, 1), (7, 384, 1024, 4), (300, 512, 2048, 0),
                                          (64, 1024, 4096, 2)])
@pytest.mark.parametrize("gated", [False, True])
def test_gemm_with_fused_rmsnorm(T, N, K, splits, gated):
    """RMSNorm folded into the GEMM (norm weight in the weight columns, per-row scale taken from the
    token tiles in shared memory) vs norm-then-matmul in fp32."""
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(T * 7 + N)
    x = (torch.randn(T, K, generator=g, device=dev) * 3.0 + 0.5).bfloat16()
    gamma = (1.0 + 0.3 * torch.randn(K, generator=g, device=dev))
    rows = 2 * N if gated else N
    w = (torch.randn(rows, K, generator=g, device=dev) * 0.03).bfloat16()
    w_folded = (w.float() * gamma[None, :]).bfloat16()
    eps = 1e-5
    xn = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + eps)
    if gated:
        h = xn @ w_folded.float().t()
        want = torch.nn.functional.silu(h[:, :N]) * h[:, N:]
        got = ops.gated_linear(x, w_folded, "silu", splits=splits, rms_eps=eps)
    else:
        res = torch.randn(T, N, generator=g, device=dev).bfloat16()
        want = xn @ w_folded.float().t() + res.float()
        got = ops.linear(x, w_folded, None, res, splits=splits, rms_eps=eps)
    torch.cuda.synchronize()
    ops.check_status(dev)
    err = (got.float() - want).abs().max().item()
    assert err < 0.03 * max(1.0, want.abs().max().item()), err


def test_gemm_on_weights_written_by_the_previous_kernel():
    """A scratch weight matrix that is rewritten before every GEMM (the GGUF dequantise -> GEMM path for
    more than 8 rows): with programmatic dependent launch the GEMM must not read weight tiles before
    the dequantise kernel has finished, whatever the scratch held before."""
    from litevllm_b200.ops import gguf_quant as gq
    ty, rows, K, M = gq.GGML_TYPES["Q8_0"], 2048, 2048, 32
    x = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    raws = [gq.random_blocks(ty, rows, K, seed=10 + i, scale=0.02).to(DEV) for i in range(6)]
    wants = [x.float().cpu() @ gq.dequantize(r.cpu(), ty, K).t() for r in raws]
    for rep in range(3):
        outs = [gq.gguf_linear(x, r, ty, K, out_dtype=torch.float32) for r in raws]   # back to back, same scratch
        torch.cuda.synchronize()
        for i, (o, w) in enumerate(zip(outs, wants)):
            _close(o.cpu(), w, 3e-2, 0.5, f"dynamic weights rep {rep} matrix {i}")
    ops.check_status(DEV)


@pytest.mark.parametrize("T,nh,nkv,hd,K,eps", [(32, 32, 4, 64, 2048, 1e-5), (5, 8, 2, 128, 1024, 0.0), (64, 4, 4, 64, 512, 0.0)])
def test_qkv_gemm_with_rotary_and_cache_write_in_the_epilogue(T, nh, nkv, hd, K, eps):
    """One kernel (projection + rotary + cache write) against GEMM followed by the rotary/cache kernel."""
    dev = DEV
    g = torch.Generator(device=dev).manual_seed(T + nh)
    N = (nh + 2 * nkv) * hd
    x = (torch.randn(T, K, generator=g, device=dev) * 0.7).bfloat16()
    w = (torch.randn(N, K, generator=g, device=dev) * 0.03).bfloat16()
    bias = (torch.randn(N, generator=g, device=dev) * 0.1).bfloat16()
    bs, nblk = 16, 40
    cos_sin = ref.build_cos_sin(hd, 512, 10000.0).to(dev)
    positions = torch.randint(0, 500, (T,), generator=g, device=dev, dtype=torch.int32)
    slots = (torch.randperm(nblk * bs - bs, generator=g, device=dev)[:T] + bs).to(torch.int32)
    slots[0] = -1                                                    # a padded row: nothing is cached
    kc1, vc1 = torch.zeros(nblk, nkv, bs, hd, device=dev, dtype=torch.bfloat16), torch.zeros(nblk, nkv, bs, hd, device=dev, dtype=torch.bfloat16)
    kc2, vc2 = torch.zeros_like(kc1), torch.zeros_like(vc1)
    assert ops.qkv_rope_cache_supported(x, w, kc1, nh, nkv, hd, hd)
    got = ops.linear_rope_cache(x, w, bias, positions, cos_sin, slots, kc1, vc1, nh, nkv, hd, rms_eps=eps)
    want = ops.linear(x, w, bias, rms_eps=eps)
    ops.rope_and_cache(want, positions, cos_sin, slots, kc2, vc2, nh, nkv, hd, hd)
    torch.cuda.synchronize()
    ops.check_status(dev)
    _close(got.float().cpu(), want.float().cpu(), 3e-2, 3e-2, "qkv buffer")
    _close(kc1.float().cpu(), kc2.float().cpu(), 3e-2, 3e-2, "k cache")
    _close(vc1.float().cpu(), vc2.float().cpu(), 3e-2, 3e-2, "v cache")
    assert float(kc1[0].abs().max()) == 0.0                          # the null block stays untouched


def test_native_sampler_thresholds_and_distribution():
    """The sampling kernel against the sort-based definition: with top-k / top-p / min-p the drawn token
    must lie in the kept set, the empirical distribution over many uniform numbers must match the
    renormalised probabilities, greedy rows return the arg-max, and a fixed uniform number is reproducible."""
    dev = torch.device(DEV, 0)
    g = torch.Generator(device=dev).manual_seed(3)
    V, n = 1000, 4096
    base = torch.randn(V, generator=g, device=dev) * 2.0
    logits = base[None, :].expand(n, V).contiguous()
    temp, k, p, mp = 0.7, 50, 0.8, 0.02
    scaled = base / temp
    srt, idx = torch.sort(scaled, descending=True)
    mask = torch.arange(V, device=dev) >= k
    probs = torch.softmax(srt.masked_fill(mask, float("-inf")), -1)
    cum = probs.cumsum(-1)
    mask |= (cum - probs) >= p
    mask |= probs < mp * probs[0]
    mask[0] = False
    final = torch.softmax(srt.masked_fill(mask, float("-inf")), -1)
    want = torch.zeros(V, device=dev)
    want[idx] = final
    u = torch.rand(n, generator=g, device=dev)
    args = (torch.full((n,), temp, device=dev), torch.full((n,), k, device=dev, dtype=torch.int32),
            torch.full((n,), p, device=dev), torch.full((n,), mp, device=dev))
    tok = ops.sample(logits, *args, u)
    assert bool((want[tok] > 0).all()), "a token outside the kept set was drawn"
    freq = torch.bincount(tok, minlength=V).float() / n
    assert float((freq - want).abs().max()) < 0.03
    assert torch.equal(tok, ops.sample(logits, *args, u))                      # same numbers, same tokens
    greedy = ops.sample(logits[:8], torch.zeros(8, device=dev), args[1][:8], args[2][:8], args[3][:8], u[:8])
    assert torch.equal(greedy, torch.full((8,), int(base.argmax()), device=dev))
    # no filters: plain temperature sampling over the whole vocabulary
    off = (torch.ones(n, device=dev), torch.zeros(n, device=dev, dtype=torch.int32), torch.ones(n, device=dev),
           torch.zeros(n, device=dev))
    tok = ops.sample(logits, *off, u)
    freq = torch.bincount(tok, minlength=V).float() / n
    assert float((freq - torch.softmax(base, -1)).abs().max()) < 0.03


@pytest.mark.parametrize("T,N,K", [(1024, 256, 512), (1500, 2560, 2048), (4096, 640, 1088), (2048, 129 * 8, 72)])
@pytest.mark.parametrize("mode", ["plain", "bias_residual", "gated"])
def test_persistent_prefill_gemm(T, N, K, mode):
    """The persistent double-accumulator GEMM (prefill sizes) against fp32 matmul, including ragged token
    and row counts and more tiles than SMs."""
    dev = torch.device(DEV, 0)
    g = torch.Generator(device=dev).manual_seed(T + N + K)
    x = (torch.randn(T, K, generator=g, device=dev) * 0.5).bfloat16()
    if mode == "gated":
        w = (torch.randn(2 * N, K, generator=g, device=dev) * 0.05).bfloat16()
        h = x.float() @ w.float().t()
        want = torch.nn.functional.silu(h[:, :N]) * h[:, N:]
        got = ops.gated_linear(x, w, "silu")
    else:
        w = (torch.randn(N, K, generator=g, device=dev) * 0.05).bfloat16()
        bias = (torch.randn(N, generator=g, device=dev) * 0.1).bfloat16() if mode == "bias_residual" else None
        res = torch.randn(T, N, generator=g, device=dev).bfloat16() if mode == "bias_residual" else None
        want = x.float() @ w.float().t()
        if bias is not None:
            want = want + bias.float() + res.float()
        import litevllm_b200.ops as O
        saved, O._PERSISTENT_PLAIN = O._PERSISTENT_PLAIN, True      # plain products take this kernel only on request
        try:
            got = ops.linear(x, w, bias, res)
        finally:
            O._PERSISTENT_PLAIN = saved
    torch.cuda.synchronize()
    ops.check_status(dev)
    err = (got.float() - want).abs().max().item()
    assert err < 0.03 * max(1.0, want.abs().max().item()), err


def test_fused_collective_epilogue_loopback_world1():
    """The collective epilogue of the tcgen05 GEMMs on ONE GPU (world size 1, the rank is its own and
    only peer): all three transfer formats of GEMM->all-reduce and the reduce-scatter form must equal
    GEMM + residual.  Covers the tile/flag/epoch logic without NVLink."""
    import os
    import torch.distributed as dist
    from litevllm_b200.parallel import fused_ops, state as pstate
    from litevllm_b200.parallel.symm import SymmetricHeap
    dev = torch.device(DEV, 0)
    created = False
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29671")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
        created = True
    saved = pstate._STATE
    heap = None
    try:
        st = pstate.ParallelState(rank=0, world_size=1, tp_size=1, ep_size=1, local_rank=0, comm_backend="fused",
                                  group=dist.group.WORLD)
        pstate._STATE = st
        heap = st.symm = SymmetricHeap(0, 1, dev, recv_bytes=64 << 20, xbuf_bytes=8 << 20)

        class L:
            quant_method, bias = None, None

        g = torch.Generator(device=dev).manual_seed(21)
        for T, N, K in [(32, 512, 256), (300, 384, 320), (1024, 256, 128)]:
            x = (torch.randn(T, K, generator=g, device=dev) * 0.5).bfloat16()
            w = (torch.randn(N, K, generator=g, device=dev) * 0.05).bfloat16()
            res = torch.randn(T, N, generator=g, device=dev).bfloat16()
            want = x.float() @ w.float().t() + res.float()
            layer = L()
            layer.weight, layer.out_features = w, N
            for mode in ([2, 0] if T <= 256 else [1]):
                for _ in range(2):      # both slab parities
                    got = fused_ops._fused_gemm_allreduce(layer, x, res, None, heap, mode)
                _close(got.float(), want, 3e-2, 3e-2, f"loopback all-reduce T{T} mode{mode}")
            if T % 128 == 0:
                got = fused_ops.gemm_reduce_scatter(x, w, res, T)
                _close(got.float(), want, 3e-2, 3e-2, f"loopback reduce-scatter T{T}")
        torch.cuda.synchronize()
        ops.check_status(dev)
        assert heap.epoch_value() > 0
    finally:
        pstate._STATE = saved
        if heap is not None:
            heap.close()
        if created:
            dist.destroy_process_group()


@pytest.mark.parametrize("tg,td", [("IQ2_XXS", "Q2_K"), ("Q8_0", "Q8_0"), ("Q2_K", "IQ2_XXS")])
@pytest.mark.parametrize("T", [3, 40])
def test_gguf_routed_experts_grouped_and_per_route(tg, td, T):
    """Routed experts stored as GGUF blocks: the per-route kernels and the expert-grouped kernels (routes
    sorted by expert, every tile of up to 8 routes streams its expert once) against the dequantise-and-matmul
    oracle, for few routes (every expert hit at most once or twice) and many (ragged tiles, several per expert)."""
    import litevllm_b200.models.deepseek_mla as dm
    from litevllm_b200.loaders.gguf import GGUFTensor
    from litevllm_b200.models.arch import arch_from_hf_config
    from litevllm_b200.models.presets import get_preset
    from litevllm_b200.ops import gguf_quant as gq
    arch = arch_from_hf_config(get_preset("tiny-deepseek-test"))
    E, I, H, K = arch.moe.num_experts, arch.moe.expert_intermediate, arch.hidden_size, arch.moe.top_k
    dev = torch.device(DEV, 0)
    with torch.device(dev):
        ex = dm.RoutedExperts(arch, torch.bfloat16)
    ex.device = dev
    tyg, tyd = gq.GGML_TYPES[tg], gq.GGML_TYPES[td]
    ex.load("gate", GGUFTensor(gq.random_blocks(tyg, E * I, H, seed=21, scale=0.05).view(E, I, -1), tyg, (E, I, H)))
    ex.load("up", GGUFTensor(gq.random_blocks(tyg, E * I, H, seed=22, scale=0.05).view(E, I, -1), tyg, (E, I, H)))
    ex.load("down", GGUFTensor(gq.random_blocks(tyd, E * H, I, seed=23, scale=0.05).view(E, H, -1), tyd, (E, H, I)))
    g = torch.Generator(device=dev).manual_seed(T)
    x = torch.randn(T, H, generator=g, device=dev).bfloat16()
    ids = torch.stack([torch.randperm(E, generator=g, device=dev)[:K] for _ in range(T)]).to(torch.int32)
    w = torch.rand(T, K, generator=g, device=dev)
    outs = {}
    saved = dm._GROUPED, dm._Q8
    try:
        dm._Q8 = False
        for mode in ("off", "on"):
            dm._GROUPED = mode
            outs[mode] = ex(x, ids, w).float()
        dm._Q8, dm._GROUPED = True, "auto"
        outs["q8"] = ex(x, ids, w).float()       # int8 activations (the 2-bit formats; Q8_0 keeps the float path)
        dense_saved, dm._DENSE_EXPERT_ROUTES = dm._DENSE_EXPERT_ROUTES, 1
        try:
            outs["tensor_core"] = ex(x, ids, w).float()     # every expert dequantised once, tcgen05 GEMMs
        finally:
            dm._DENSE_EXPERT_ROUTES = dense_saved
    finally:
        dm._GROUPED, dm._Q8 = saved
    torch.cuda.synchronize()
    cpu = dm.RoutedExperts.__new__(dm.RoutedExperts)
    cpu.__dict__.update(ex.__dict__)
    cpu.raw = {k: v.cpu() for k, v in ex.raw.items()}
    want = dm.RoutedExperts.forward(cpu, x.cpu(), ids.cpu().long(), w.cpu()).float()
    for mode, got in outs.items():
        err = (got.cpu() - want).abs().max().item()
        assert err < 0.03 * max(1.0, want.abs().max().item()), (mode, err, want.abs().max().item())
    assert (outs["on"] - outs["off"]).abs().max().item() < 0.02 * max(1.0, want.abs().max().item())


def test_gguf_dense_layer_resident_copy_budget(monkeypatch):
    """A GGUF linear layer keeps its blocks when the budget for 16-bit copies is zero and swaps them for a
    dense weight (same results within rounding) when there is room."""
    from litevllm_b200.layers.linear import LiteLinear
    from litevllm_b200.layers.quantization import gguf as gl
    from litevllm_b200.loaders.gguf import GGUFTensor
    from litevllm_b200.ops import gguf_quant as gq
    dev = torch.device(DEV, 0)
    N, K = 384, 512
    raw = gq.random_blocks(gq.GGML_TYPES["Q8_0"], N, K, seed=5, scale=0.05)
    x = torch.randn(5, K, device=dev).bfloat16()
    outs = {}
    for budget in ("0", "1"):
        monkeypatch.setenv("FI_GGUF_DENSE_RESIDENT_GB", budget)
        monkeypatch.setattr(gl, "_resident_used", [0])
        with torch.device(dev):
            layer = LiteLinear(K, N, dtype=torch.bfloat16, quant_config=gl.GGUFConfig(), prefix="blk.0.attn_q")
        layer.quant_method.load_piece(layer, 0, "weight", GGUFTensor(raw, gq.GGML_TYPES["Q8_0"], (N, K)), (0, N))
        outs[budget] = layer(x).float()
        assert (layer.g_raw is None) == (budget == "1") and (layer.weight is not None) == (budget == "1")
    want = x.float().cpu() @ gq.dequantize(raw, gq.GGML_TYPES["Q8_0"], K).t()
    for k, got in outs.items():
        assert (got.cpu() - want).abs().max().item() < 0.03 * max(1.0, want.abs().max().item()), k


def test_select_blocks_kernel_and_sparse_decode():
    """The block-selection kernel against its CPU form, and decode attention over the compact table against
    the fp32 oracle evaluated on exactly the kept tokens."""
    torch.manual_seed(31)
    nh, nkv, hd, bs = 8, 2, 64, 16
    lens = [16 * 9 + 5, 7, 16 * 40, 33]
    B = len(lens)
    kc, vc, bt = _fill_paged(B, lens, nkv, hd, bs, False)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    tab, sel_len = ops.select_blocks(bt, sl, bs, 4, 2)
    tab_c, len_c = ops.select_blocks(bt.cpu(), sl.cpu(), bs, 4, 2)
    assert torch.equal(tab.cpu(), tab_c) and torch.equal(sel_len.cpu(), len_c)
    q = torch.randn(B, nh * hd, device=DEV).bfloat16()
    scale = 1.0 / math.sqrt(hd)
    y = ops.paged_attention_decode(q, kc, vc, tab, sel_len, nh, nkv, hd, scale, 0, 0.0, 1.0, 1.0,
                                   max_kv_len=max(lens))
    cu = torch.arange(B + 1, dtype=torch.int32, device=DEV)
    yr = ref.paged_attention(q, kc, vc, tab, sel_len, cu, nh, nkv, hd, scale, 0, 0.0, 1.0, 1.0, out_dtype=torch.float32)
    _close(y, yr, 2e-2, 2e-2, "sparse decode over the compact table")
    assert sel_len.tolist()[2] < lens[2] // 2


@pytest.mark.parametrize("nh,splits", [(20, 1), (64, 1), (16, 3), (40, 5)])
def test_mla_absorbed_decode_kernel(nh, splits):
    """The latent-space attention kernel (576-value cache rows shared by all heads, the first 512 values are
    also the value) against fp32 PyTorch: several 64-row chunks, ragged lengths, head counts that do not fill
    a 16-row tile, one launch and split launches with the merge, rows that share a block table."""
    from litevllm_b200.ops import _lib, _p, _stream
    torch.manual_seed(nh + splits)
    dev = torch.device(DEV, 0)
    bs, nb, KD, VD = 16, 100, 576, 512
    lens = [1, 70, 300, 129, 64]
    seq_of_row = [0, 1, 2, 2, 3]                 # rows 2 and 3 read the same sequence with different lengths
    max_blocks = 20
    cache = (torch.randn(nb, 1, bs, KD, device=dev) * 0.5).bfloat16()
    bt = torch.zeros(4, max_blocks, dtype=torch.int32, device=dev)
    perm = torch.randperm(nb - 1, device=dev)[: 4 * max_blocks].view(4, max_blocks) + 1
    bt.copy_(perm.to(torch.int32))
    rows = len(lens)
    q = (torch.randn(rows, nh, KD, device=dev) * 0.3).bfloat16()
    row_lens = torch.tensor(lens, dtype=torch.int32, device=dev)
    sor = torch.tensor(seq_of_row, dtype=torch.int32, device=dev)
    out = torch.zeros(nh, rows, VD, dtype=torch.bfloat16, device=dev)
    ws_o = torch.empty(rows * nh * splits * VD, dtype=torch.float32, device=dev) if splits > 1 else None
    ws_ml = torch.empty(rows * nh * splits * 2, dtype=torch.float32, device=dev) if splits > 1 else None
    scale = 192 ** -0.5
    rc = _lib.kernels().fi_mla_decode(_p(q), _p(cache), _p(out), out.stride(0), out.stride(1), _p(bt), _p(row_lens),
                                      _p(sor), _p(ws_o), _p(ws_ml), rows, nh, max_blocks, bs, splits, scale, 0, _stream())
    assert rc == 0
    torch.cuda.synchronize()
    flat = cache.view(nb * bs, KD).float()
    for r in range(rows):
        idx = torch.tensor([int(bt[seq_of_row[r], t // bs]) * bs + t % bs for t in range(lens[r])], device=dev)
        k = flat[idx]
        p = torch.softmax(q[r].float() @ k.t() * scale, dim=-1)
        want = p @ k[:, :VD]
        got = out[:, r].float()
        assert (got - want).abs().max().item() < 0.02 * max(1.0, want.abs().max().item()), (r, nh, splits)
