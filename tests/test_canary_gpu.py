"""Out-of-bounds writes, caught without a memory checker: every kernel writes into a view that sits
inside a larger buffer pre-filled with a sentinel; after the call the guard region must still hold
the sentinel.  Shapes are ragged on purpose (token counts, row counts and row pitches that are not
multiples of the tile sizes)."""
import math

import pytest
import torch

from litevllm_b200 import ops
from litevllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"
SENTINEL = -1024.0      # exactly representable in bf16 and fp16


class Guarded:
    """A [rows, cols] output view with ``pad`` guard rows above/below and guard columns to the right."""

    def __init__(self, rows, cols, dtype, pad_rows=3, pad_cols=8):
        self.buf = torch.full((rows + 2 * pad_rows, cols + pad_cols), SENTINEL, dtype=dtype, device=DEV)
        self.view = self.buf[pad_rows:pad_rows + rows, :cols]
        self.r0, self.rows, self.cols = pad_rows, rows, cols

    def intact(self) -> bool:
        b = self.buf.float()
        ok = bool((b[:self.r0] == SENTINEL).all()) and bool((b[self.r0 + self.rows:] == SENTINEL).all())
        return ok and bool((b[:, self.cols:] == SENTINEL).all())


def test_dense_gemm_variants_stay_inside_their_output():
    g = torch.Generator(device=DEV).manual_seed(1)
    for T, N, K in [(1, 136, 72), (19, 264, 320), (33, 1032, 256), (150, 520, 128)]:
        x = (torch.randn(T, K, generator=g, device=DEV) * 0.5).bfloat16()
        w = (torch.randn(N, K, generator=g, device=DEV) * 0.05).bfloat16()
        res = torch.randn(T, N, generator=g, device=DEV).bfloat16()
        for splits in (0, 1, 3):
            out = Guarded(T, N, torch.bfloat16)
            ops.linear(x, w, residual=res, out=out.view, splits=splits)
            torch.cuda.synchronize()
            assert out.intact(), f"linear T{T} N{N} K{K} splits{splits} wrote outside its output"
            want = x.float() @ w.float().t() + res.float()
            assert float((out.view.float() - want).abs().max()) < 0.05 * max(1.0, float(want.abs().max()))
        if K % 64 == 0:
            out = Guarded(T, N, torch.bfloat16)
            ops.linear(x, w, out=out.view, rms_eps=1e-5)
            torch.cuda.synchronize()
            assert out.intact(), f"rmsnorm-fused linear T{T} N{N}"
        if N % 16 == 0:
            out = Guarded(T, N // 2, torch.bfloat16)
            ops.gated_linear(x, w, "silu", out=out.view, rms_eps=1e-5 if K % 64 == 0 else 0.0)
            torch.cuda.synchronize()
            assert out.intact(), f"gated linear T{T} N{N}"
    ops.check_status(torch.device(DEV, 0))


def test_int4_gemm_stays_inside_its_output():
    from litevllm_b200.ops import awq
    g = torch.Generator(device=DEV).manual_seed(2)
    for T, N, K, G in [(3, 136, 256, 128), (40, 264, 128, 32)]:
        nib = torch.randint(0, 16, (N, K), generator=g, device=DEV, dtype=torch.uint8)
        sc = (torch.rand(N, K // G, generator=g, device=DEV) * 0.01 + 0.001).bfloat16()
        zp = torch.randint(0, 16, (N, K // G), generator=g, device=DEV, dtype=torch.uint8) if G == 128 else None
        w = awq.Int4Weight(nib, sc, zp, G, torch.bfloat16)
        x = (torch.randn(T, K, generator=g, device=DEV) * 0.5).bfloat16()
        out = Guarded(T, N, torch.bfloat16)
        awq.int4_linear(x, w, out=out.view)
        torch.cuda.synchronize()
        assert out.intact(), f"int4 GEMM T{T} N{N}"
    ops.check_status(torch.device(DEV, 0))


def test_small_ops_stay_inside_their_outputs():
    g = torch.Generator(device=DEV).manual_seed(3)
    T, H = 37, 264
    x = torch.randn(T, H, generator=g, device=DEV).bfloat16()
    w = torch.randn(H, generator=g, device=DEV).bfloat16()
    out = Guarded(T, H, torch.bfloat16)
    ops.rmsnorm(x, w, 1e-5, out=out.view)
    table = torch.randn(100, H, generator=g, device=DEV).bfloat16()
    ids = torch.randint(0, 100, (T,), generator=g, device=DEV)
    emb = Guarded(T, H, torch.bfloat16, pad_cols=0)
    emb_out = emb.view
    ops.embedding(ids, table, out=emb_out if emb_out.is_contiguous() else None)
    act = Guarded(T, H // 2, torch.bfloat16)
    ops.act_mul(x, "silu", out=act.view if act.view.is_contiguous() else None)
    torch.cuda.synchronize()
    assert out.intact() and emb.intact() and act.intact()
    # arg-max writes exactly `rows` int64 values
    logits = torch.randn(T, 1000, generator=g, device=DEV)
    ids_buf = torch.full((T + 16,), -7, dtype=torch.int64, device=DEV)
    ops.argmax(logits, out=ids_buf[8:8 + T])
    torch.cuda.synchronize()
    assert bool((ids_buf[:8] == -7).all()) and bool((ids_buf[8 + T:] == -7).all())
    assert torch.equal(ids_buf[8:8 + T], logits.argmax(-1))
    # block-table row gather
    tab = torch.randint(0, 50, (9, 21), generator=g, device=DEV, dtype=torch.int32)
    idx = torch.tensor([4, 0, 8, 8, 2], device=DEV, dtype=torch.int32)
    gb = torch.full((5 + 4, 21), -7, dtype=torch.int32, device=DEV)
    ops.gather_rows_i32(tab, idx, gb[2:7])
    torch.cuda.synchronize()
    assert torch.equal(gb[2:7], tab[idx.long()]) and bool((gb[:2] == -7).all()) and bool((gb[7:] == -7).all())


def test_attention_and_cache_writes_stay_inside():
    torch.manual_seed(9)
    nh, nkv, hd, bs = 8, 2, 64, 16
    lens = [1, 17, 130, 64, 33]
    B = len(lens)
    max_blocks = (max(lens) + bs - 1) // bs + 1
    nb = 1 + B * max_blocks
    # the cache itself is a guarded view: blocks 0..1 and nb+2.. are guard blocks
    kbuf = torch.full((nb + 4, nkv, bs, hd), SENTINEL, dtype=torch.bfloat16, device=DEV)
    vbuf = kbuf.clone()
    kc, vc = kbuf[2:2 + nb], vbuf[2:2 + nb]
    kc.copy_(torch.randn(nb, nkv, bs, hd, device=DEV) * 0.5)
    vc.copy_(torch.randn(nb, nkv, bs, hd, device=DEV) * 0.5)
    bt = torch.zeros(B, max_blocks, dtype=torch.int32, device=DEV)
    perm = torch.randperm(nb - 1, device=DEV) + 1
    used = 0
    for b in range(B):
        n = (lens[b] + bs - 1) // bs
        bt[b, :n] = perm[used:used + n].to(torch.int32)
        used += n
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(hd)
    # cache write of the newest token of every sequence (+ one skipped row)
    qkv = torch.randn(B + 1, (nh + 2 * nkv) * hd, device=DEV).bfloat16()
    pos = torch.tensor([l - 1 for l in lens] + [5], dtype=torch.int32, device=DEV)
    slots = torch.tensor([int(bt[b, (lens[b] - 1) // bs]) * bs + (lens[b] - 1) % bs for b in range(B)] + [-1],
                         dtype=torch.int32, device=DEV)
    cs = ref.build_cos_sin(hd, 256, 10000.0).to(DEV)
    ops.rope_and_cache(qkv, pos, cs, slots, kc, vc, nh, nkv, hd, hd)
    for splits in (1, 2, 3):
        out = Guarded(B, nh * hd, torch.bfloat16, pad_cols=0)      # contiguous rows: guard rows above and below
        ops.paged_attention_decode(qkv[:B], kc, vc, bt, sl, nh, nkv, hd, scale, out=out.view, splits=splits,
                                   max_kv_len=max(lens))
        torch.cuda.synchronize()
        assert out.intact(), f"decode attention splits {splits}"
    torch.cuda.synchronize()
    for buf in (kbuf, vbuf):
        assert bool((buf[:2].float() == SENTINEL).all()) and bool((buf[2 + nb:].float() == SENTINEL).all()), \
            "cache write left the pool"
    ops.check_status(torch.device(DEV, 0))


def test_mrope_three_position_streams():
    """Multimodal rotary embedding: every frequency takes its angle from one of three position streams
    (time / height / width); the streams here are all different."""
    torch.manual_seed(12)
    nh, nkv, hd, rot, bs, nb, T = 8, 2, 128, 128, 16, 9, 29
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV).bfloat16()
    pos = torch.stack([torch.randint(0, 300, (T,)), torch.randint(0, 40, (T,)), torch.randint(0, 40, (T,))]).to(
        device=DEV, dtype=torch.int32).contiguous()
    sections = [16, 24, 24]                                      # half = 64 frequencies: t, h, w
    fs = torch.cat([torch.full((n,), i) for i, n in enumerate(sections)]).to(device=DEV, dtype=torch.int32)
    cs = ref.build_cos_sin(rot, 512, 10000.0).to(DEV)
    slots = (torch.randperm((nb - 1) * bs, device=DEV)[:T] + bs).to(torch.int32)
    kc = torch.zeros(nb, nkv, bs, hd, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    kcr, vcr = kc.clone(), vc.clone()
    a, b = qkv.clone(), qkv.clone()
    ops.rope_and_cache(a, pos, cs, slots, kc, vc, nh, nkv, hd, rot, freq_stream=fs)
    ref.rope_and_cache(b, pos, cs, slots, kcr, vcr, nh, nkv, hd, rot, freq_stream=fs)
    assert float((a.float() - b.float()).abs().max()) < 3e-2
    assert float((kc.float() - kcr.float()).abs().max()) < 3e-2 and float((vc.float() - vcr.float()).abs().max()) < 3e-2
    # and it differs from the single-stream rotation (the streams really are used)
    c = qkv.clone()
    ops.rope_and_cache(c, pos[0].contiguous(), cs, slots, kc.clone(), vc.clone(), nh, nkv, hd, rot)
    assert float((a.float() - c.float()).abs().max()) > 0.1
