"""DeepSeek-V4-Flash building blocks: batched PyTorch forms against literal per-element restatements
(CPU), native kernels against the PyTorch forms (GPU)."""
import math

import pytest
import torch

from litevllm_b200.models import deepseek_v4_flash as v4


def _hadamard_loops(row):
    out = row.clone().double()
    stride = 1
    while stride < 128:
        for base in range(0, 128, 2 * stride):
            l, r = out[base:base + stride].clone(), out[base + stride:base + 2 * stride].clone()
            out[base:base + stride], out[base + stride:base + 2 * stride] = l + r, l - r
        stride <<= 1
    return (out / math.sqrt(128)).float()


def test_hadamard_and_e2m1_roundtrip():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(3, 128, generator=g)
    h = v4.hadamard128(x)
    for i in range(3):
        assert torch.allclose(h[i], _hadamard_loops(x[i]), atol=1e-5)
    assert torch.allclose(v4.hadamard128(h), x, atol=1e-4)            # involution up to the scale
    q = v4.e2m1_roundtrip(torch.tensor([[0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0] + [0.0] * 24]))
    assert q[0, :8].tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0]   # ties go to the even code
    y = v4.indexer_qat(x)
    assert y.shape == x.shape and float((y - h).abs().max()) <= float(h.abs().max()) * 0.26


def test_fp8_and_q8k_roundtrips():
    g = torch.Generator().manual_seed(1)
    row = torch.randn(2, 512, generator=g) * 3
    out = v4.fp8_kv_qat(row, head_dim=512, rotary_dim=64)
    assert torch.equal(out[:, 448:], row[:, 448:])                         # rotary tail untouched
    assert float((out[:, :448] - row[:, :448]).abs().max()) < 0.07 * float(row.abs().max())
    r = v4.q8_k_roundtrip(row)
    assert float((r - row).abs().max()) <= float(row.abs().max()) / 127 + 1e-6


def test_hyper_connection_shapes_and_doubly_stochastic_mix():
    g = torch.Generator().manual_seed(2)
    T, hc, H = 3, 4, 32
    streams = torch.randn(T, hc, H, generator=g)
    n_mix = 2 * hc + hc * hc
    st = v4.hyper_connection_pre(streams, torch.randn(hc * H, n_mix, generator=g) * 0.1,
                                 torch.randn(n_mix, generator=g) * 0.1, torch.tensor([1.0, 0.5, 2.0]))
    assert st.mixed.shape == (T, H) and st.post.shape == (T, hc) and st.combine.shape == (T, hc, hc)
    assert torch.allclose(st.combine.sum(-1), torch.ones(T, hc), atol=5e-2)   # rows: approximately
    assert torch.allclose(st.combine.sum(-2), torch.ones(T, hc), atol=1e-2)
    new = v4.hyper_connection_post(torch.randn(T, H, generator=g), streams, st)
    assert new.shape == (T, hc, H)
    # one token equals the batched result
    one = v4.hyper_connection_pre(streams[1:2], *[torch.zeros(hc * H, n_mix), torch.zeros(n_mix), torch.ones(3)])
    assert torch.allclose(one.post, torch.ones(1, hc), atol=1e-6)         # 2 * sigmoid(0)


def test_shared_kv_attention_sinks_and_index_paths():
    g = torch.Generator().manual_seed(3)
    q, rows = torch.randn(4, 128, generator=g), torch.randn(40, 128, generator=g)
    sinks = torch.randn(4, generator=g)
    out = v4.shared_kv_attention(q, rows, sinks)
    logits = torch.cat([q @ rows.t() / math.sqrt(128), sinks[:, None]], 1)
    want = torch.softmax(logits, -1)[:, :-1] @ rows
    assert torch.allclose(out, want, atol=1e-5)
    sel = torch.tensor([3, 7, 39])
    assert torch.allclose(v4.compressed_row_attention(q, rows, sel), v4.shared_kv_attention(q, rows[sel]), atol=1e-6)
    table = torch.tensor([2, 0, 1], dtype=torch.int32)                     # 3 pages of 16 rows
    pool = torch.zeros(48, 128)
    v4.update_latent_cache(pool, rows[:40], torch.arange(40, dtype=torch.int32), table, 16)
    paged = v4.shared_kv_attention(q, pool, sinks, row_index=torch.arange(40, dtype=torch.int32), page_table=table,
                                   page_rows=16)
    assert torch.allclose(paged, want, atol=1e-5)


def test_indexer_scores_router_and_compressor():
    g = torch.Generator().manual_seed(4)
    iq, iw, rows = torch.randn(8, 128, generator=g), torch.rand(8, generator=g), torch.randn(20, 128, generator=g)
    s = v4.indexer_scores(iq, iw, rows)
    want = torch.stack([(iw * (iq @ rows[r]).clamp_min(0)).sum() for r in range(20)]) / math.sqrt(8 * 128)
    assert torch.allclose(s, want, atol=1e-5) and v4.indexer_topk(s, 5).tolist() == want.topk(5).indices.tolist()
    ids, w = v4.sqrt_softplus_router(torch.randn(3, 16, generator=g), torch.randn(12, 16, generator=g), 4,
                                     correction_bias=torch.zeros(12))
    assert ids.shape == (3, 4) and torch.allclose(w.sum(-1), torch.full((3,), 1.5), atol=1e-5)
    table = torch.randint(0, 12, (4, 50), generator=g)
    assert v4.hash_routed_expert_ids(table, torch.tensor([7, 49])).tolist() == table[:, [7, 49]].t().tolist()
    with pytest.raises(ValueError):
        v4.hash_routed_expert_ids(table, torch.tensor([50]))
    # ratio 128-style (single window) compressor with ratio 2: emits the softmax-weighted mean every 2 tokens
    st = v4.CompressorState.empty(4, 2)
    kvs, scs, ape = torch.randn(4, 4, generator=g), torch.randn(4, 4, generator=g), torch.zeros(2, 4)
    st, e0 = v4.compressor_step(st, kvs[0], scs[0], ape, 0, 4, 2)
    st, e1 = v4.compressor_step(st, kvs[1], scs[1], ape, 1, 4, 2)
    assert e0 is None and torch.allclose(e1, (torch.softmax(scs[:2], 0) * kvs[:2]).sum(0), atol=1e-6)
    # ratio 4 keeps two overlapping windows of double width
    st4 = v4.CompressorState.empty(4, 4)
    emitted = []
    for t in range(8):
        st4, e = v4.compressor_step(st4, torch.randn(8, generator=g), torch.randn(8, generator=g), torch.zeros(4, 8), t, 4, 4)
        emitted.append(e)
    assert [e is not None for e in emitted] == [False, False, False, True] * 2 and emitted[7].shape == (4,)


@pytest.mark.gpu
def test_native_kernels_match_torch_forms():
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(5)
    x = torch.randn(37, 128, generator=g)
    assert torch.allclose(v4.indexer_qat(x.to(dev)).cpu(), v4.indexer_qat(x), atol=1e-5)
    q, rows, sinks = torch.randn(64, 512, generator=g), torch.randn(200, 512, generator=g), torch.randn(64, generator=g)
    want = v4.shared_kv_attention(q, rows, sinks)
    got = v4.shared_kv_attention(q.to(dev), rows.to(dev), sinks.to(dev))
    assert torch.allclose(got.cpu(), want, atol=2e-4)
    sel = torch.randperm(200, generator=g)[:77].to(torch.int32)
    got = v4.compressed_row_attention(q.to(dev), rows.to(dev), sel.to(dev), sinks.to(dev))
    assert torch.allclose(got.cpu(), v4.compressed_row_attention(q, rows, sel, sinks), atol=2e-4)
    table = torch.randperm(16, generator=g).to(torch.int32)
    pool = torch.zeros(16 * 16, 512, device=dev)
    v4.update_latent_cache(pool, rows.to(dev), torch.arange(200, dtype=torch.int32, device=dev), table.to(dev), 16)
    got = v4.shared_kv_attention(q.to(dev), pool, sinks.to(dev), row_index=torch.arange(200, dtype=torch.int32, device=dev),
                                 page_table=table.to(dev), page_rows=16)
    assert torch.allclose(got.cpu(), want, atol=2e-4)
    iq, iw, crow = torch.randn(64, 128, generator=g), torch.rand(64, generator=g), torch.randn(1000, 128, generator=g)
    assert torch.allclose(v4.indexer_scores(iq.to(dev), iw.to(dev), crow.to(dev)).cpu(), v4.indexer_scores(iq, iw, crow),
                          atol=1e-3, rtol=1e-4)
