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


def test_compressor_run_matches_token_by_token():
    """A run of tokens pooled at once gives the rows, and leaves the state, of feeding them one at a time."""
    from litevllm_b200.models.deepseek_v4_flash import native as nv
    from litevllm_b200.models.deepseek_v4_flash.attention import CompressorState, compressor_step
    g = torch.Generator().manual_seed(0)
    for ratio, D in ((4, 16), (8, 16), (3, 8)):
        width = (2 if ratio == 4 else 1) * D
        ape = torch.randn(ratio, width, generator=g)
        for p0, n in ((0, 11), (0, 3), (5, 9), (7, 1), (6, 20), (2, 2)):
            one, run = CompressorState.empty(D, ratio), CompressorState.empty(D, ratio)
            kvs, scs = torch.randn(p0 + n, width, generator=g), torch.randn(p0 + n, width, generator=g)
            for t in range(p0):
                one, _ = compressor_step(one, kvs[t], scs[t], ape, t, D, ratio)
                run, _ = compressor_step(run, kvs[t], scs[t], ape, t, D, ratio)
            want = []
            for t in range(p0, p0 + n):
                one, e = compressor_step(one, kvs[t], scs[t], ape, t, D, ratio)
                if e is not None:
                    want.append(e)
            got = nv.compressor_run_(run, kvs[p0:], scs[p0:], ape, p0, D, ratio)
            assert got.shape[0] == len(want)
            if want:
                torch.testing.assert_close(got, torch.stack(want))
            more = torch.randn(2, 2 * ratio, width, generator=g)
            for i in range(2 * ratio):           # both continue token by token: the next windows agree as well
                one, ea = compressor_step(one, more[0, i], more[1, i], ape, p0 + n + i, D, ratio)
                run, eb = compressor_step(run, more[0, i], more[1, i], ape, p0 + n + i, D, ratio)
                assert (ea is None) == (eb is None)
                if ea is not None:
                    torch.testing.assert_close(ea, eb)


def test_attention_run_matches_token_by_token():
    """The run form (window spans of one linear buffer + a prefix or a selection of compressed rows) against
    one ``shared_kv_attention`` call per token."""
    from litevllm_b200.models.deepseek_v4_flash.attention import shared_kv_attention, shared_kv_attention_run
    g = torch.Generator().manual_seed(4)
    n, heads, D, W = 7, 3, 128, 5
    q = torch.randn(n, heads, D, generator=g)
    lin, comp = torch.randn(n + W - 1, D, generator=g), torch.randn(9, D, generator=g)
    sinks = torch.randn(heads, generator=g)
    ends = [W - 1 + j + 1 for j in range(n)]
    a0 = [max(0, e - W) for e in ends]
    na = [e - a for e, a in zip(ends, a0)]
    nb = [min(9, 2 + j) for j in range(n)]
    spans = torch.tensor([a0, na, nb], dtype=torch.int32)
    got = shared_kv_attention_run(q, lin, comp, spans, None, sinks, 0.11)
    for j in range(n):
        rows = torch.cat([lin[a0[j]:a0[j] + na[j]], comp[:nb[j]]])
        torch.testing.assert_close(got[j], shared_kv_attention(q[j], rows, sinks, 0.11))
    sel = torch.stack([torch.randperm(9, generator=g)[:4] for _ in range(n)]).to(torch.int32)
    spans[2] = torch.tensor([min(4, v) for v in nb], dtype=torch.int32)
    got = shared_kv_attention_run(q, lin, comp, spans, sel, sinks, 0.11)
    for j in range(n):
        k = int(spans[2, j])
        rows = torch.cat([lin[a0[j]:a0[j] + na[j]], comp[sel[j, :k].long()]])
        torch.testing.assert_close(got[j], shared_kv_attention(q[j], rows, sinks, 0.11))


def test_layer_rows_grow_and_keep_their_rows():
    from litevllm_b200.models.deepseek_v4_flash.model import LayerRows
    lr = LayerRows(pool=torch.zeros(4 + 2, 8), window=4, index_pool=torch.zeros(2, 128), ratio=4)
    rows = torch.arange(40 * 8, dtype=torch.float32).reshape(40, 8)
    idx = torch.arange(40 * 128, dtype=torch.float32).reshape(40, 128)
    lr.append_compressed(rows[0], idx[0])
    lr.append_compressed_many(rows[1:30], idx[1:30])
    for i in range(30, 40):
        lr.append_compressed(rows[i], idx[i])
    assert lr.n_comp == 40 and lr.pool.shape[0] >= 44
    torch.testing.assert_close(lr.compressed, rows)
    torch.testing.assert_close(lr.index_rows, idx)
    assert lr.bytes() == lr.pool.numel() * 4 + lr.index_pool.numel() * 4
