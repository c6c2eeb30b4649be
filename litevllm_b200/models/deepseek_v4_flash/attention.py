"""Shared-latent attention of DeepSeek-V4-Flash.

Every head attends over the same latent rows, which serve as keys AND values (K = V, width 512);
a per-head sink logit joins the softmax denominator without a value row.  Layers differ in which
rows they see: the sliding-window rows, the rows a compressor emits every ``ratio`` tokens, or (with
the lightning indexer) the top-k compressed rows by indexer score.  fp32 CUDA tensors run the native
kernels (csrc/deepseek/dsv4_kernels.cu); everything else the PyTorch form below.
Reference: vllm/model_executor/models/deepseek_v4_flash/attention.py:429-763 and
compressed_kv.py:289-455 (lazily grown paged pools).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ... import ops
from ...ops import _lib


def _native(*tensors) -> bool:
    return all(t is None or (t.is_cuda and t.dtype in (torch.float32, torch.int32)) for t in tensors)


def shared_kv_attention(queries: torch.Tensor, rows: torch.Tensor, sinks: torch.Tensor | None = None,
                        softmax_scale: float | None = None, row_index: torch.Tensor | None = None,
                        page_table: torch.Tensor | None = None, page_rows: int = 0,
                        out: torch.Tensor | None = None) -> torch.Tensor:
    """queries ``[heads, D]``; ``rows`` ``[n, D]`` (or the whole pool when ``row_index`` / ``page_table``
    address it); returns ``[heads, D]`` fp32 (written into ``out`` when given)."""
    heads, D = queries.shape
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    n_rows = int(row_index.shape[0]) if row_index is not None else (
        rows.shape[0] if page_table is None else page_rows * int(page_table.shape[0]))
    if _native(queries, rows, sinks, row_index, page_table) and D % 128 == 0 and D <= 512:
        if out is None or not out.is_contiguous():
            dst = torch.empty(heads, D, dtype=torch.float32, device=queries.device)
        else:
            dst = out
        rc = _lib.kernels().fi_dsv4_shared_kv_attention(
            ops._p(queries.contiguous()), ops._p(rows), ops._p(row_index), ops._p(page_table), page_rows,
            ops._p(sinks), heads, n_rows, D, scale, ops._p(dst), ops._stream())
        _lib.check(rc, "fi_dsv4_shared_kv_attention")
        if out is not None and dst is not out:
            out.copy_(dst)
            return out
        return dst
    logical = row_index.long() if row_index is not None else torch.arange(n_rows, device=rows.device)
    if page_table is not None:
        logical = page_table.long()[logical // page_rows] * page_rows + logical % page_rows
    kv = rows.float()[logical]
    logits = queries.float() @ kv.t() * scale
    if sinks is not None:
        logits = torch.cat([logits, sinks.float().reshape(-1, 1)], dim=-1)
    probs = torch.softmax(logits, dim=-1)
    res = probs[:, :kv.shape[0]] @ kv
    if out is not None:
        out.copy_(res)
        return out
    return res


def shared_kv_attention_run(queries: torch.Tensor, lin: torch.Tensor, comp: torch.Tensor, spans: torch.Tensor,
                            sel: torch.Tensor | None = None, sinks: torch.Tensor | None = None,
                            softmax_scale: float | None = None) -> torch.Tensor:
    """A run of consecutive tokens of one request at once.  queries ``[T, heads, D]``; token t attends the window
    rows ``lin[a0:a0 + na]`` and ``nb`` compressed rows of ``comp`` (the first ``nb``, or ``sel[t, :nb]``), where
    ``(a0, na, nb) = spans[:, t]`` (int32 ``[3, T]``).  Returns ``[T, heads, D]`` fp32."""
    T, heads, D = queries.shape
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    if _native(queries, lin, comp, spans, sel, sinks) and D % 128 == 0 and D <= 512 and T <= 65535:
        out = torch.empty(T, heads, D, dtype=torch.float32, device=queries.device)
        spans = spans.contiguous()
        rc = _lib.kernels().fi_dsv4_shared_kv_attention_run(
            ops._p(queries.contiguous()), ops._p(lin), ops._p(comp), spans[0].data_ptr(), spans[1].data_ptr(),
            spans[2].data_ptr(), ops._p(sel), 0 if sel is None else sel.stride(0), ops._p(sinks), T, heads, D, scale,
            ops._p(out), ops._stream())
        _lib.check(rc, "fi_dsv4_shared_kv_attention_run")
        return out
    out = torch.empty(T, heads, D, dtype=torch.float32, device=queries.device)
    host = spans.tolist()
    for t in range(T):
        a0, na, nb = host[0][t], host[1][t], host[2][t]
        rows = lin[a0:a0 + na]
        if nb:
            rows = torch.cat([rows, comp[sel[t, :nb].long()] if sel is not None else comp[:nb]], 0)
        out[t] = shared_kv_attention(queries[t], rows.contiguous(), sinks, softmax_scale=scale)
    return out


def compressed_row_attention(queries, compressed_rows, selected: torch.Tensor, sinks=None, softmax_scale=None):
    """Attention over the selected compressed rows only (indexer top-k)."""
    return shared_kv_attention(queries, compressed_rows, sinks, softmax_scale, row_index=selected.to(torch.int32))


def update_latent_cache(pool: torch.Tensor, rows: torch.Tensor, positions: torch.Tensor,
                        page_table: torch.Tensor | None = None, page_rows: int = 0) -> None:
    """Write latent rows at logical positions through the page table."""
    if _native(pool, rows, positions, page_table):
        rc = _lib.kernels().fi_dsv4_cache_update(ops._p(rows.contiguous()), ops._p(positions), ops._p(page_table),
                                                 page_rows, rows.shape[0], rows.shape[1], ops._p(pool), ops._stream())
        _lib.check(rc, "fi_dsv4_cache_update")
        return
    logical = positions.long()
    if page_table is not None:
        logical = page_table.long()[logical // page_rows] * page_rows + logical % page_rows
    pool[logical] = rows.to(pool.dtype)


def indexer_scores(indexer_query: torch.Tensor, indexer_weights: torch.Tensor, compressed_rows: torch.Tensor,
                   scale: float | None = None) -> torch.Tensor:
    """``score[r] = scale * sum_h w[h] * relu(q[h] . row[r])``; q ``[H, 128]``, rows ``[n, 128]``."""
    H, d = indexer_query.shape
    s = float(scale) if scale is not None else 1.0 / math.sqrt(H * d)
    if _native(indexer_query, indexer_weights, compressed_rows) and d == 128 and compressed_rows.shape[0] > 0:
        out = torch.empty(compressed_rows.shape[0], dtype=torch.float32, device=indexer_query.device)
        rc = _lib.kernels().fi_dsv4_indexer_scores(ops._p(indexer_query.contiguous()), ops._p(indexer_weights),
                                                   ops._p(compressed_rows.contiguous()), compressed_rows.shape[0], H, s,
                                                   ops._p(out), ops._stream())
        _lib.check(rc, "fi_dsv4_indexer_scores")
        return out
    per_head = (indexer_query.float() @ compressed_rows.float().t()).clamp_min(0.0)
    return (indexer_weights.float().reshape(-1, 1) * per_head).sum(0) * s


def indexer_topk(scores: torch.Tensor, top_k: int) -> torch.Tensor:
    return torch.topk(scores.float(), k=min(top_k, scores.numel()), sorted=True).indices


@dataclass
class CompressorState:
    """Rolling window of the KV compressor: ``ratio`` rows (two overlapping windows for ratio 4)."""
    kv: torch.Tensor
    score: torch.Tensor

    @classmethod
    def empty(cls, head_dim: int, ratio: int, device=None) -> "CompressorState":
        coff = 2 if ratio == 4 else 1
        shape = (coff * ratio, coff * head_dim)
        return cls(torch.zeros(shape, dtype=torch.float32, device=device),
                   torch.full(shape, float("-inf"), dtype=torch.float32, device=device))


def compressor_step(state: CompressorState, kv_cur: torch.Tensor, score_cur: torch.Tensor, ape: torch.Tensor,
                    token_idx: int, head_dim: int, ratio: int):
    """Feed one token's (kv, gate score) projections; returns (new state, emitted row or None).
    A row is emitted every ``ratio`` tokens as the softmax(score)-weighted mean over the window
    (ratio 4: the previous window's first half-width joined with the current window's second half).
    ``ape`` is the learned position bias ``[ratio, width]`` (or transposed)."""
    coff = 2 if ratio == 4 else 1
    width = coff * head_dim
    pos = token_idx % ratio
    ape_pos = ape[:, pos] if ape.shape == (width, ratio) else ape[pos]
    row = ratio + pos if ratio == 4 else pos
    kv, score = state.kv.clone(), state.score.clone()
    kv[row] = kv_cur.float()
    score[row] = score_cur.float() + ape_pos.float()
    emitted = None
    if (token_idx + 1) % ratio == 0:
        if ratio == 4:
            sc = torch.cat([score[:ratio, :head_dim], score[ratio:, head_dim:]], 0)
            vals = torch.cat([kv[:ratio, :head_dim], kv[ratio:, head_dim:]], 0)
        else:
            sc, vals = score[:ratio, :head_dim], kv[:ratio, :head_dim]
        w = torch.softmax(sc, dim=0)
        emitted = (torch.nan_to_num(w) * vals).sum(0)
        if ratio == 4:     # the current window becomes the previous one
            kv[:ratio] = kv[ratio:]
            score[:ratio] = score[ratio:]
    return CompressorState(kv, score), emitted
