"""DeepSeek-V4-Flash: the model-owned data plane built from the blocks of this package.

Unlike the other model families this one does not run through the paged KV cache and the batched
executors: every request owns its latent rows (a sliding window per layer, plus compressed rows and indexer
rows on the compressed layers) and the model returns token ids, not logits.  A prefill chunk or a decode
batch goes through the layers as one group: projections, hyper-connections, router and experts are batched
over the group's tokens; only the row appends, the compressor state machine and the attention walk the
tokens in order.  One token through one layer:

    hyper-connection pre (Sinkhorn-mixed streams -> layer input) -> RMSNorm -> q (low rank) and the shared
    latent row (K = V) -> per-head RMS norm of q, rotary on the tail channels, fp8 round trip of the latent
    -> append to the window -> shared-latent attention with sinks over [window rows | compressed rows emitted
    by earlier tokens (fine layers: the indexer's top-k of them)] -> feed the compressor (and the indexer's
    compressor), which emit one normed, rotated row every ``ratio`` tokens -> inverse rotary on the output tail -> grouped low-rank output projection -> hyper-connection
    post -> RMSNorm -> router (token-id hash table on the first layers, sqrt-softplus top-k elsewhere) ->
    routed experts (+ shared expert) on the Q8_K round-tripped input -> hyper-connection post

and after the last layer: sigmoid-gated sum of the streams -> RMSNorm -> lm_head -> arg-max.

Weights: a ``deepseek4`` GGUF file binds by tensor name; its block-quantised projections and routed experts stay
in HBM in their block formats (``BlockMatrix``, the expert-grouped GGUF kernels), the rest is dequantised once.
A synthetic checkpoint draws dense weights from a seeded generator, or, for full-size geometries, random blocks
in the checkpoint family's formats.  The whole model is resident: the reference's weight stager with its byte
budget and expert LRU has no counterpart here.  Decode steps replay CUDA graphs of their static stretches
(``_decode_step_graphs``); a prefill chunk of one request runs as one pass per layer (``_attention_run``).
Reference: vllm/model_executor/models/deepseek_v4_flash/model.py:249-304, 537-607, 933-1130
(prefill_request / decode_tokens_batch / token steps), gpu_layers.py:684-926, 1247-1610 (layer forwards),
compressed_kv.py:289-455 (row pools), kv_lifecycle.py (release).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass

import torch
from torch import nn

from .attention import (CompressorState, indexer_scores, indexer_topk, shared_kv_attention,
                        shared_kv_attention_run)
from . import native as nv
from .moe import sqrt_softplus_router
from ...utils.profiling import stage
from ...ops import gguf_quant as gq
from .ops import indexer_qat


# decode steps replay CUDA graphs of their static stretches (FI_V4_DECODE_GRAPHS=0: every launch from Python)
_DECODE_GRAPHS = os.environ.get("FI_V4_DECODE_GRAPHS", "1") != "0"
_DECODE_GRAPH_MAX_T = 8          # up to the batch the block-format GEMV serves in one pass


@dataclass
class V4Config:
    hidden: int
    layers: int
    heads: int
    head_dim: int            # width of a latent row (keys = values)
    rotary_dim: int
    q_lora: int
    window: int
    ratios: tuple            # per layer: 0 = sliding window only, 4 = compressor + indexer top-k, other = compressor
    indexer_heads: int
    indexer_topk: int
    hc: int                  # hyper-connection streams
    o_groups: int
    o_lora: int
    experts: int
    top_k: int
    expert_inter: int
    shared_inter: int
    hash_layers: int         # the first layers route by token id
    routed_scale: float
    vocab: int
    eps: float
    rope_theta: float
    swiglu_clamp: float
    rope_theta_compressed: float = 160000.0   # compressed layers: long-context base with YaRN interpolation
    rope_factor: float = 16.0
    rope_original_context: int = 65536
    rope_beta_fast: float = 32.0
    rope_beta_slow: float = 1.0
    block_experts: bool = False      # routed experts only ever exist as GGUF blocks (no dense expert parameters)
    expert_staging_gb: float = 0.0   # device budget for routed experts (0: the environment switch, else all resident)

    @classmethod
    def from_hf(cls, cfg: dict) -> "V4Config":
        g = cfg.get
        return cls(hidden=int(cfg["hidden_size"]), layers=int(cfg["num_hidden_layers"]),
                   heads=int(cfg["num_attention_heads"]), head_dim=int(g("head_dim", 512)),
                   rotary_dim=int(g("qk_rope_head_dim", 64)), q_lora=int(g("q_lora_rank", 1024)),
                   window=int(g("sliding_window", 128)),
                   ratios=tuple(int(r) for r in (g("layer_compress_ratios") or cls.default_ratios(
                       int(cfg["num_hidden_layers"]), int(g("compress_ratio_coarse", 128))))),
                   indexer_heads=int(g("index_n_heads", 4)), indexer_topk=int(g("index_topk", 512)),
                   hc=int(g("hc_mult", 4)), o_groups=int(g("o_groups", 4)), o_lora=int(g("o_lora_rank", 256)),
                   experts=int(g("n_routed_experts", 8)), top_k=int(g("num_experts_per_tok", 2)),
                   expert_inter=int(g("moe_intermediate_size", 256)), shared_inter=int(g("shared_intermediate_size", g("moe_intermediate_size", 256))),
                   hash_layers=int(g("num_hash_layers", 1)), routed_scale=float(g("routed_scaling_factor", 1.5)),
                   vocab=int(cfg["vocab_size"]), eps=float(g("rms_norm_eps", 1e-6)),
                   rope_theta=float(g("rope_theta", 10000.0)), swiglu_clamp=float(g("swiglu_limit", 0.0)),
                   rope_theta_compressed=float(g("compressed_rope_theta", 160000.0)),
                   rope_factor=float(g("rope_scaling_factor", 16.0)),
                   rope_original_context=int(g("rope_original_context", 65536)),
                   rope_beta_fast=float(g("rope_beta_fast", 32.0)), rope_beta_slow=float(g("rope_beta_slow", 1.0)),
                   expert_staging_gb=float(g("expert_staging_gb", 0.0) or 0.0),
                   block_experts=bool(g("synthetic_block_weights", False)) or
                   (g("quantization_config") or {}).get("quant_method") == "gguf")

    def rope_inv_freq(self, compressed: bool) -> torch.Tensor:
        """Angle per position for each rotary pair.  Window-only layers: ``theta^(-2i/rot)``.  Compressed layers:
        the long-context base, each pair blended between its interpolated (``/ factor``) and its extrapolated
        frequency by the YaRN ramp over the correction range of (beta_fast, beta_slow) rotations."""
        rot = self.rotary_dim
        i = torch.arange(rot // 2, dtype=torch.float32)
        if not compressed:
            return self.rope_theta ** (-2.0 * i / rot)
        base = self.rope_theta_compressed
        extrap = base ** (-2.0 * i / rot)

        def corr(n_rot: float) -> float:
            return rot * math.log(self.rope_original_context / (n_rot * 2.0 * math.pi)) / (2.0 * math.log(base))

        low = max(0.0, float(math.floor(corr(self.rope_beta_fast))))
        high = min(float(rot - 1), float(math.ceil(corr(self.rope_beta_slow))))
        ramp = 1.0 - ((i - low) / max(0.001, high - low)).clamp(0.0, 1.0)
        return extrap * (ramp + (1.0 - ramp) / self.rope_factor)

    @staticmethod
    def default_ratios(layers: int, coarse: int = 128) -> list:
        """The checkpoint family's pattern: the first two layers see the window only, then fine (ratio 4,
        indexer-selected) and coarse (all rows) compressed layers alternate."""
        return [0 if i < 2 else (4 if i % 2 == 0 else coarse) for i in range(layers)]


@dataclass
class LayerRows:
    """One request's rows of one layer: ``pool`` holds the sliding-window ring in its first ``window`` rows and the
    compressed rows after them (so a full window plus all compressed rows is one contiguous range); ``index_pool``
    the indexer row of every compressed row.  Both grow by doubling."""
    pool: torch.Tensor                         # [window + capacity, head_dim]
    window: int
    count: int = 0                             # tokens seen
    n_comp: int = 0                            # compressed rows emitted
    index_pool: torch.Tensor | None = None     # [capacity, 128]
    comp_state: CompressorState | None = None
    index_state: CompressorState | None = None
    ratio: int = 0

    def append_compressed(self, row: torch.Tensor, index_row: torch.Tensor | None) -> None:
        cap = self.pool.shape[0] - self.window
        if self.n_comp == cap:
            grown = torch.zeros(self.window + max(16, 2 * cap), self.pool.shape[1], dtype=self.pool.dtype, device=self.pool.device)
            grown[: self.pool.shape[0]] = self.pool
            self.pool = grown
            if self.index_pool is not None:
                gi = torch.zeros(max(16, 2 * cap), 128, dtype=torch.float32, device=self.pool.device)
                gi[:cap] = self.index_pool
                self.index_pool = gi
        self.pool[self.window + self.n_comp] = row
        if index_row is not None:
            self.index_pool[self.n_comp] = index_row
        self.n_comp += 1

    def append_compressed_many(self, rows: torch.Tensor, index_rows: torch.Tensor | None) -> None:
        n = rows.shape[0]
        cap = self.pool.shape[0] - self.window
        if self.n_comp + n > cap:
            new_cap = max(16, 2 * cap, self.n_comp + n)
            grown = torch.zeros(self.window + new_cap, self.pool.shape[1], dtype=self.pool.dtype, device=self.pool.device)
            grown[: self.pool.shape[0]] = self.pool
            self.pool = grown
            if self.index_pool is not None:
                gi = torch.zeros(new_cap, 128, dtype=torch.float32, device=self.pool.device)
                gi[:cap] = self.index_pool
                self.index_pool = gi
        self.pool[self.window + self.n_comp: self.window + self.n_comp + n] = rows
        if index_rows is not None:
            self.index_pool[self.n_comp: self.n_comp + n] = index_rows
        self.n_comp += n

    @property
    def compressed(self) -> torch.Tensor:
        return self.pool[self.window: self.window + self.n_comp]

    @property
    def index_rows(self) -> torch.Tensor:
        return self.index_pool[: self.n_comp] if self.index_pool is not None else self.pool.new_zeros(0, 128)

    def bytes(self) -> int:
        n = self.pool.numel() * self.pool.element_size()
        return n + (self.index_pool.numel() * 4 if self.index_pool is not None else 0)


@dataclass
class RequestRows:
    layers: list
    pos: int = 0

    def bytes(self) -> int:
        return sum(lr.bytes() for lr in self.layers)


class BlockMatrix:
    """A ``[N, K]`` matrix kept in its GGUF block format (Q8_0, Q4_K, ...): decode-sized products stream the
    blocks through the GEMV kernel, larger ones dequantise into scratch in front of the tensor-core GEMM."""

    def __init__(self, raw: torch.Tensor, ggml_type: int, K: int, device):
        self.raw = raw.reshape(-1, raw.shape[-1]).contiguous().to(device)
        self.ggml_type, self.K, self.N = int(ggml_type), int(K), self.raw.shape[0]
        self._dense = None

    def dense(self) -> torch.Tensor:
        if self._dense is None:
            self._dense = gq.dequantize(self.raw.cpu(), self.ggml_type, self.K).to(self.raw.device)
        return self._dense

    def linear(self, x: torch.Tensor) -> torch.Tensor:
        if x.is_cuda:
            return gq.gguf_linear(x.to(torch.bfloat16).contiguous(), self.raw, self.ggml_type, self.K,
                                  out_dtype=torch.float32)
        return x.float() @ self.dense().t()

    def nbytes(self) -> int:
        return 0 if self.raw is None else self.raw.numel()


def _lin(x: torch.Tensor, w) -> torch.Tensor:
    """``x @ w.T`` with an fp32 result: block-format matrices through their kernels, dense ones in the weight's
    dtype (tensor cores for 16-bit weights on a GPU)."""
    if isinstance(w, BlockMatrix):
        return w.linear(x)
    return torch.nn.functional.linear(x.to(w.dtype), w).float()


class V4Layer(nn.Module):
    def __init__(self, c: V4Config, i: int, dtype):
        super().__init__()
        H, D, hc = c.hidden, c.head_dim, c.hc
        n_mix = 2 * hc + hc * hc
        P = lambda *s: nn.Parameter(torch.empty(*s, dtype=dtype), requires_grad=False)
        self.ratio = r = c.ratios[i]
        self.compressed, self.indexed = r > 0, r == 4
        self.hash_routed = i < c.hash_layers
        # hyper-connections (attention and feed-forward halves)
        self.hc_attn_fn, self.hc_attn_base, self.hc_attn_scale = P(hc * H, n_mix), P(n_mix), P(3)
        self.hc_ffn_fn, self.hc_ffn_base, self.hc_ffn_scale = P(hc * H, n_mix), P(n_mix), P(3)
        self.attn_norm, self.ffn_norm = P(H), P(H)
        self.q_a, self.q_a_norm, self.q_b = P(c.q_lora, H), P(c.q_lora), P(c.heads * D, c.q_lora)
        self.kv_proj, self.kv_norm = P(D, H), P(D)
        self.sinks = P(c.heads)
        gh = c.heads // c.o_groups
        self.o_a = P(c.o_groups, c.o_lora, gh * D)
        self.o_b = P(H, c.o_groups * c.o_lora)
        if self.compressed:
            width = (2 if r == 4 else 1) * D
            self.comp_kv, self.comp_gate, self.comp_ape, self.comp_norm = P(width, H), P(width, H), P(r, width), P(D)
        if self.indexed:
            self.idx_q = P(c.indexer_heads * 128, c.q_lora)          # from the normed low-rank query
            self.idx_w = P(c.indexer_heads, H)
            self.idx_kv, self.idx_gate, self.idx_ape, self.idx_norm = P(256, H), P(256, H), P(4, 256), P(128)
        self.router = P(c.experts, H)
        self.router_bias = nn.Parameter(torch.zeros(c.experts, dtype=torch.float32), requires_grad=False)
        if self.hash_routed:
            self.register_buffer("hash_table", torch.zeros(c.top_k, c.vocab, dtype=torch.int32))
        if c.block_experts:       # a full-size model's experts do not fit as dense tensors: blocks only
            self.w_gate = self.w_up = self.w_down = None
        else:
            self.w_gate, self.w_up = P(c.experts, c.expert_inter, H), P(c.experts, c.expert_inter, H)
            self.w_down = P(c.experts, H, c.expert_inter)
        self.s_gate, self.s_up, self.s_down = P(c.shared_inter, H), P(c.shared_inter, H), P(H, c.shared_inter)
        self.routed = None          # RoutedExperts over raw GGUF blocks, once a checkpoint delivers block tensors


class DeepseekV4FlashForCausalLM(nn.Module):
    supports_lora = False
    supports_multimodal = False
    supports_cuda_graph = False
    model_owned_data_plane = True

    def __init__(self, vllm_config):
        super().__init__()
        mc = vllm_config.model_config
        self.cfg = c = V4Config.from_hf(mc.hf_config or {})
        self.dtype = mc.dtype
        self.seed = int(getattr(mc, "seed", 0) or 0)
        self.synthetic = bool(getattr(mc, "synthetic", False))
        self.embed = nn.Parameter(torch.empty(c.vocab, c.hidden, dtype=mc.dtype), requires_grad=False)
        self.layers = nn.ModuleList([V4Layer(c, i, mc.dtype) for i in range(c.layers)])
        self.final_norm = nn.Parameter(torch.empty(c.hidden, dtype=mc.dtype), requires_grad=False)
        self.out_hc_fn = nn.Parameter(torch.empty(c.hc, c.hc * c.hidden, dtype=mc.dtype), requires_grad=False)
        self.out_hc_base = nn.Parameter(torch.empty(c.hc, dtype=mc.dtype), requires_grad=False)
        self.out_hc_scale = nn.Parameter(torch.empty(1, dtype=mc.dtype), requires_grad=False)
        self.lm_head = nn.Parameter(torch.empty(c.vocab, c.hidden, dtype=mc.dtype), requires_grad=False)
        self.requests: dict[str, RequestRows] = {}
        self._f32_cache: dict = {}
        self._merged: dict = {}
        self._dgraphs: dict = {}
        self._ar = None
        self.register_buffer("inv_freq_window", c.rope_inv_freq(False).to(self.embed.device), persistent=False)
        self.register_buffer("inv_freq_compressed", c.rope_inv_freq(True).to(self.embed.device), persistent=False)
        self.max_model_len = int(mc.max_model_len)

    # ------------------------------------------------------------------ weights
    def kv_cache_specs(self):
        # the generic paged pool is not used by this model: one minimal layer keeps the stock allocator happy
        return [(1, 16)]

    # GGUF tensor names of the checkpoint family -> parameter names of this module
    _GGUF_TOP = {"token_embd.weight": "embed", "output_norm.weight": "final_norm", "output.weight": "lm_head",
                 "output_hc_fn.weight": "out_hc_fn", "output_hc_base.weight": "out_hc_base",
                 "output_hc_scale.weight": "out_hc_scale"}
    _GGUF_LAYER = {
        "attn_norm.weight": "attn_norm", "attn_sinks.weight": "sinks", "attn_q_a.weight": "q_a",
        "attn_q_a_norm.weight": "q_a_norm", "attn_q_b.weight": "q_b", "attn_kv.weight": "kv_proj",
        "attn_kv_a_norm.weight": "kv_norm", "attn_output_a.weight": "o_a", "attn_output_b.weight": "o_b",
        "attn_compressor_kv.weight": "comp_kv", "attn_compressor_gate.weight": "comp_gate",
        "attn_compressor_ape.weight": "comp_ape", "attn_compressor_norm.weight": "comp_norm",
        "indexer.attn_q_b.weight": "idx_q", "indexer.proj.weight": "idx_w",
        "indexer_compressor_kv.weight": "idx_kv", "indexer_compressor_gate.weight": "idx_gate",
        "indexer_compressor_ape.weight": "idx_ape", "indexer_compressor_norm.weight": "idx_norm",
        "ffn_norm.weight": "ffn_norm", "ffn_gate_inp.weight": "router", "exp_probs_b.bias": "router_bias",
        "ffn_gate_tid2eid.weight": "hash_table", "ffn_gate_exps.weight": "w_gate", "ffn_up_exps.weight": "w_up",
        "ffn_down_exps.weight": "w_down", "ffn_gate_shexp.weight": "s_gate", "ffn_up_shexp.weight": "s_up",
        "ffn_down_shexp.weight": "s_down",
        "hc_attn_fn.weight": "hc_attn_fn", "hc_attn_base.weight": "hc_attn_base", "hc_attn_scale.weight": "hc_attn_scale",
        "hc_ffn_fn.weight": "hc_ffn_fn", "hc_ffn_base.weight": "hc_ffn_base", "hc_ffn_scale.weight": "hc_ffn_scale",
    }

    @classmethod
    def param_name(cls, name: str) -> str:
        """Checkpoint tensor name -> parameter name (names that are already parameter names pass through)."""
        if name in cls._GGUF_TOP:
            return cls._GGUF_TOP[name]
        if name.startswith("blk."):
            _, idx, suffix = name.split(".", 2)
            if suffix in cls._GGUF_LAYER:
                return f"layers.{idx}.{cls._GGUF_LAYER[suffix]}"
        return name

    # matrices that are only ever the weight of ``x @ W.T``: these may stay in their block format
    _LINEAR = {"q_a", "q_b", "kv_proj", "o_b", "comp_kv", "comp_gate", "idx_q", "idx_w", "idx_kv", "idx_gate",
               "s_gate", "s_up", "s_down", "lm_head"}
    _EXPERTS = {"w_gate": "gate", "w_up": "up", "w_down": "down"}

    def _owner(self, pname: str):
        if pname.startswith("layers."):
            _, idx, attr = pname.split(".", 2)
            return (self.layers[int(idx)] if int(idx) < len(self.layers) else None), attr
        return self, pname

    def _routed_experts(self, layer: V4Layer):
        if layer.routed is None:
            from types import SimpleNamespace
            from ..deepseek_mla import RoutedExperts
            c = self.cfg
            shim = SimpleNamespace(hidden_size=c.hidden, extra={"swiglu_clamp": c.swiglu_clamp, "moe_blocks": len(self.layers),
                                                                "expert_staging_gb": c.expert_staging_gb or None},
                                   moe=SimpleNamespace(num_experts=c.experts, expert_intermediate=c.expert_inter,
                                                       top_k=c.top_k))
            layer.routed = RoutedExperts(shim, torch.bfloat16)
            layer.routed.device = self.embed.device
        return layer.routed

    def load_weights(self, weights, strict: bool = True):
        """Named tensors (parameter names, or the checkpoint family's GGUF names) go into the parameters.  Dense
        tensors are copied; one with the right element count but another layout of the same matrix (transposed
        position table, flattened groups) is reshaped.  Block-quantised tensors stay in HBM as they are where
        the model only multiplies by them (projections -> ``BlockMatrix``, routed experts -> the expert-grouped
        GGUF kernels) and are dequantised once otherwise (embedding, tables, grouped output factor).  A synthetic
        checkpoint has no tensors and gets seeded random weights (norm gains 1, hyper-connection scales small,
        a random hash table).  ``strict``: a checkpoint that delivers tensors has to deliver all of them."""
        from ...loaders.gguf import GGUFTensor
        consumed = set()
        bound = set()                       # parameter names that received a tensor
        for name, t in weights:
            pname = self.param_name(name)
            owner, attr = self._owner(pname)
            target = getattr(owner, attr, None) if owner is not None else None
            expert = attr in self._EXPERTS and isinstance(owner, V4Layer)
            if not isinstance(target, (torch.Tensor, BlockMatrix)) and not (
                    expert and (isinstance(t, GGUFTensor) or self.cfg.block_experts)):
                continue
            if isinstance(t, GGUFTensor) or (expert and target is None):
                if expert:
                    self._routed_experts(owner).load(self._EXPERTS[attr], t)
                    owner._parameters.pop(attr, None)
                    setattr(owner, attr, None)
                    consumed.add(name)
                    bound.add(pname)
                    continue
                rows = t.raw.reshape(-1, t.raw.shape[-1])
                if attr in self._LINEAR and isinstance(target, torch.Tensor) and target.dim() == 2:
                    if (rows.shape[0], t.K) != tuple(target.shape):
                        raise ValueError(f"{name}: {tuple(t.shape)} does not fit {tuple(target.shape)}")
                    owner._parameters.pop(attr, None)
                    setattr(owner, attr, BlockMatrix(rows, t.ggml_type, t.K, self.embed.device))
                    consumed.add(name)
                    bound.add(pname)
                    continue
                t = gq.dequantize(rows, t.ggml_type, t.K).reshape(t.shape)
            if isinstance(target, BlockMatrix):
                raise ValueError(f"{name}: already loaded in block format")
            if t.shape != target.shape:
                if t.numel() != target.numel():
                    raise ValueError(f"{name}: {tuple(t.shape)} does not fit {tuple(target.shape)}")
                t = t.t() if t.dim() == 2 and t.shape == target.shape[::-1] else t.reshape(target.shape)
            target.data.copy_(t.to(target.dtype))
            consumed.add(name)
            bound.add(pname)
        if not consumed:
            self._init_synthetic()
        elif strict:
            # a checkpoint binds every tensor of the model or none: a parameter left as allocated would be noise
            expected = {n for n, _ in self.named_parameters()} | {n for n, _ in self.named_buffers() if "inv_freq" not in n}
            expected |= {f"layers.{i}.{a}" for i, l in enumerate(self.layers) for a in self._EXPERTS
                         if l.routed is not None or self.cfg.block_experts}
            expected -= {f"layers.{i}.router_bias" for i in range(len(self.layers))}     # optional: zeros without it
            missing = sorted(expected - bound)
            if missing:
                raise ValueError(f"checkpoint leaves {len(missing)} tensors of the model unbound: "
                                 + ", ".join(missing[:8]) + (" ..." if len(missing) > 8 else ""))
        self._f32_cache.clear()
        self._merged.clear()
        self._dgraphs.clear()
        for layer in self.layers:
            if layer.hash_routed and bool(((layer.hash_table < 0) | (layer.hash_table >= self.cfg.experts)).any()):
                raise ValueError("token-id routing table names an expert that does not exist")
        return consumed

    def _init_synthetic(self) -> None:
        g = torch.Generator().manual_seed(1000 + self.seed)
        c = self.cfg
        dev = self.embed.device
        if c.block_experts:
            # the checkpoint family's formats, drawn on the device: IQ2_XXS gate / up, Q2_K down, Q8_0 projections
            from ...loaders.gguf import GGUFTensor
            for li, layer in enumerate(self.layers):
                routed = self._routed_experts(layer)
                for which, ty, rows, K in (("gate", 16, c.expert_inter, c.hidden), ("up", 16, c.expert_inter, c.hidden),
                                           ("down", 10, c.hidden, c.expert_inter)):
                    raw = gq.random_blocks(ty, c.experts * rows, K, 7919 * li + ty + len(which) + self.seed, 0.02, str(dev))
                    routed.load(which, GGUFTensor(raw.view(c.experts, rows, -1), ty, (c.experts, rows, K)))
                for attr in sorted(self._LINEAR - {"lm_head"}):
                    p = getattr(layer, attr, None)
                    if isinstance(p, torch.Tensor) and p.shape[1] % 32 == 0 and p.numel() >= 1 << 20:
                        N, K = p.shape
                        raw = gq.random_blocks(8, N, K, 104729 * li + len(attr) + N, 0.5 / math.sqrt(K) / 64, str(dev))
                        layer._parameters.pop(attr, None)
                        setattr(layer, attr, BlockMatrix(raw, 8, K, dev))
        gdev = None
        for name, p in self.named_parameters():
            if name.endswith("norm"):
                p.data.fill_(1.0)
            elif name.endswith("_scale"):
                p.data.fill_(0.1)
            elif name.endswith(("_base", "router_bias", "sinks")):
                p.data.copy_((torch.randn(p.shape, generator=g) * 0.1).to(p.dtype))
            else:
                fan_in = max(p.shape) if name.endswith("_fn") else p.shape[-1]
                if p.is_cuda and p.numel() >= 1 << 24:       # large tensors of full-size models: drawn on the device
                    if gdev is None:
                        gdev = torch.Generator(device=p.device).manual_seed(2000 + self.seed)
                    p.data.copy_((torch.randn(p.shape, generator=gdev, device=p.device) / math.sqrt(fan_in)).to(p.dtype))
                else:
                    p.data.copy_((torch.randn(p.shape, generator=g) / math.sqrt(fan_in)).to(p.dtype))
        for layer in self.layers:
            if layer.hash_routed:        # top_k distinct experts per token id: the first columns of a random permutation
                tab = torch.rand(c.vocab, c.experts, generator=g).argsort(dim=1)[:, : c.top_k].t()
                layer.hash_table.copy_(tab.to(torch.int32))

    # ------------------------------------------------------------------ request state
    def _new_request(self, device) -> RequestRows:
        c = self.cfg
        layers = []
        for i in range(c.layers):
            r = c.ratios[i]
            cap = 0 if r == 0 else 16
            lr = LayerRows(pool=torch.zeros(c.window + cap, c.head_dim, dtype=torch.float32, device=device),
                           window=c.window, ratio=r)
            if r > 0:
                lr.comp_state = CompressorState.empty(c.head_dim, r, device)
            if r == 4:
                lr.index_state = CompressorState.empty(128, 4, device)
                lr.index_pool = torch.zeros(cap, 128, dtype=torch.float32, device=device)
            layers.append(lr)
        return RequestRows(layers)

    def release_request(self, request_id: str) -> bool:
        return self.requests.pop(request_id, None) is not None

    def request_bytes(self) -> int:
        return sum(r.bytes() for r in self.requests.values())

    def kv_stats(self) -> dict:
        """Gauges of the per-request rows (reported with the model events and the engine statistics)."""
        self._active_high_water = max(getattr(self, "_active_high_water", 0), len(self.requests))
        return {"active_requests": len(self.requests), "active_requests_high_water": self._active_high_water,
                "row_bytes": self.request_bytes(),
                "compressed_rows": sum(lr.n_comp for r in self.requests.values() for lr in r.layers)}

    # ------------------------------------------------------------------ a group of tokens, layer by layer
    def _f32(self, owner, attr: str) -> torch.Tensor:
        """fp32 copy of a small parameter (norm gains, hyper-connection tables, sinks, position biases), made once."""
        key = (id(owner), attr)
        t = self._f32_cache.get(key)
        if t is None:
            t = self._f32_cache[key] = getattr(owner, attr).detach().float().contiguous()
        return t

    def _project(self, layer: V4Layer, names: tuple, x: torch.Tensor) -> list:
        """Several projections of the same input as one product: the weights (all dense, or all blocks of one
        format) are stacked row-wise once per layer, the result is split into views."""
        key = (id(layer), names)
        merged = self._merged.get(key)
        if merged is None:
            ws = [getattr(layer, n) for n in names]
            sizes = [w.N if isinstance(w, BlockMatrix) else w.shape[0] for w in ws]
            if all(isinstance(w, BlockMatrix) for w in ws) and len({(w.ggml_type, w.K) for w in ws}) == 1:
                stacked = BlockMatrix(torch.cat([w.raw for w in ws]), ws[0].ggml_type, ws[0].K, ws[0].raw.device)
            elif all(isinstance(w, torch.Tensor) for w in ws) and x.is_cuda:
                stacked = torch.cat([w.detach() for w in ws])
            else:
                stacked = False
            merged = self._merged[key] = (stacked, sizes)
            if stacked is not False and x.is_cuda:       # the single matrices are not used again on this device
                for n, w in zip(names, ws):
                    if isinstance(w, BlockMatrix):
                        w.raw = None
        stacked, sizes = merged
        if stacked is False:
            return [_lin(x, getattr(layer, n)) for n in names]
        return list(_lin(x, stacked).split(sizes, dim=-1))

    def _arange(self, n: int) -> torch.Tensor:
        if self._ar is None or self._ar.numel() < n:
            self._ar = torch.arange(max(1024, 2 * n), dtype=torch.int32, device=self.embed.device)
        return self._ar[:n]

    def _attention(self, layer: V4Layer, rows_of: list, h: torch.Tensor, pos: torch.Tensor, positions: list,
                   li: int) -> torch.Tensor:
        """``h`` ``[T, H]``: the projections run once for the whole group; the row appends, compressor steps
        and the attention itself walk the tokens in order (token t of a request sees the rows of tokens <= t)."""
        ctx = self._attn_pre(layer, h, pos)
        out = torch.empty(h.shape[0], self.cfg.heads, self.cfg.head_dim, dtype=torch.float32, device=h.device)
        self._attn_rows(layer, li, rows_of, positions, pos, ctx, out)
        return self._attn_post(layer, out, pos)

    def _attn_pre(self, layer: V4Layer, h: torch.Tensor, pos: torch.Tensor) -> dict:
        """Everything in front of the rows: layer-input norm, the stacked projection of everything that reads it,
        low-rank query, per-head norm and rotary, the latent row (norm, rotary, fp8 round trip).  A pure function
        of its inputs with static shapes (the decode path captures it in a CUDA graph)."""
        c, f = self.cfg, self._f32
        T, D = h.shape[0], c.head_dim
        freq = self.inv_freq_compressed if layer.compressed else self.inv_freq_window
        x = nv.norm_rope(h, f(layer, "attn_norm"), None, None, c.eps)
        names = ("q_a", "kv_proj") + (("comp_kv", "comp_gate") if layer.compressed else ()) + \
            (("idx_kv", "idx_gate", "idx_w") if layer.indexed else ())
        proj = self._project(layer, names, x)
        q_low = nv.norm_rope(proj[0], f(layer, "q_a_norm"), None, None, c.eps)
        q = nv.norm_rope(_lin(q_low, layer.q_b).view(T, c.heads, D), None, freq, pos, c.eps)
        kv = nv.norm_rope(proj[1], f(layer, "kv_norm"), freq, pos, c.eps, fp8=True)
        return {"q": q, "kv": kv, "q_low": q_low, "proj": proj, "freq": freq}

    def _attn_post(self, layer: V4Layer, out: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """Inverse rotary of the attention output and the grouped low-rank output projection (static shapes)."""
        c = self.cfg
        T, D = out.shape[0], c.head_dim
        freq = self.inv_freq_compressed if layer.compressed else self.inv_freq_window
        out = nv.norm_rope(out, None, freq, pos, c.eps, norm=False, inverse=True)
        gh = c.heads // c.o_groups
        og = out.view(T, c.o_groups, gh * D).to(layer.o_a.dtype)
        low = torch.einsum("grk,tgk->tgr", layer.o_a, og).float()
        return _lin(low.reshape(T, -1), layer.o_b)

    def _attn_rows(self, layer: V4Layer, li: int, rows_of: list, positions: list, pos: torch.Tensor, ctx: dict,
                   out: torch.Tensor) -> None:
        """The part that touches per-request state: window-row appends, attention over each request's rows,
        compressor steps and emitted rows.  Writes ``out`` ``[T, heads, D]``."""
        c, f = self.cfg, self._f32
        q, kv, q_low, proj, freq = ctx["q"], ctx["kv"], ctx["q_low"], ctx["proj"], ctx["freq"]
        T, D, W = q.shape[0], c.head_dim, c.window
        h = q
        if layer.compressed:
            ckv, cgate, comp_ape = proj[2], proj[3], f(layer, "comp_ape")
        if layer.indexed:
            ikv, igate, iw, idx_ape = proj[4], proj[5], proj[6], f(layer, "idx_ape")
            iq = None                           # only needed once a request has more rows than the indexer keeps
        sinks = f(layer, "sinks")
        scale = 1.0 / math.sqrt(D)
        r = layer.ratio
        singles: list = []                      # tokens that are alone in their request (a decode batch)
        lone = sum(1 for j in range(T) if (j == 0 or rows_of[j - 1] is not rows_of[j])
                   and (j == T - 1 or rows_of[j + 1] is not rows_of[j]))
        batch_singles = h.is_cuda and lone >= 2  # one request alone: the pointer tables cost more than they save
        t = 0
        while t < T:
            t1 = t + 1
            while t1 < T and rows_of[t1] is rows_of[t]:
                t1 += 1
            lr: LayerRows = rows_of[t].layers[li]
            if t1 - t == 1 and batch_singles:
                singles.append(t)
                t = t1
                continue
            if t1 - t >= 2:
                # a run of consecutive tokens of one request (a prefill chunk): compressor windows, row
                # post-processing, indexer selection and attention each run once for the whole run
                run = slice(t, t1)
                if layer.indexed and iq is None and lr.n_comp + (t1 - t + 3) // 4 > c.indexer_topk:
                    iq = indexer_qat(nv.norm_rope(_lin(q_low, layer.idx_q).view(T, c.indexer_heads, 128), None, freq, pos,
                                                  c.eps, norm=False))
                self._attention_run(layer, lr, positions[t], q[run], kv[run],
                                    (ckv[run], cgate[run], comp_ape) if layer.compressed else None,
                                    (ikv[run], igate[run], idx_ape, None if iq is None else iq[run], iw[run]) if layer.indexed else None,
                                    freq, sinks, scale, out[run])
                t = t1
                continue
            p = positions[t]
            lr.pool[lr.count % W] = kv[t]
            lr.count += 1
            n_win, n_comp = min(lr.count, W), lr.n_comp
            index = None
            if n_comp and layer.indexed and n_comp > c.indexer_topk:
                # the fine layers keep the indexer's top-k of the rows emitted by earlier tokens
                if iq is None:
                    iq = indexer_qat(nv.norm_rope(_lin(q_low, layer.idx_q).view(T, c.indexer_heads, 128), None, freq, pos,
                                                  c.eps, norm=False))
                keep = indexer_topk(indexer_scores(iq[t], iw[t], lr.index_rows), c.indexer_topk)
                index = torch.cat([self._arange(n_win), keep.to(torch.int32) + W])
            elif n_comp and n_win < W:
                index = torch.cat([self._arange(n_win), self._arange(W + n_comp)[W:]])
            if index is not None:
                shared_kv_attention(q[t], lr.pool, sinks, softmax_scale=scale, row_index=index, out=out[t])
            else:
                shared_kv_attention(q[t], lr.pool[: n_win + n_comp], sinks, softmax_scale=scale, out=out[t])
            if layer.compressed:
                emitted = nv.compressor_step_(lr.comp_state, ckv[t], cgate[t], comp_ape, p, D, r)
                idx_row = nv.compressor_step_(lr.index_state, ikv[t], igate[t], idx_ape, p, 128, 4) if layer.indexed else None
                if emitted is not None:
                    at = pos[t: t + 1] + (1 - r)
                    emitted = nv.norm_rope(emitted.unsqueeze(0), f(layer, "comp_norm"), freq, at, c.eps, fp8=True)[0]
                    if idx_row is not None:
                        idx_row = indexer_qat(nv.norm_rope(idx_row.unsqueeze(0), f(layer, "idx_norm"), freq, at, c.eps))[0]
                    lr.append_compressed(emitted, idx_row)
            t = t1
        if singles:
            if layer.indexed and iq is None and any(rows_of[t].layers[li].n_comp > c.indexer_topk for t in singles):
                iq = indexer_qat(nv.norm_rope(_lin(q_low, layer.idx_q).view(T, c.indexer_heads, 128), None, freq, pos,
                                              c.eps, norm=False))
            self._attention_singles(layer, li, singles, rows_of, positions, pos, q, kv,
                                    (ckv, cgate, comp_ape) if layer.compressed else None,
                                    (ikv, igate, idx_ape, iq, iw) if layer.indexed else None, freq, sinks, scale, out)

    def _attention_singles(self, layer: V4Layer, li: int, ts: list, rows_of: list, positions: list, pos, q, kv, comp, idx,
                           freq, sinks, scale, out) -> None:
        """One token of each of several requests (a decode batch) on a GPU: the window-row writes, the attention and
        the compressor steps of all of them are one launch each; per-request pools and states are addressed
        through pointer arrays built on the host."""
        c, f = self.cfg, self._f32
        n, T, D, W, r = len(ts), q.shape[0], c.head_dim, c.window, layer.ratio
        dev = q.device
        lrs = [rows_of[t].layers[li] for t in ts]
        whole = n == T
        pick = None if whole else torch.tensor(ts, device=dev)
        take = (lambda x: x) if whole else (lambda x: x[pick])
        dst = [lr.pool.data_ptr() + (lr.count % W) * D * 4 for lr in lrs]
        for lr in lrs:
            lr.count += 1
        n_win = [min(lr.count, W) for lr in lrs]
        nb = [lr.n_comp for lr in lrs]
        use_sel = [0] * n
        sel = None
        if idx is not None and max(nb) > c.indexer_topk:
            sel = torch.zeros(n, c.indexer_topk, dtype=torch.int32, device=dev)
            for i, (t, lr) in enumerate(zip(ts, lrs)):
                if nb[i] > c.indexer_topk:
                    sel[i] = indexer_topk(indexer_scores(idx[3][t], idx[4][t], lr.index_rows), c.indexer_topk).to(torch.int32)
                    use_sel[i], nb[i] = 1, c.indexer_topk
        ptr_rows = [dst, [lr.pool.data_ptr() for lr in lrs]]
        if comp is not None:
            ptr_rows += [[lr.comp_state.kv.data_ptr() for lr in lrs], [lr.comp_state.score.data_ptr() for lr in lrs]]
        if idx is not None:
            ptr_rows += [[lr.index_state.kv.data_ptr() for lr in lrs], [lr.index_state.score.data_ptr() for lr in lrs]]
        ptrs = torch.tensor(ptr_rows, dtype=torch.int64, device=dev)
        meta = torch.tensor([n_win, nb, use_sel], dtype=torch.int32, device=dev)
        lib, P, S = nv._k(), nv._p, nv._s
        kv_s, q_s = take(kv).contiguous(), take(q).contiguous()
        nv._call(lib.fi_dsv4_scatter_rows(P(kv_s), D, ptrs[0].data_ptr(), n, D, S()), "fi_dsv4_scatter_rows")
        o = out if whole else torch.empty(n, c.heads, D, dtype=torch.float32, device=dev)
        nv._call(lib.fi_dsv4_shared_kv_attention_ptrs(
            P(q_s), ptrs[1].data_ptr(), meta[0].data_ptr(), meta[1].data_ptr(), meta[2].data_ptr(), P(sel),
            0 if sel is None else sel.stride(0), W, P(sinks), n, c.heads, D, scale, P(o), S()),
            "fi_dsv4_shared_kv_attention_ptrs")
        if not whole:
            out[pick] = o
        if comp is None:
            return
        pos_s = take(pos).contiguous()
        emits = [i for i, t in enumerate(ts) if (positions[t] + 1) % r == 0]

        def step(state_rows: int, cur, gate, ape, head_dim: int, ratio: int) -> torch.Tensor:
            cur, gate = take(cur), take(gate)
            width = (2 if ratio == 4 else 1) * head_dim
            sp, sc = (ape.stride(1), ape.stride(0)) if ape.shape == (width, ratio) else (ape.stride(0), ape.stride(1))
            em = torch.empty(n, head_dim, dtype=torch.float32, device=dev)
            nv._call(lib.fi_dsv4_compressor_step_batch(
                ptrs[state_rows].data_ptr(), ptrs[state_rows + 1].data_ptr(), P(cur), P(gate), cur.stride(0), P(ape), sp, sc,
                P(pos_s), n, ratio, head_dim, P(em), S()), "fi_dsv4_compressor_step_batch")
            return em

        emitted = step(2, comp[0], comp[1], comp[2], D, r)
        idx_rows = step(4, idx[0], idx[1], idx[2], 128, 4) if idx is not None else None
        if emits:
            e = torch.tensor(emits, device=dev)
            at = pos_s[e] + (1 - r)
            rows = nv.norm_rope(emitted[e], f(layer, "comp_norm"), freq, at, c.eps, fp8=True)
            irows = indexer_qat(nv.norm_rope(idx_rows[e], f(layer, "idx_norm"), freq, at, c.eps)) if idx_rows is not None else None
            for k, i in enumerate(emits):
                lrs[i].append_compressed(rows[k], None if irows is None else irows[k])

    def _attention_run(self, layer: V4Layer, lr: LayerRows, p0: int, q, kv, comp, idx, freq, sinks, scale, out) -> None:
        """``n >= 2`` consecutive tokens of one request starting at position ``p0``.  Token j sees the window that ends
        at its own row and the compressed rows emitted by earlier tokens; the rows the run itself emits become
        visible one token after the token that completes their window."""
        c, f = self.cfg, self._f32
        n, D, W, r = q.shape[0], c.head_dim, c.window, layer.ratio
        dev = q.device
        count0, n_comp0 = lr.count, lr.n_comp
        n_prev = min(count0, W - 1)
        if n_prev:
            ring = [(count0 - n_prev + i) % W for i in range(n_prev)]
            lin = torch.cat([lr.pool[torch.tensor(ring, device=dev)], kv])
        else:
            lin = kv.contiguous()
        emit_at: list = []                               # run-relative token index that completes each emitted row
        if comp is not None:
            base = p0 - p0 % r
            ckv, cgate, comp_ape = comp
            emitted = nv.compressor_run_(lr.comp_state, ckv, cgate, comp_ape, p0, D, r)
            idx_rows = nv.compressor_run_(lr.index_state, idx[0], idx[1], idx[2], p0, 128, 4) if idx is not None else None
            if emitted.shape[0]:
                starts = [base + k * r for k in range(emitted.shape[0])]
                emit_at = [s0 + r - 1 - p0 for s0 in starts]
                at = torch.tensor(starts, dtype=torch.long, device=dev)
                emitted = nv.norm_rope(emitted, f(layer, "comp_norm"), freq, at, c.eps, fp8=True)
                if idx_rows is not None:
                    idx_rows = indexer_qat(nv.norm_rope(idx_rows, f(layer, "idx_norm"), freq, at, c.eps))
                lr.append_compressed_many(emitted, idx_rows)
        ends = [n_prev + j + 1 for j in range(n)]
        a0 = [max(0, e - W) for e in ends]
        na = [e - a for e, a in zip(ends, a0)]
        nb, k = [], 0
        for j in range(n):
            while k < len(emit_at) and emit_at[k] < j:
                k += 1
            nb.append(n_comp0 + k)
        sel = None
        if idx is not None and nb[-1] > c.indexer_topk:
            # indexer scores of every token of the run over all rows, rows a token cannot see yet masked out
            iq, iw = idx[3], idx[4]
            rows = lr.index_rows
            n_rows = rows.shape[0]
            keep = min(c.indexer_topk, n_rows)
            sel = torch.empty(n, keep, dtype=torch.int32, device=dev)
            visible = torch.tensor(nb, device=dev)
            s_scale = 1.0 / math.sqrt(c.indexer_heads * 128)
            step = max(1, (64 << 20) // max(1, c.indexer_heads * n_rows))
            for j0 in range(0, n, step):
                blk = slice(j0, min(n, j0 + step))
                per_head = torch.einsum("thd,rd->thr", iq[blk], rows).clamp_min_(0.0)
                scores = (iw[blk].unsqueeze(-1) * per_head).sum(1) * s_scale
                scores.masked_fill_(torch.arange(n_rows, device=dev)[None] >= visible[blk, None], float("-inf"))
                sel[blk] = torch.topk(scores, keep, dim=-1, sorted=True).indices.to(torch.int32)
            nb = [min(v, c.indexer_topk) for v in nb]
        spans = torch.tensor([a0, na, nb], dtype=torch.int32, device=dev)
        out.copy_(shared_kv_attention_run(q, lin, lr.pool[W:], spans, sel, sinks, scale))
        m = min(n, W)
        ring = [(count0 + n - m + i) % W for i in range(m)]
        lr.pool[torch.tensor(ring, device=dev)] = kv[n - m:]
        lr.count += n

    def _ffn(self, layer: V4Layer, h: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
        c, f = self.cfg, self._f32
        x = nv.norm_rope(h, f(layer, "ffn_norm"), None, None, c.eps)
        if layer.hash_routed:
            scores = torch.sqrt(torch.nn.functional.softplus(x @ f(layer, "router").t()))
            key = (id(layer), "hash_rows")
            table = self._f32_cache.get(key)                          # [vocab, top_k] int64, validated at load
            if table is None:
                table = self._f32_cache[key] = layer.hash_table.t().long().contiguous()
            ids = table[token_ids]
            w = torch.nn.functional.normalize(scores.gather(1, ids), p=1.0, dim=-1, eps=1e-20) * c.routed_scale
        else:
            ids, w = sqrt_softplus_router(x, f(layer, "router"), c.top_k, layer.router_bias, c.routed_scale)
            ids = ids.long()
        xq = nv.q8k(x) if x.shape[-1] % 256 == 0 else x

        def mlp(g_w, u_w, d_w, inp):
            g, u = _lin(inp, g_w), _lin(inp, u_w)
            if c.swiglu_clamp > 0:
                g, u = g.clamp(max=c.swiglu_clamp), u.clamp(-c.swiglu_clamp, c.swiglu_clamp)
            return _lin(torch.nn.functional.silu(g) * u, d_w)

        g, u = self._project(layer, ("s_gate", "s_up"), x)
        if c.swiglu_clamp > 0:
            g, u = g.clamp(max=c.swiglu_clamp), u.clamp(-c.swiglu_clamp, c.swiglu_clamp)
        y = _lin(torch.nn.functional.silu(g) * u, layer.s_down)
        if layer.routed is not None:
            act = torch.bfloat16 if x.is_cuda else torch.float32
            return y + layer.routed(xq.to(act).contiguous(), ids.to(torch.int32).contiguous(), w.float().contiguous()).float()
        for e in torch.unique(ids).tolist():
            tok, slot = torch.nonzero(ids == e, as_tuple=True)
            y.index_add_(0, tok, w[tok, slot].unsqueeze(-1) * mlp(layer.w_gate[e], layer.w_up[e], layer.w_down[e], xq[tok]))
        return y

    @torch.inference_mode()
    def forward_tokens(self, entries: list) -> torch.Tensor:
        """``entries``: (request rows, token id) pairs; the tokens of one request appear in prompt order.  Runs
        them through every layer and returns the final hidden vectors ``[T, H]`` (fp32)."""
        c, f = self.cfg, self._f32
        dev = self.embed.device
        seen: dict[int, int] = {}
        positions = []
        for rows, _ in entries:
            k = seen.get(id(rows), 0)
            positions.append(rows.pos + k)
            seen[id(rows)] = k + 1
        rows_of = [r for r, _ in entries]
        ids = torch.tensor([int(t) for _, t in entries], dtype=torch.long, device=dev)
        pos = torch.tensor(positions, dtype=torch.long, device=dev)
        streams = self.embed[ids].float().unsqueeze(1).repeat(1, c.hc, 1)          # [T, hc, H]
        for li, layer in enumerate(self.layers):
            with stage("v4_attention"):
                st = nv.hc_pre(streams, f(layer, "hc_attn_fn"), f(layer, "hc_attn_base"), f(layer, "hc_attn_scale"), c.eps)
                streams = nv.hc_post(self._attention(layer, rows_of, st.mixed, pos, positions, li), streams, st)
            with stage("v4_experts"):
                st = nv.hc_pre(streams, f(layer, "hc_ffn_fn"), f(layer, "hc_ffn_base"), f(layer, "hc_ffn_scale"), c.eps)
                streams = nv.hc_post(self._ffn(layer, st.mixed, ids), streams, st)
        done = set()
        for rows, _ in entries:
            if id(rows) not in done:
                rows.pos += seen[id(rows)]
                done.add(id(rows))
        # collapse the streams (sigmoid gains from the normalised flattened streams), then the final norm
        hidden = nv.hc_collapse(streams, f(self, "out_hc_fn"), f(self, "out_hc_base"), f(self, "out_hc_scale"), c.eps)
        return nv.norm_rope(hidden, f(self, "final_norm"), None, None, c.eps)

    def _next_tokens(self, hidden: torch.Tensor) -> list[int]:
        return torch.argmax(_lin(hidden, self.lm_head), dim=-1).tolist()

    # ------------------------------------------------------------------ request API (token ids in, token ids out)
    @torch.inference_mode()
    def prefill_request(self, request_id: str, token_ids: list[int], start: int = 0, final: bool = True) -> int | None:
        """Feed ``token_ids`` (the chunk beginning at prompt position ``start``) token by token; with ``final``
        return the first generated token."""
        dev = self.embed.device
        if start == 0 or request_id not in self.requests:
            self.requests[request_id] = self._new_request(dev)
        rows = self.requests[request_id]
        if rows.pos != start:
            raise RuntimeError(f"request {request_id}: chunk starts at {start} but {rows.pos} tokens were processed")
        if not token_ids:
            return None
        hidden = self.forward_tokens([(rows, int(t)) for t in token_ids])
        return self._next_tokens(hidden[-1:])[0] if final else None

    @torch.inference_mode()
    def decode_tokens_batch(self, request_ids: list[str], last_tokens: list[int]) -> list[int]:
        """One token for each request; the projections and experts of the whole batch run together."""
        rows = [self.requests[r] for r in request_ids]
        if self._decode_graphs_ok(rows):
            return self._decode_step_graphs(rows, [int(t) for t in last_tokens])
        hidden = self.forward_tokens([(r, int(t)) for r, t in zip(rows, last_tokens)])
        return self._next_tokens(hidden)

    # ------------------------------------------------------------------ decode steps through CUDA graphs
    # A decode step alternates between work with static shapes (everything except the rows) and work on
    # per-request state whose sizes change from step to step (window appends, attention over a growing row set,
    # compressor emissions).  The static stretches - from the output of one layer's attention to the input of the
    # next layer's - are captured once per batch size and replayed: one launch instead of about forty-five.
    def _decode_graphs_ok(self, rows: list) -> bool:
        # dense (non-block) experts group their routes with a host read, which a capture cannot contain
        return (_DECODE_GRAPHS and self.embed.is_cuda and 1 <= len(rows) <= _DECODE_GRAPH_MAX_T
                and len({id(r) for r in rows}) == len(rows) and all(l.routed is not None and l.routed.stage_budget is None for l in self.layers))

    def _layer_tail(self, li: int, out: torch.Tensor, g: dict) -> None:
        """Static stretch after layer ``li``'s rows: output projection, the feed-forward half, and either the next
        layer's front or the head of the model.  Reads and writes the tensors kept in ``g``."""
        c, f = self.cfg, self._f32
        layer = self.layers[li]
        streams = nv.hc_post(self._attn_post(layer, out, g["pos"]), g["streams"][li], g["state"][li])
        st = nv.hc_pre(streams, f(layer, "hc_ffn_fn"), f(layer, "hc_ffn_base"), f(layer, "hc_ffn_scale"), c.eps)
        streams = nv.hc_post(self._ffn(layer, st.mixed, g["ids"]), streams, st)
        if li + 1 < len(self.layers):
            self._layer_front(li + 1, streams, g)
        else:
            hidden = nv.hc_collapse(streams, f(self, "out_hc_fn"), f(self, "out_hc_base"), f(self, "out_hc_scale"), c.eps)
            hidden = nv.norm_rope(hidden, f(self, "final_norm"), None, None, c.eps)
            g["tokens"] = torch.argmax(_lin(hidden, self.lm_head), dim=-1)

    def _layer_front(self, li: int, streams: torch.Tensor, g: dict) -> None:
        c, f = self.cfg, self._f32
        layer = self.layers[li]
        st = nv.hc_pre(streams, f(layer, "hc_attn_fn"), f(layer, "hc_attn_base"), f(layer, "hc_attn_scale"), c.eps)
        g["streams"][li], g["state"][li] = streams, st
        g["ctx"][li] = self._attn_pre(layer, st.mixed, g["pos"])

    def _capture_decode_graphs(self, T: int) -> dict:
        c = self.cfg
        dev = self.embed.device
        L = len(self.layers)
        g = {"ids": torch.zeros(T, dtype=torch.long, device=dev), "pos": torch.zeros(T, dtype=torch.long, device=dev),
             "streams": [None] * L, "state": [None] * L, "ctx": [None] * L, "tokens": None,
             "out": [torch.zeros(T, c.heads, c.head_dim, dtype=torch.float32, device=dev) for _ in range(L)]}

        def front0():
            streams = self.embed[g["ids"]].float().unsqueeze(1).repeat(1, c.hc, 1)
            self._layer_front(0, streams, g)

        # once eagerly on a side stream: lazily built caches, stacked projections, scratch buffers, kernel attributes
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            front0()
            for li in range(L):
                self._layer_tail(li, g["out"][li], g)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        graphs, pool = [], None
        for k in range(L + 1):
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, pool=pool):
                if k == 0:
                    front0()
                else:
                    self._layer_tail(k - 1, g["out"][k - 1], g)
            pool = pool or gr.pool()
            graphs.append(gr)
        g["graphs"] = graphs
        return g

    def _decode_step_graphs(self, rows: list, tokens: list) -> list[int]:
        T = len(rows)
        g = self._dgraphs.get(T)
        if g is None:
            g = self._dgraphs[T] = self._capture_decode_graphs(T)
        positions = [r.pos for r in rows]
        meta = torch.tensor([tokens, positions], dtype=torch.long, device=self.embed.device)
        g["ids"].copy_(meta[0])
        g["pos"].copy_(meta[1])
        g["graphs"][0].replay()
        for li, layer in enumerate(self.layers):
            self._attn_rows(layer, li, rows, positions, g["pos"], g["ctx"][li], g["out"][li])
            g["graphs"][li + 1].replay()
        for r in rows:
            r.pos += 1
        return g["tokens"].tolist()

    def forward(self, batch, kv_caches, inputs_embeds=None):
        raise RuntimeError("DeepSeek-V4-Flash runs through its own executors (token ids in, token ids out)")
