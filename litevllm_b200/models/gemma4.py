"""Gemma4 decoder (dense and 26B-A4B-style mixture of experts).

Per layer: ``h += post_attn_ln(attn(input_ln(h)))``; then the feed-forward block
``h += post_ffn_ln(branches)`` and ``h *= layer_scalar``, where for dense layers ``branches`` is the
GELU-tanh gated MLP of ``pre_ffn_ln(h)`` and for MoE layers it is
``post_ffn_ln_1(shared_mlp(pre_ffn_ln(h))) + post_ffn_ln_2(experts(pre_ffn_ln_2(h)))`` with the router
reading the raw residual (scale-free RMSNorm x learned scale x hidden^-0.5, softmax -> top-k ->
renormalise -> per-expert scale).  Attention: sliding-window layers and global layers (every 6th by
default) may differ in head_dim / kv heads / rope base; logits scale 1.0 with learned q/k RMSNorm
and a weightless v norm, optional k == v, attention-logit softcap, fp8-e4m3 KV by default.
Embeddings are scaled by sqrt(hidden); final logits are soft-capped.
Reference: vllm/model_executor/models/gemma4/{model,layer,attention,mlp,moe}.py.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..layers.linear import LiteLinear
from ..layers.rope import get_cos_sin
from ..ops import moe as moe_ops
from ..ops.awq import Int4Weight, unpack_nibbles
from ..parallel import state as pstate
from ..utils.profiling import stage
from .arch import ModelArch
from .llama import RMSNormWeight


class Gemma4Attention(nn.Module):
    def __init__(self, arch: ModelArch, layer_idx: int, dtype, qc, prefix: str):
        super().__init__()
        tp = pstate.tp_size()
        self.is_sliding = arch.layer_type(layer_idx) == "sliding"
        total_kv, self.hd = arch.kv_shape(layer_idx)
        self.total_heads, self.total_kv = arch.num_heads, total_kv
        self.nh = self.total_heads // tp
        self.kv_replicas = max(1, tp // total_kv)
        self.nkv = max(1, total_kv // tp)
        self.window = arch.sliding_window if self.is_sliding else 0
        self.softcap = arch.attn_softcap
        self.rope_theta = arch.rope_theta if self.is_sliding else (arch.global_rope_theta or arch.rope_theta)
        self.rot_dim = self.hd if self.is_sliding else int(self.hd * float(arch.extra.get("global_partial_rotary_factor", 1.0)))
        self.k_eq_v = bool(arch.extra.get("attention_k_eq_v", False)) and not self.is_sliding
        self.qkv_proj = LiteLinear(arch.hidden_size, (self.nh + 2 * self.nkv) * self.hd, dtype=dtype, quant_config=qc,
                                   prefix=prefix + ".qkv_proj",
                                   out_splits=[self.nh * self.hd, self.nkv * self.hd, self.nkv * self.hd])
        self.o_proj = LiteLinear(self.total_heads * self.hd, arch.hidden_size, dtype=dtype, shard="row",
                                 quant_config=qc, prefix=prefix + ".o_proj")
        self.q_norm = RMSNormWeight(self.hd, arch.rms_eps, dtype)
        self.k_norm = RMSNormWeight(self.hd, arch.rms_eps, dtype)
        self.eps = arch.rms_eps
        self._cos_sin = None
        self.max_pos = 0

    def qkv_source_rows(self, which: str) -> tuple[int, int]:
        r = pstate.tp_rank()
        if which == "q":
            return r * self.nh * self.hd, self.nh * self.hd
        return (r // self.kv_replicas) * self.nkv * self.hd, self.nkv * self.hd

    def cos_sin(self, device, max_pos):
        if self._cos_sin is None or self._cos_sin.device != device or self.max_pos < max_pos:
            self._cos_sin = get_cos_sin(self.rot_dim, max_pos, self.rope_theta, None, device)
            self.max_pos = max_pos
        return self._cos_sin

    def forward(self, x, batch, kv, max_pos):
        qkv = self.qkv_proj(x, lora_mapping=batch.lora_mapping)
        k_cache, v_cache = kv
        cfg = batch.config
        ops.rope_and_cache(qkv, batch.positions, self.cos_sin(qkv.device, max_pos), batch.slot_mapping, k_cache,
                           v_cache, self.nh, self.nkv, self.hd, self.rot_dim, q_norm_w=self.q_norm.weight,
                           k_norm_w=self.k_norm.weight, qk_norm_mode=0, v_norm=True, eps=self.eps,
                           k_scale=cfg.k_scale, v_scale=cfg.v_scale)
        if batch.is_decode:
            attn = ops.paged_attention_decode(qkv, k_cache, v_cache, *batch.attention_tables(self.window), self.nh,
                                              self.nkv, self.hd, 1.0, self.window, self.softcap, cfg.k_scale,
                                              cfg.v_scale, max_kv_len=batch.max_kv_len)
        else:
            attn = ops.paged_attention_prefill(qkv, k_cache, v_cache, batch.block_tables, batch.seq_lens, batch.cu_q,
                                               batch.max_q_len, self.nh, self.nkv, self.hd, 1.0, self.window,
                                               self.softcap, cfg.k_scale, cfg.v_scale)
        return self.o_proj(attn, lora_mapping=batch.lora_mapping)


class Gemma4MLP(nn.Module):
    def __init__(self, arch: ModelArch, inter: int, dtype, qc, prefix: str):
        super().__init__()
        # the tcgen05 GEMMs step through K in blocks of 64: an intermediate width whose per-rank share is not a
        # multiple of that (2112 over two ranks) stays whole on every rank instead of being sharded
        sharded = inter % (64 * pstate.tp_size()) == 0
        self.gate_up_proj = LiteLinear(arch.hidden_size, 2 * inter, dtype=dtype, shard="column" if sharded else None,
                                       quant_config=qc, prefix=prefix + ".gate_up_proj", gated_act="gelu_tanh",
                                       out_splits=[inter, inter])
        self.down_proj = LiteLinear(inter, arch.hidden_size, dtype=dtype, shard="row" if sharded else None,
                                    quant_config=qc, prefix=prefix + ".down_proj")

    def forward(self, x, batch):
        return self.down_proj(self.gate_up_proj(x, lora_mapping=batch.lora_mapping), lora_mapping=batch.lora_mapping)


class Gemma4Router(nn.Module):
    def __init__(self, arch: ModelArch, dtype):
        super().__init__()
        E, H = arch.moe.num_experts, arch.hidden_size
        self.proj = nn.Parameter(torch.empty(E, H, dtype=dtype), requires_grad=False)
        self.scale = nn.Parameter(torch.ones(H, dtype=dtype), requires_grad=False)
        self.per_expert_scale = nn.Parameter(torch.ones(E, dtype=torch.float32), requires_grad=False)
        self.top_k, self.eps, self.H = arch.moe.top_k, arch.rms_eps, H

    def forward(self, residual):
        # scale-free RMSNorm x learned scale x hidden^-0.5, then the router projection in fp32
        x = ops.rmsnorm(residual, self.scale, self.eps, w_mode=0, out_scale=self.H ** -0.5)
        logits = ops.linear(x, self.proj, out_dtype=torch.float32)
        return moe_ops.route(logits, self.top_k, "softmax", None, self.per_expert_scale, True, 1.0)


class Gemma4Experts(nn.Module):
    """Expert-major packed int4 (group 32, symmetric): ``gate_up [E, 2I, H/8]`` + scales
    ``[E, 2I, H/32]``, ``down [E, H, I/8]`` + scales ``[E, H, I/32]``; experts are sharded over the
    expert-parallel ranks."""

    def __init__(self, arch: ModelArch, dtype, group: int = 32):
        super().__init__()
        ep, r = pstate.ep_size(), pstate.ep_rank()
        self.E, self.I, self.H, self.group = arch.moe.num_experts, arch.moe.expert_intermediate, arch.hidden_size, group
        assert self.E % ep == 0
        self.e_local = self.E // ep
        self.e_lo = r * self.e_local
        self.dtype = dtype
        self.device = torch.empty(0).device      # the construction-time default device
        self._parts: dict[str, torch.Tensor] = {}
        self.w_gate_up: Int4Weight | None = None
        self.w_down: Int4Weight | None = None

    def load(self, suffix: str, which: str, tensor: torch.Tensor) -> None:
        """which in {gate_up, down}; suffix in {qweight, scales}; tensor has the expert axis first."""
        self._parts[f"{which}.{suffix}"] = tensor[self.e_lo:self.e_lo + self.e_local].to(self.device)

    def finalize(self) -> None:
        if self.w_gate_up is not None or len(self._parts) < 4:
            return
        dt = self.dtype if self.dtype != torch.float32 else torch.float16
        def build(which, rows, cols):
            q = self._parts.pop(f"{which}.qweight").reshape(self.e_local * rows, cols // 8)
            s = self._parts.pop(f"{which}.scales").reshape(self.e_local * rows, cols // self.group)
            return Int4Weight(unpack_nibbles(q), s, None, self.group, dt)
        self.w_gate_up = build("gate_up", 2 * self.I, self.H)
        self.w_down = build("down", self.H, self.I)

    def forward(self, x, ids, weights):
        self.finalize()
        heap = None
        if pstate.ep_size() > 1:
            from ..parallel import ep_alltoall, fused_ops
            if ep_alltoall.ENABLED:        # tokens sharded over the ranks, routes travel by all-to-all
                def run(rows, expert_ids):
                    one = torch.ones(rows.shape[0], 1, dtype=torch.float32, device=rows.device)
                    return moe_ops.fused_experts(rows, self.w_gate_up, self.w_down, expert_ids.view(-1, 1).to(ids.dtype), one,
                                                 self.e_local, self.e_lo, "gelu_tanh")
                return ep_alltoall.sharded_moe(x, ids, weights, self.e_local, run)
            heap = fused_ops.ep_heap(x)
        out = moe_ops.fused_experts(x, self.w_gate_up, self.w_down, ids, weights, self.e_local, self.e_lo, "gelu_tanh",
                                    ep_heap=heap)
        if pstate.ep_size() > 1 and heap is None:
            out = fused_ops.all_reduce_activations(out)
        return out


class Gemma4DecoderLayer(nn.Module):
    def __init__(self, arch: ModelArch, i: int, dtype, qc):
        super().__init__()
        H, eps = arch.hidden_size, arch.rms_eps
        p = f"model.layers.{i}"
        self.self_attn = Gemma4Attention(arch, i, dtype, qc, p + ".self_attn")
        self.input_layernorm = RMSNormWeight(H, eps, dtype)
        self.post_attention_layernorm = RMSNormWeight(H, eps, dtype)
        self.pre_feedforward_layernorm = RMSNormWeight(H, eps, dtype)
        self.post_feedforward_layernorm = RMSNormWeight(H, eps, dtype)
        self.layer_scalar = nn.Parameter(torch.tensor(1.0), requires_grad=False)
        self._scalar = 1.0
        self.use_moe = arch.moe.num_experts > 0
        if self.use_moe:
            self.pre_feedforward_layernorm_2 = RMSNormWeight(H, eps, dtype)
            self.post_feedforward_layernorm_1 = RMSNormWeight(H, eps, dtype)
            self.post_feedforward_layernorm_2 = RMSNormWeight(H, eps, dtype)
            self.router = Gemma4Router(arch, dtype)
            self.experts = Gemma4Experts(arch, dtype, arch.quant.group_size if arch.quant.method != "none" else 32)
            self.shared_mlp = Gemma4MLP(arch, arch.moe.shared_intermediate or arch.intermediate_size, dtype, qc,
                                        p + ".mlp.shared_mlp")
        else:
            self.mlp = Gemma4MLP(arch, arch.intermediate_size, dtype, qc, p + ".mlp")

    def forward(self, h, batch, kv, max_pos):
        with stage("layer.attention"):
            a = self.self_attn(self.input_layernorm(h), batch, kv, max_pos)
            h = ops.rmsnorm(a, self.post_attention_layernorm.weight, self.post_attention_layernorm.eps, addend=h)
        x = self.pre_feedforward_layernorm(h)
        if self.use_moe:
            with stage("layer.moe.shared"):
                dense = self.post_feedforward_layernorm_1(self.shared_mlp(x, batch))
            with stage("layer.moe.router"):
                ids, w = self.router(h)
            with stage("layer.moe.experts"):
                sparse = self.experts(self.pre_feedforward_layernorm_2(h), ids, w)
            y = ops.rmsnorm(sparse, self.post_feedforward_layernorm_2.weight, self.post_feedforward_layernorm_2.eps,
                            addend=dense)
        else:
            with stage("layer.mlp"):
                y = self.mlp(x, batch)
        h = ops.rmsnorm(y, self.post_feedforward_layernorm.weight, self.post_feedforward_layernorm.eps, addend=h)
        if self._scalar != 1.0:
            h = h * self._scalar
        return h


class Gemma4ForCausalLM(nn.Module):
    supports_lora = False
    supports_multimodal = False

    def __init__(self, vllm_config):
        super().__init__()
        mc = vllm_config.model_config
        arch: ModelArch = mc.arch
        self.arch, self.dtype = arch, mc.dtype
        qc = vllm_config.quant_config
        from ..parallel import ep_alltoall
        if ep_alltoall.ENABLED and pstate.ep_size() > 1:
            self.supports_cuda_graph = False      # the all-to-all split sizes are read on the host every step
        self.embed_tokens = nn.Parameter(torch.empty(arch.vocab_size, arch.hidden_size, dtype=mc.dtype), requires_grad=False)
        self.layers = nn.ModuleList([Gemma4DecoderLayer(arch, i, mc.dtype, qc) for i in range(arch.num_layers)])
        self.norm = RMSNormWeight(arch.hidden_size, arch.rms_eps, mc.dtype)
        self.tie = arch.tie_embeddings
        if not self.tie:
            self.lm_head = LiteLinear(arch.hidden_size, arch.vocab_size, dtype=mc.dtype, shard="column", prefix="lm_head")
        self.max_pos = max(mc.max_model_len, 16)
        self.final_softcap = arch.final_softcap
        if arch.vision:
            from .gemma4_vision import Gemma4VisionTower
            self.vision_tower = Gemma4VisionTower(arch, mc.dtype)
            self.supports_multimodal = True

    def kv_cache_specs(self):
        return [(l.self_attn.nkv, l.self_attn.hd) for l in self.layers]

    def embed(self, input_ids):
        return ops.embedding(input_ids, self.embed_tokens, self.arch.embed_scale)

    def get_multimodal_embeddings(self, **mm_inputs):
        return self.vision_tower(**mm_inputs)

    def forward(self, batch, kv_caches, inputs_embeds=None):
        h = inputs_embeds if inputs_embeds is not None else self.embed(batch.input_ids)
        for i, layer in enumerate(self.layers):
            h = layer(h, batch, kv_caches[i], self.max_pos)
        last = h if batch.logits_indices is None else h.index_select(0, batch.logits_indices)
        x = self.norm(last)
        if self.tie:
            logits = ops.linear(x, self.embed_tokens, out_dtype=torch.float32)
        else:
            logits = self.lm_head(x, out_dtype=torch.float32)
            if self.lm_head.tp > 1:
                logits = pstate.all_gather_last_dim(logits)
        if self.final_softcap and self.final_softcap > 0:
            logits = torch.tanh(logits / self.final_softcap) * self.final_softcap
        return logits

    def load_weights(self, weights):
        from ..loaders.weight_utils import finalize_quantized, load_mapped
        m: dict = {"model.embed_tokens": ("param", self.embed_tokens), "model.norm": ("norm", self.norm)}
        if not self.tie:
            m["lm_head"] = ("linear", self.lm_head, 0, None)
        for i, L in enumerate(self.layers):
            p = f"model.layers.{i}."
            at = L.self_attn
            m[p + "self_attn.q_proj"] = ("linear", at.qkv_proj, 0, at.qkv_source_rows("q"))
            m[p + "self_attn.k_proj"] = ("linear", at.qkv_proj, 1, at.qkv_source_rows("k"))
            m[p + "self_attn.v_proj"] = ("linear", at.qkv_proj, 2, at.qkv_source_rows("v"))
            m[p + "self_attn.o_proj"] = ("linear", at.o_proj, 0, None)
            m[p + "self_attn.q_norm"] = ("norm", at.q_norm)
            m[p + "self_attn.k_norm"] = ("norm", at.k_norm)
            for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm",
                      "post_feedforward_layernorm", "pre_feedforward_layernorm_2", "post_feedforward_layernorm_1",
                      "post_feedforward_layernorm_2"):
                if hasattr(L, n):
                    m[p + n] = ("norm", getattr(L, n))
            def set_scalar(suffix, t, L=L):
                L.layer_scalar.data.copy_(t.reshape(()))
                L._scalar = float(t.reshape(()))
            m[p[:-1]] = ("custom", lambda suffix, t, f=set_scalar: f(suffix, t) if suffix == "layer_scalar" else None)
            mlp = L.shared_mlp if L.use_moe else L.mlp
            mp = p + ("mlp.shared_mlp." if L.use_moe else "mlp.")
            m[mp + "gate_proj"] = ("linear", mlp.gate_up_proj, 0, None)
            m[mp + "up_proj"] = ("linear", mlp.gate_up_proj, 1, None)
            m[mp + "down_proj"] = ("linear", mlp.down_proj, 0, None)
            if L.use_moe:
                def router_load(suffix, t, R=L.router):
                    if suffix == "scale":
                        R.scale.data.copy_(t.to(R.scale.dtype))
                    elif suffix == "per_expert_scale":
                        R.per_expert_scale.data.copy_(t.float())
                m[p + "mlp.router"] = ("custom", router_load)
                m[p + "mlp.router.proj"] = ("custom", lambda s, t, R=L.router: R.proj.data.copy_(t.to(R.proj.dtype)) if s == "weight" else None)
                m[p + "mlp.experts.gate_up_proj"] = ("custom", lambda s, t, X=L.experts: X.load(s, "gate_up", t))
                m[p + "mlp.experts.down_proj"] = ("custom", lambda s, t, X=L.experts: X.load(s, "down", t))
        consumed = load_mapped(m, weights)
        finalize_quantized(self)
        for L in self.layers:
            if L.use_moe:
                L.experts.finalize()
            if L.self_attn.k_eq_v:
                self._tie_v_to_k(L.self_attn)
        return consumed

    @staticmethod
    def _tie_v_to_k(at) -> None:
        lin = at.qkv_proj
        k0, v0, n = at.nh * at.hd, (at.nh + at.nkv) * at.hd, at.nkv * at.hd
        if lin.quant_method is None:
            lin.weight.data[v0:v0 + n].copy_(lin.weight.data[k0:k0 + n])
