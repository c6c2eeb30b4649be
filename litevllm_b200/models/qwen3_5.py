"""Qwen3.5 / Qwen3-Next style hybrid decoder: three of every four layers are GatedDeltaNet linear
attention, every fourth is gated full attention.

Linear-attention layer (per token t, per value head):
  qkv = SiLU(causal depthwise conv1d_k4(in_proj_qkv(x)));  q, k L2-normalised, q scaled by dk^-0.5
  beta = sigmoid(in_proj_b(x));  g = -exp(A_log) * softplus(in_proj_a(x) + dt_bias)
  S <- S * exp(g);  delta = (v - S^T k) * beta;  S <- S + k (x) delta;  o = S^T q
  out = out_proj( RMSNorm(o) * w * SiLU(in_proj_z(x)) )
The recurrent state S [value heads, dk, dv] and the last three conv inputs live in per-layer pools
indexed by the request's slot (the same index that selects its block-table row), so a batch needs no
gather/scatter of Python-side state: prefill walks each sequence with the chunk-64 form of the rule
(``ops.linear_attn.gated_delta_chunked``), decode runs one convolution-step kernel and one
delta-rule-step kernel for the whole batch (csrc/linear_attn/gated_delta.cu), which also makes the
decode step capturable in a CUDA graph.  A sequence whose first position is 0 starts from a zero state.
Full-attention layer: q_proj emits [q | gate] per head, per-head (1+w) RMSNorm on q and k, partial
rotary (first 25 % of the head), paged attention, output multiplied by sigmoid(gate).
MoE variant (``num_experts > 0``): softmax router -> top-k (-> renormalise) over 16-bit experts stacked
``[E, 2I, H]`` / ``[E, H, I]`` plus a shared expert scaled by ``sigmoid(shared_expert_gate(x))``.
Reference: vllm/model_executor/models/qwen3_5.py:42-1573 (linear attention :127-260, MoE :382-606).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops
from ..ops import linear_attn as la_ops
from ..layers.linear import LiteLinear
from ..layers.rope import get_cos_sin
from ..parallel import state as pstate
from .arch import ModelArch
from .llama import LlamaMLP, RMSNormWeight


class GatedDeltaNet(nn.Module):
    def __init__(self, arch: ModelArch, i: int, dtype, qc, prefix: str):
        super().__init__()
        e = arch.extra
        self.nk = int(e.get("linear_num_key_heads", 4))
        self.nv = int(e.get("linear_num_value_heads", 8))
        self.dk = int(e.get("linear_key_head_dim", 64))
        self.dv = int(e.get("linear_value_head_dim", 64))
        self.kw = int(e.get("linear_conv_kernel_dim", 4))
        H = arch.hidden_size
        self.qkv_dim = 2 * self.nk * self.dk + self.nv * self.dv
        self.in_proj_qkv = LiteLinear(H, self.qkv_dim, dtype=dtype, quant_config=qc, prefix=prefix + ".in_proj_qkv")
        self.in_proj_z = LiteLinear(H, self.nv * self.dv, dtype=dtype, quant_config=qc, prefix=prefix + ".in_proj_z")
        self.in_proj_ba = LiteLinear(H, 2 * self.nv, dtype=dtype, prefix="", out_splits=[self.nv, self.nv])
        self.conv_weight = nn.Parameter(torch.empty(self.qkv_dim, self.kw, dtype=dtype), requires_grad=False)
        self.A_log = nn.Parameter(torch.zeros(self.nv, dtype=torch.float32), requires_grad=False)
        self.dt_bias = nn.Parameter(torch.zeros(self.nv, dtype=torch.float32), requires_grad=False)
        self.norm = RMSNormWeight(self.dv, arch.rms_eps, dtype)
        self.out_proj = LiteLinear(self.nv * self.dv, H, dtype=dtype, shard=None, quant_config=qc, prefix=prefix + ".out_proj")
        self.eps = arch.rms_eps

    # ------------------------------------------------------------------ state pools
    def ensure_pools(self, num_slots: int, device, dtype) -> None:
        """State of every slot: S fp32 [slots, nv, dk, dv] and the conv window [slots, C, kw - 1]."""
        cur = getattr(self, "state_pool", None)
        if cur is not None and cur.shape[0] >= num_slots and cur.device == device:
            return
        with torch.inference_mode(False):
            pool = torch.zeros(num_slots, self.nv, self.dk, self.dv, dtype=torch.float32, device=device)
            conv = torch.zeros(num_slots, self.qkv_dim, self.kw - 1, dtype=dtype, device=device)
        if cur is not None:
            pool[: cur.shape[0]].copy_(cur)
            conv[: cur.shape[0]].copy_(self.conv_pool)
        self.state_pool, self.conv_pool = pool, conv

    def _heads(self, mixed):
        """fp32 [n, C] conv output -> q, k [n, nv, dk] (normalised, q scaled, repeated per value head), v [n, nv, dv]."""
        n = mixed.shape[0]
        q = mixed[:, : self.nk * self.dk].view(n, self.nk, self.dk)
        k = mixed[:, self.nk * self.dk: 2 * self.nk * self.dk].view(n, self.nk, self.dk)
        v = mixed[:, 2 * self.nk * self.dk:].view(n, self.nv, self.dv)
        q = F.normalize(q, dim=-1) * self.dk ** -0.5
        k = F.normalize(k, dim=-1)
        rep = self.nv // self.nk
        if rep > 1:
            q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
        return q.contiguous(), k.contiguous(), v.contiguous()

    def forward(self, x, h, batch, slots):
        """x [T, H]; ``slots`` int32 [num_seqs]: state-pool row of every sequence (negative = padded row)."""
        qkv_all = self.in_proj_qkv(x)
        z_all = self.in_proj_z(x)
        ba = self.in_proj_ba(x).float()
        beta_all = torch.sigmoid(ba[:, : self.nv]).contiguous()
        g_all = (-torch.exp(self.A_log) * F.softplus(ba[:, self.nv:] + self.dt_bias)).contiguous()
        T = x.shape[0]
        if batch.is_decode:
            mixed = la_ops.conv1d_step(qkv_all, self.conv_pool, slots, self.conv_weight)
            q, k, v = self._heads(mixed)
            o = la_ops.gated_delta_step(self.state_pool, slots, q, k, v, g_all, beta_all)
            valid = (slots >= 0).view(-1, 1, 1)
            o = torch.where(valid, o, torch.zeros((), device=o.device))
        else:
            o = torch.empty(T, self.nv, self.dv, dtype=torch.float32, device=x.device)
            slot_list = slots.tolist()
            off = 0
            for b, n in enumerate(batch.q_lens_cpu):
                sl = slot_list[b]
                seq = qkv_all[off:off + n]
                ctx = torch.cat([self.conv_pool[sl].t(), seq], dim=0)            # [kw-1+n, C]
                win = ctx.unfold(0, self.kw, 1)                                    # [n, C, kw]
                mixed = F.silu((win.float() * self.conv_weight.float()).sum(-1))
                self.conv_pool[sl].copy_(ctx[-(self.kw - 1):].t())
                q, k, v = self._heads(mixed)
                oo, S = la_ops.gated_delta_chunked(q, k, v, g_all[off:off + n], beta_all[off:off + n],
                                                   self.state_pool[sl])
                self.state_pool[sl].copy_(S)
                o[off:off + n] = oo
                off += n
        on = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + self.eps) * self.norm.weight.float()
        gate = F.silu(z_all.float().view(T, self.nv, self.dv))
        outs = (on * gate).reshape(T, -1).to(x.dtype)
        return self.out_proj(outs, residual=h, out=h)


class Qwen35SparseMoe(nn.Module):
    """Softmax-routed experts plus a sigmoid-gated shared expert (reference: qwen3_5.py:382-606).
    Expert weights are 16-bit tensors stacked on the expert axis; routing and the per-expert GEMMs
    go through ``layers.fused_moe.fused_moe`` (native router kernel + tcgen05 GEMMs on a GPU)."""

    def __init__(self, arch: ModelArch, dtype, qc, prefix: str):
        super().__init__()
        m = arch.moe
        H, I, E = arch.hidden_size, m.expert_intermediate, m.num_experts
        self.top_k, self.renorm, self.E, self.I = m.top_k, m.renormalize, E, I
        self.gate = nn.Parameter(torch.empty(E, H, dtype=dtype), requires_grad=False)
        self.w_gate_up = nn.Parameter(torch.empty(E, 2 * I, H, dtype=dtype), requires_grad=False)
        self.w_down = nn.Parameter(torch.empty(E, H, I, dtype=dtype), requires_grad=False)
        self.shared = None
        if m.shared_intermediate > 0:
            import copy
            sa = copy.copy(arch)
            sa.intermediate_size = m.shared_intermediate
            self.shared = LlamaMLP(sa, dtype, qc, prefix + ".shared_expert")
            self.shared_gate = nn.Parameter(torch.empty(1, H, dtype=dtype), requires_grad=False)

    def forward(self, x, h, batch):
        from ..layers.fused_moe.fused_moe import fused_moe
        logits = ops.linear(x, self.gate, out_dtype=torch.float32)
        y = fused_moe(x, self.w_gate_up, self.w_down, logits, self.top_k, renormalize=self.renorm, act="silu")
        if self.shared is not None:
            zero = torch.zeros_like(h)
            sh = self.shared(x, zero, batch)                       # residual-free shared expert output
            sg = torch.sigmoid(ops.linear(x, self.shared_gate, out_dtype=torch.float32))
            y = (y.float() + sh.float() * sg).to(x.dtype)
        h.add_(y)
        return h


class GatedFullAttention(nn.Module):
    def __init__(self, arch: ModelArch, i: int, dtype, qc, prefix: str):
        super().__init__()
        self.nh, self.nkv, self.hd = arch.num_heads, arch.num_kv_heads, arch.head_dim
        H = arch.hidden_size
        self.gated = bool(arch.extra.get("attn_output_gate", True))
        q_out = self.nh * self.hd * (2 if self.gated else 1)
        self.q_proj = LiteLinear(H, q_out, dtype=dtype, quant_config=qc, prefix=prefix + ".q_proj")
        self.kv_proj = LiteLinear(H, 2 * self.nkv * self.hd, dtype=dtype, quant_config=qc, prefix=prefix + ".kv_proj",
                                  out_splits=[self.nkv * self.hd, self.nkv * self.hd])
        self.o_proj = LiteLinear(self.nh * self.hd, H, dtype=dtype, quant_config=qc, prefix=prefix + ".o_proj")
        self.q_norm = RMSNormWeight(self.hd, arch.rms_eps, dtype, plus_one=True)
        self.k_norm = RMSNormWeight(self.hd, arch.rms_eps, dtype, plus_one=True)
        self.rot_dim = max(2, int(self.hd * arch.partial_rotary_factor) // 2 * 2)
        self.rope_theta, self.eps = arch.rope_theta, arch.rms_eps
        self._cs = None

    def forward(self, x, h, batch, kv, max_pos):
        T = x.shape[0]
        qg = self.q_proj(x).view(T, self.nh, -1)
        q = qg[..., : self.hd]
        kvp = self.kv_proj(x)
        qkv = torch.cat([q.reshape(T, -1), kvp], dim=1).contiguous()
        if self._cs is None or self._cs.device != x.device:
            self._cs = get_cos_sin(self.rot_dim, max_pos, self.rope_theta, None, x.device)
        k_cache, v_cache = kv
        cfg = batch.config
        ops.rope_and_cache(qkv, batch.positions, self._cs, batch.slot_mapping, k_cache, v_cache, self.nh, self.nkv,
                           self.hd, self.rot_dim, q_norm_w=self.q_norm.weight, k_norm_w=self.k_norm.weight,
                           qk_norm_mode=1, eps=self.eps, k_scale=cfg.k_scale, v_scale=cfg.v_scale)
        if batch.is_decode:
            attn = ops.paged_attention_decode(qkv, k_cache, v_cache, *batch.attention_tables(0), self.nh,
                                              self.nkv, self.hd, self.hd ** -0.5, 0, 0.0, cfg.k_scale, cfg.v_scale,
                                              max_kv_len=batch.max_kv_len)
        else:
            attn = ops.paged_attention_prefill(qkv, k_cache, v_cache, batch.block_tables, batch.seq_lens, batch.cu_q,
                                               batch.max_q_len, self.nh, self.nkv, self.hd, self.hd ** -0.5, 0, 0.0,
                                               cfg.k_scale, cfg.v_scale)
        if self.gated:
            gate = torch.sigmoid(qg[..., self.hd:].float()).reshape(T, -1)
            attn = (attn.float() * gate).to(x.dtype)
        return self.o_proj(attn, residual=h, out=h)


class Qwen35DecoderLayer(nn.Module):
    def __init__(self, arch: ModelArch, i: int, dtype, qc):
        super().__init__()
        p = f"model.layers.{i}"
        self.is_linear = arch.layer_type(i) == "linear"
        self.input_layernorm = RMSNormWeight(arch.hidden_size, arch.rms_eps, dtype, plus_one=True)
        self.post_attention_layernorm = RMSNormWeight(arch.hidden_size, arch.rms_eps, dtype, plus_one=True)
        if self.is_linear:
            self.linear_attn = GatedDeltaNet(arch, i, dtype, qc, p + ".linear_attn")
        else:
            self.self_attn = GatedFullAttention(arch, i, dtype, qc, p + ".self_attn")
        self.is_moe = arch.moe.num_experts > 0
        self.mlp = Qwen35SparseMoe(arch, dtype, qc, p + ".mlp") if self.is_moe else LlamaMLP(arch, dtype, qc, p + ".mlp")


class Qwen35ForCausalLM(nn.Module):
    supports_lora = False
    supports_multimodal = False
    supports_cuda_graph = True        # decode touches only device tensors (state pools indexed by slot)

    def __init__(self, vllm_config):
        super().__init__()
        mc = vllm_config.model_config
        arch: ModelArch = mc.arch
        assert pstate.tp_size() == 1, "the Qwen3.5 hybrid model runs on a single GPU"
        self.arch, self.dtype = arch, mc.dtype
        qc = vllm_config.quant_config
        self.embed_tokens = nn.Parameter(torch.empty(arch.vocab_size, arch.hidden_size, dtype=mc.dtype), requires_grad=False)
        self.layers = nn.ModuleList([Qwen35DecoderLayer(arch, i, mc.dtype, qc) for i in range(arch.num_layers)])
        self.norm = RMSNormWeight(arch.hidden_size, arch.rms_eps, mc.dtype, plus_one=True)
        self.lm_head = LiteLinear(arch.hidden_size, arch.vocab_size, dtype=mc.dtype, prefix="lm_head")
        self.max_pos = max(mc.max_model_len, 16)
        self.linear_idx = [i for i, l in enumerate(self.layers) if l.is_linear]
        self.supports_cuda_graph = arch.moe.num_experts == 0   # the generic expert loop reads counts back to the host
        sc = getattr(vllm_config, "scheduler_config", None)
        self.num_slots = max(int(getattr(sc, "max_num_seqs", 8) or 8), 256)   # >= the planner's slot cap

    def kv_cache_specs(self):
        # linear layers keep no KV; a zero-head spec keeps layer indexing uniform
        return [(0 if l.is_linear else self.arch.num_kv_heads, self.arch.head_dim) for l in self.layers]

    def _slots(self, batch):
        """State-pool row per sequence (int32, negative for the padded rows of a decode bucket).  A prefill
        sequence that starts at position 0 begins from a zero state."""
        ids = batch.extras.get("slot_ids")
        if ids is None:
            raise RuntimeError("the batch carries no slot ids (linear-attention state is pooled by slot)")
        dev, dt = self.embed_tokens.device, self.dtype
        for i in self.linear_idx:
            self.layers[i].linear_attn.ensure_pools(self.num_slots, dev, dt)
        if batch.is_decode:
            return torch.where(batch.seq_lens > 0, ids, torch.full_like(ids, -1)).to(torch.int32).contiguous()
        slots = ids.to(torch.int32).contiguous()
        first = batch.positions.view(-1, batch.positions.shape[-1])[0][batch.cu_q[:-1].long()]
        fresh = slots[first == 0].long()
        if fresh.numel():
            for i in self.linear_idx:
                la = self.layers[i].linear_attn
                la.state_pool.index_fill_(0, fresh, 0)
                la.conv_pool.index_fill_(0, fresh, 0)
        return slots

    def forward(self, batch, kv_caches, inputs_embeds=None):
        h = inputs_embeds if inputs_embeds is not None else ops.embedding(batch.input_ids, self.embed_tokens)
        slots = self._slots(batch)
        for i, layer in enumerate(self.layers):
            x = layer.input_layernorm(h)
            if layer.is_linear:
                h = layer.linear_attn(x, h, batch, slots)
            else:
                h = layer.self_attn(x, h, batch, kv_caches[i], self.max_pos)
            h = layer.mlp(layer.post_attention_layernorm(h), h, batch)
        last = h if batch.logits_indices is None else h.index_select(0, batch.logits_indices)
        return self.lm_head(self.norm(last), out_dtype=torch.float32)

    def load_weights(self, weights):
        from ..loaders.weight_utils import finalize_quantized, load_mapped
        m: dict = {"model.embed_tokens": ("param", self.embed_tokens), "model.norm": ("norm", self.norm),
                   "lm_head": ("linear", self.lm_head, 0, None)}
        for i, L in enumerate(self.layers):
            p = f"model.layers.{i}."
            m[p + "input_layernorm"] = ("norm", L.input_layernorm)
            m[p + "post_attention_layernorm"] = ("norm", L.post_attention_layernorm)
            if L.is_moe:
                mo = L.mlp
                m[p + "mlp.gate"] = ("param", mo.gate)
                if mo.shared is not None:
                    m[p + "mlp.shared_expert.gate_proj"] = ("linear", mo.shared.gate_up_proj, 0, None)
                    m[p + "mlp.shared_expert.up_proj"] = ("linear", mo.shared.gate_up_proj, 1, None)
                    m[p + "mlp.shared_expert.down_proj"] = ("linear", mo.shared.down_proj, 0, None)
                    m[p + "mlp.shared_expert_gate"] = ("param", mo.shared_gate)

                def expert(e, which, mo=mo):
                    def put(suffix, t):
                        if suffix != "weight":
                            return
                        if which == "gate_proj":
                            mo.w_gate_up.data[e, : mo.I].copy_(t)
                        elif which == "up_proj":
                            mo.w_gate_up.data[e, mo.I:].copy_(t)
                        else:
                            mo.w_down.data[e].copy_(t)
                    return put
                for e in range(mo.E):
                    for which in ("gate_proj", "up_proj", "down_proj"):
                        m[p + f"mlp.experts.{e}.{which}"] = ("custom", expert(e, which))
            else:
                m[p + "mlp.gate_proj"] = ("linear", L.mlp.gate_up_proj, 0, None)
                m[p + "mlp.up_proj"] = ("linear", L.mlp.gate_up_proj, 1, None)
                m[p + "mlp.down_proj"] = ("linear", L.mlp.down_proj, 0, None)
            if L.is_linear:
                la = L.linear_attn
                m[p + "linear_attn.in_proj_qkv"] = ("linear", la.in_proj_qkv, 0, None)
                m[p + "linear_attn.in_proj_z"] = ("linear", la.in_proj_z, 0, None)
                m[p + "linear_attn.in_proj_b"] = ("linear", la.in_proj_ba, 0, None)
                m[p + "linear_attn.in_proj_a"] = ("linear", la.in_proj_ba, 1, None)
                m[p + "linear_attn.out_proj"] = ("linear", la.out_proj, 0, None)
                m[p + "linear_attn.norm"] = ("norm", la.norm)

                def misc(suffix, t, la=la):
                    if suffix == "A_log":
                        la.A_log.data.copy_(t.float())
                    elif suffix == "dt_bias":
                        la.dt_bias.data.copy_(t.float())
                m[p + "linear_attn"] = ("custom", misc)
                m[p + "linear_attn.conv1d"] = ("custom", lambda s, t, la=la: la.conv_weight.data.copy_(
                    t.reshape(la.qkv_dim, la.kw).to(la.conv_weight.dtype)) if s == "weight" else None)
            else:
                sa = L.self_attn
                m[p + "self_attn.q_proj"] = ("linear", sa.q_proj, 0, None)
                m[p + "self_attn.k_proj"] = ("linear", sa.kv_proj, 0, None)
                m[p + "self_attn.v_proj"] = ("linear", sa.kv_proj, 1, None)
                m[p + "self_attn.o_proj"] = ("linear", sa.o_proj, 0, None)
                m[p + "self_attn.q_norm"] = ("norm", sa.q_norm)
                m[p + "self_attn.k_norm"] = ("norm", sa.k_norm)
        consumed = load_mapped(m, weights)
        finalize_quantized(self)
        return consumed
