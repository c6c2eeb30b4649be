"""AWQ zero-point int4 (group 128 by default): config + per-layer method.
Reference: vllm/model_executor/layers/quantization/awq.py:14-146 and the ``AWQWeight`` record in
tensor.py:1008-1147 (fused Triton path or dense-fallback LRU; here there is only the fused path)."""
from __future__ import annotations

import torch

from ...ops import awq as awq_ops
from ...parallel import state as pstate


class Int4LinearMethod:
    """Collects the checkpoint pieces of a (merged, TP-sharded) layer, then repacks once."""

    def __init__(self, bits: int, group_size: int, zero_point: bool, layout: str = "auto"):
        assert bits == 4, "only 4-bit weights are supported"
        self.group = group_size
        self.zero_point = zero_point
        self.layout = layout     # "rowmajor" | "autoawq" | "auto" (by shape, row-major when ambiguous)

    def _is_autoawq(self, layer, name: str, t: torch.Tensor) -> bool:
        if self.layout != "auto":
            return self.layout == "autoawq"
        K, G = layer.full_in, self.group
        if name == "qweight":
            return t.shape[1] * 8 != K and t.shape[0] == K
        if name == "scales":
            return t.shape[1] != K // G and t.shape[0] == K // G
        if name == "qzeros":
            return t.shape[1] != (K // G + 7) // 8 and t.shape[0] == K // G
        return False

    def create_weights(self, layer, dtype) -> None:
        N, K = layer.out_features, layer.in_features
        dev = torch.empty(0).device
        layer._q_dtype = dtype
        layer._q_nib = torch.zeros(N, K, dtype=torch.uint8, device=dev)
        layer._q_scales = torch.zeros(N, K // self.group, dtype=torch.float16 if dtype == torch.float32 else dtype, device=dev)
        layer._q_zeros = torch.full((N, K // self.group), 8, dtype=torch.uint8, device=dev) if self.zero_point else None
        layer.int4 = None

    def _k_slice(self, layer, t: torch.Tensor, per: int) -> torch.Tensor:
        """Column slice of a row-sharded (K-split) layer; ``per`` = K elements per column of t."""
        if layer.shard != "row" or layer.tp == 1:
            return t
        k = layer.in_features // per
        r = pstate.tp_rank()
        return t[:, r * k:(r + 1) * k]

    def load_piece(self, layer, piece: int, name: str, tensor: torch.Tensor, src_rows=None) -> None:
        dst0 = layer.piece_offset(piece)
        full_rows = layer.out_splits[piece]
        if src_rows is None:
            src_rows = layer.shard_rows(full_rows)
        start, n = src_rows
        dev = layer._q_nib.device
        if name == "qweight":
            t = tensor.to(dev)
            if self._is_autoawq(layer, name, t):      # AutoAWQ [K, N/8] orientation
                layer._autoawq = getattr(layer, "_autoawq", {})
                layer._autoawq[(piece, "qweight")] = t
                return self._try_autoawq(layer, piece, src_rows)
            nib = awq_ops.unpack_nibbles(t[start:start + n])
            layer._q_nib[dst0:dst0 + n].copy_(self._k_slice(layer, nib, 1))
        elif name == "scales":
            t = tensor.to(dev)
            if self._is_autoawq(layer, name, t):
                layer._autoawq = getattr(layer, "_autoawq", {})
                layer._autoawq[(piece, "scales")] = t
                return self._try_autoawq(layer, piece, src_rows)
            layer._q_scales[dst0:dst0 + n].copy_(self._k_slice(layer, t[start:start + n], self.group).to(layer._q_scales.dtype))
        elif name == "qzeros":
            t = tensor.to(dev)
            if self._is_autoawq(layer, name, t):
                layer._autoawq = getattr(layer, "_autoawq", {})
                layer._autoawq[(piece, "qzeros")] = t
                return self._try_autoawq(layer, piece, src_rows)
            z = awq_ops.unpack_nibbles(t[start:start + n])[:, : layer.full_in // self.group]
            if layer._q_zeros is not None:
                layer._q_zeros[dst0:dst0 + n].copy_(self._k_slice(layer, z, self.group))
        elif name in ("weight_shape", "g_idx"):
            return
        elif name == "weight":   # an unquantised tensor inside a quantised checkpoint: quantise on the fly
            raise ValueError(f"layer {layer.prefix} expects packed int4 tensors, got a dense weight")
        else:
            raise KeyError(f"unexpected quantised tensor suffix {name!r} for {layer.prefix}")

    def _try_autoawq(self, layer, piece, src_rows) -> None:
        need = [(piece, "qweight"), (piece, "scales")] + ([(piece, "qzeros")] if self.zero_point else [])
        if not all(k in layer._autoawq for k in need):
            return
        qz = layer._autoawq.pop((piece, "qzeros")) if self.zero_point else None
        nib, scales, zeros = awq_ops.autoawq_to_rowmajor(layer._autoawq.pop((piece, "qweight")),
                                                         layer._autoawq.pop((piece, "scales")), qz)
        dst0 = layer.piece_offset(piece)
        start, n = src_rows
        layer._q_nib[dst0:dst0 + n].copy_(self._k_slice(layer, nib[start:start + n], 1))
        layer._q_scales[dst0:dst0 + n].copy_(self._k_slice(layer, scales[start:start + n], self.group).to(layer._q_scales.dtype))
        if zeros is not None and layer._q_zeros is not None:
            layer._q_zeros[dst0:dst0 + n].copy_(self._k_slice(layer, zeros[start:start + n], self.group))

    def process_weights_after_loading(self, layer) -> None:
        if layer.int4 is not None:
            return
        dt = layer._q_dtype if layer._q_dtype != torch.float32 else torch.float16
        layer.int4 = awq_ops.Int4Weight(layer._q_nib, layer._q_scales, layer._q_zeros, self.group, dt)
        if layer._q_nib.is_cuda:
            layer._q_nib = layer._q_scales = layer._q_zeros = None

    def apply(self, layer, x, residual=None, out=None, out_dtype=None, ungated: bool = False,
              use_bias: bool = True):
        if layer.int4 is None:
            self.process_weights_after_loading(layer)
        gated = None if ungated else layer.gated_act
        if ungated and layer.gated_act is not None and x.is_cuda:
            # rare path (LoRA on a gated layer): run the merged weight as a plain [2I, K] GEMM
            w = layer.int4
            return awq_ops.int4_linear(x, w, out_dtype=out_dtype)
        return awq_ops.int4_linear(x, layer.int4, bias=layer.bias if use_bias else None, residual=residual, gated_act=gated,
                                   out=out, out_dtype=out_dtype)


class AWQConfig:
    name = "awq"

    def __init__(self, bits: int = 4, group_size: int = 128, zero_point: bool = True,
                 skip_modules: tuple[str, ...] = ("lm_head",), layout: str = "auto"):
        self.bits, self.group_size, self.zero_point = bits, group_size, zero_point
        self.skip_modules = skip_modules
        self.layout = layout

    def get_method(self, layer):
        if any(s in layer.prefix for s in self.skip_modules) or not layer.prefix:
            return None
        return Int4LinearMethod(self.bits, self.group_size, self.zero_point, self.layout)

    def __repr__(self) -> str:
        return f"AWQConfig(bits={self.bits}, group_size={self.group_size}, zero_point={self.zero_point})"
