"""GGUF block-quantised linear layers: the raw file blocks (Q8_0, Q2_K, IQ2_XXS) stay as they are
and are consumed by the GGUF kernels; pieces of a merged layer that arrive as plain float tensors or
in different block formats are dequantised into one dense weight instead.
Reference: vllm/model_executor/layers/quantization/gguf.py:18-78 (CPU dequantisation + cache)."""
from __future__ import annotations

import os

import torch

from ...ops import gguf_quant as gq
from ...parallel import state as pstate


_resident_used = [0]


def _resident_budget(device) -> int:
    v = os.environ.get("FI_GGUF_DENSE_RESIDENT_GB")
    if v is not None and v != "":
        return int(float(v) * (1 << 30))
    return torch.cuda.get_device_properties(device).total_memory // 5


class GGUFLinearMethod:
    def create_weights(self, layer, dtype) -> None:
        layer._g_dtype = dtype
        layer._g_pieces = {}          # piece -> (GGUFTensor | dense tensor, src_rows)
        layer.g_raw = None
        layer.g_type = None
        layer.weight = None
        layer._g_device = torch.empty(0).device

    def load_piece(self, layer, piece: int, name: str, tensor, src_rows=None) -> None:
        if name != "weight":
            raise KeyError(f"unexpected GGUF tensor suffix {name!r} for {layer.prefix}")
        layer._g_pieces[piece] = (tensor, src_rows)

    def _rows(self, layer, piece, src_rows):
        if src_rows is None:
            src_rows = layer.shard_rows(layer.out_splits[piece])
        return src_rows

    def process_weights_after_loading(self, layer) -> None:
        if layer.g_raw is not None or layer.weight is not None or not layer._g_pieces:
            return
        from ...loaders.gguf import GGUFTensor
        pieces = [layer._g_pieces[i] for i in sorted(layer._g_pieces)]
        dev, K = layer._g_device, layer.in_features
        types = {t.ggml_type if isinstance(t, GGUFTensor) else -1 for t, _ in pieces}
        r, tp = pstate.tp_rank(), layer.tp
        if len(types) == 1 and -1 not in types:
            ty = types.pop()
            vals, nb = gq.BLOCK[ty]
            if layer.shard != "row" or tp == 1 or (K % vals == 0):
                rows = []
                for i, (t, src) in enumerate(pieces):
                    start, n = self._rows(layer, sorted(layer._g_pieces)[i], src)
                    raw = t.raw[start:start + n]
                    if layer.shard == "row" and tp > 1:
                        rb = K // vals * nb
                        raw = raw[:, r * rb:(r + 1) * rb]
                    rows.append(raw)
                layer.g_raw = torch.cat(rows, 0).contiguous().to(dev)
                layer.g_type = ty
                layer._g_pieces = {}
                self._maybe_make_resident(layer)
                return
        # mixed formats / float tensors: one dense weight
        dt = layer._g_dtype
        rows = []
        for i, (t, src) in enumerate(pieces):
            start, n = self._rows(layer, sorted(layer._g_pieces)[i], src)
            if isinstance(t, GGUFTensor):
                w = gq.dequantize(t.raw[start:start + n], t.ggml_type, t.shape[-1])
            else:
                w = t[start:start + n].float()
            if layer.shard == "row" and tp > 1:
                w = w[:, r * K:(r + 1) * K]
            rows.append(w.to(dt))
        layer.weight = torch.nn.Parameter(torch.cat(rows, 0).to(dev), requires_grad=False)
        layer._g_pieces = {}

    def _maybe_make_resident(self, layer) -> None:
        """Keep a 16-bit copy instead of the blocks when the budget for such copies has room: the dense
        (non-expert) matrices of a GGUF model are a few GB on a 180 GB part, and at decode sizes the
        tcgen05 GEMM on 16-bit weights (8-12 us per launch, with its fused epilogues) beats the
        block-streaming GEMV (43 us per launch on the DeepSeek-shaped model) although it reads twice
        the bytes.  ``FI_GGUF_DENSE_RESIDENT_GB`` sets the budget (default: a fifth of the device
        memory; 0 keeps every matrix as blocks)."""
        raw = layer.g_raw
        if raw is None or not raw.is_cuda or layer._g_dtype not in (torch.bfloat16, torch.float16):
            return
        need = raw.shape[0] * layer.in_features * 2
        if _resident_used[0] + need > _resident_budget(raw.device):
            return
        w = gq.dequantize_cuda(raw, layer.g_type, layer.in_features, layer._g_dtype)
        layer.weight = torch.nn.Parameter(w, requires_grad=False)
        layer.g_raw = None
        _resident_used[0] += need

    def apply(self, layer, x, residual=None, out=None, out_dtype=None, ungated: bool = False, use_bias: bool = True):
        from ... import ops
        if layer.g_raw is None and layer.weight is None:
            self.process_weights_after_loading(layer)
        gated = None if ungated else layer.gated_act
        if layer.weight is not None:
            if gated:
                return ops.gated_linear(x, layer.weight, gated, out=out)
            return ops.linear(x, layer.weight, layer.bias if use_bias else None, residual, out=out, out_dtype=out_dtype)
        if gated:
            y = gq.gguf_linear(x, layer.g_raw, layer.g_type, layer.in_features)
            return ops.act_mul(y, gated, out=out)
        return gq.gguf_linear(x, layer.g_raw, layer.g_type, layer.in_features, out=out, residual=residual,
                              out_dtype=out_dtype)


class GGUFConfig:
    name = "gguf"

    def get_method(self, layer):
        if not layer.prefix:
            return None
        return GGUFLinearMethod()

    def __repr__(self) -> str:
        return "GGUFConfig()"
