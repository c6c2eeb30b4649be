"""Linear layers.

``LiteLinear`` owns one ``[out, in]`` weight (possibly the row-wise merge of several projections,
e.g. q|k|v or gate|up) or a quantised weight record, and runs it through the op layer.  Tensor
parallelism is expressed by ``shard``: ``"column"`` splits output rows across ranks, ``"row"``
splits the input dimension and the caller (or the fused kernel) reduces the partial sums.
Reference: vllm/model_executor/layers/lite_linear.py:8-83 (single GPU, lazy weights, LoRA hook).
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..parallel import state as pstate


class LiteLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = False,
                 dtype: torch.dtype = torch.bfloat16, shard: str | None = None,
                 quant_config=None, prefix: str = "", gated_act: str | None = None,
                 out_splits: list[int] | None = None):
        super().__init__()
        tp = pstate.tp_size() if shard else 1
        self.shard = shard
        self.tp = tp
        self.prefix = prefix
        self.gated_act = gated_act          # set: weight is [gate; up] and forward returns act(g)*u
        self.full_in, self.full_out = in_features, out_features
        self.out_splits = out_splits or [out_features]   # logical pieces of a merged weight
        self.in_features = in_features // tp if shard == "row" else in_features
        self.out_features = out_features // tp if shard == "column" else out_features
        self.quant_method = quant_config.get_method(self) if quant_config is not None else None
        self.lora = None                     # set by LoRAManager.bind_to_model
        if self.quant_method is not None:
            self.quant_method.create_weights(self, dtype)
        else:
            self.weight = nn.Parameter(torch.empty(self.out_features, self.in_features, dtype=dtype),
                                       requires_grad=False)
        if bias:
            self.bias = nn.Parameter(torch.zeros(self.out_features, dtype=dtype), requires_grad=False)
        else:
            self.bias = None

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None,
                out: torch.Tensor | None = None, out_dtype=None, lora_mapping=None,
                norm_eps: float = 0.0, lora_x: torch.Tensor | None = None) -> torch.Tensor:
        """x: [T, in].  With ``residual`` the result is ``x W^T + residual`` (fused epilogue).  With
        ``norm_eps`` the rows of x are RMS-normalised inside the GEMM (the norm weight must have been
        folded into this layer with :meth:`fold_input_norm`)."""
        if self.shard == "row" and self.tp > 1:
            return self._row_parallel(x, residual, out)
        y = self._matmul(x, residual, out, out_dtype, norm_eps=norm_eps)
        if self.lora is not None and lora_mapping is not None:
            # with a folded input norm the adapters still see the normalised, weighted activations
            y = self.lora.apply(self, lora_x if lora_x is not None else x, y, lora_mapping)
        return y

    def _matmul(self, x, residual=None, out=None, out_dtype=None, use_bias: bool = True, norm_eps: float = 0.0):
        if self.quant_method is not None:
            assert norm_eps == 0.0, "the fused input norm needs an unquantised weight"
            return self.quant_method.apply(self, x, residual=residual, out=out, out_dtype=out_dtype,
                                           use_bias=use_bias)
        if self.gated_act is not None:
            return ops.gated_linear(x, self.weight, self.gated_act, out=out, rms_eps=norm_eps)
        return ops.linear(x, self.weight, self.bias if use_bias else None, residual, out=out,
                          out_dtype=out_dtype, rms_eps=norm_eps)

    def fold_input_norm(self, norm_weight: torch.Tensor, plus_one: bool = False) -> bool:
        """Multiply the weight columns by the RMSNorm weight of the layer's input (in place), so the
        norm in front of this layer reduces to a per-row scale that the GEMM kernel applies itself.
        Returns False (and changes nothing) for quantised layers and input widths the kernel cannot
        take."""
        if self.quant_method is not None or self.in_features % 64 != 0 or self.shard == "row":
            return False
        g = norm_weight.float() + (1.0 if plus_one else 0.0)
        self.weight.data = (self.weight.data.float() * g.to(self.weight.device)[None, :]).to(self.weight.dtype)
        self.input_norm_folded = True
        return True

    def _row_parallel(self, x, residual, out):
        from ..parallel import fused_ops
        return fused_ops.row_parallel_linear(self, x, residual, out)

    # ------------------------------------------------------------------ loading
    def shard_rows(self, full_rows: int) -> tuple[int, int]:
        r = pstate.tp_rank() if self.shard == "column" else 0
        n = full_rows // self.tp if self.shard == "column" else full_rows
        return r * n, n

    def piece_offset(self, piece: int) -> int:
        """First local row of logical piece ``piece`` inside the merged parameter."""
        div = self.tp if self.shard == "column" else 1
        return sum(s // div for s in self.out_splits[:piece])

    def load_piece(self, piece: int, tensor: torch.Tensor, name: str = "weight",
                   src_rows: tuple[int, int] | None = None) -> None:
        """Copy one logical projection (index ``piece`` of ``out_splits``) into the merged,
        TP-sharded parameter.  ``src_rows=(start, n)`` overrides the default row slice of the
        source tensor (used when KV heads are replicated across ranks)."""
        if self.quant_method is not None and name != "bias":
            self.quant_method.load_piece(self, piece, name, tensor, src_rows)
            return
        param = getattr(self, name)
        dst0 = self.piece_offset(piece)
        if src_rows is None:
            src_rows = self.shard_rows(self.out_splits[piece])
        start, n = src_rows
        src = tensor[start:start + n]
        if name == "weight" and self.shard == "row":
            k = self.in_features
            src = src[:, pstate.tp_rank() * k:(pstate.tp_rank() + 1) * k]
        param.data[dst0:dst0 + n].copy_(src.to(param.dtype))

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, shard={self.shard}, gated={self.gated_act}"


# Names kept for users of the reference's layer vocabulary.
ColumnParallelLinear = LiteLinear
RowParallelLinear = LiteLinear
ReplicatedLinear = LiteLinear
