"""Forward-hook statistics per module (mean, max |x|, NaN/Inf counts) for chasing numerical drift.
Reference: vllm/debug/activation_sniffer.py."""
from __future__ import annotations

import re
from dataclasses import dataclass

import torch


@dataclass
class ActivationStat:
    name: str
    calls: int = 0
    abs_max: float = 0.0
    mean: float = 0.0
    rms: float = 0.0
    nan: int = 0
    inf: int = 0


class ActivationSniffer:
    """``with ActivationSniffer(model, pattern=r"layers\\.0\\.") as s: ...; s.report()``.
    Hooks synchronise the device (``.item()``), so CUDA-graph capture must be off while sniffing."""

    def __init__(self, model: torch.nn.Module, pattern: str | None = None, leaf_only: bool = True):
        self.model, self.leaf_only = model, leaf_only
        self.pattern = re.compile(pattern) if pattern else None
        self.stats: dict[str, ActivationStat] = {}
        self._handles = []

    def _hook(self, name):
        def fn(_module, _inputs, output):
            t = output[0] if isinstance(output, (tuple, list)) else output
            if not isinstance(t, torch.Tensor) or not t.is_floating_point() or t.numel() == 0:
                return
            f = t.detach().float()
            st = self.stats.setdefault(name, ActivationStat(name))
            finite = torch.isfinite(f)
            st.calls += 1
            st.nan += int(torch.isnan(f).sum().item())
            st.inf += int(torch.isinf(f).sum().item())
            g = torch.where(finite, f, torch.zeros_like(f))
            st.abs_max = max(st.abs_max, float(g.abs().max().item()))
            st.mean = float(g.mean().item())
            st.rms = float(g.pow(2).mean().sqrt().item())
        return fn

    def __enter__(self):
        for name, mod in self.model.named_modules():
            if not name or (self.leaf_only and any(True for _ in mod.children())):
                continue
            if self.pattern is not None and not self.pattern.search(name):
                continue
            self._handles.append(mod.register_forward_hook(self._hook(name)))
        return self

    def __exit__(self, *exc):
        for h in self._handles:
            h.remove()
        self._handles.clear()
        return False

    def report(self, top: int | None = None) -> str:
        rows = sorted(self.stats.values(), key=lambda s: -s.abs_max)
        if top:
            rows = rows[:top]
        lines = [f"{'module':60s} {'calls':>5s} {'absmax':>10s} {'rms':>10s} {'nan':>5s} {'inf':>5s}"]
        lines += [f"{s.name[:60]:60s} {s.calls:5d} {s.abs_max:10.4g} {s.rms:10.4g} {s.nan:5d} {s.inf:5d}" for s in rows]
        return "\n".join(lines)
