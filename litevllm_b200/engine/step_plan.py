"""Plan of one engine step (reference: vllm/engine/step_plan.py)."""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class PrefillItem:
    request_id: str
    start: int        # tokens of the prompt already in cache
    chunk_len: int    # prompt tokens to process this step

    @property
    def end(self) -> int:
        return self.start + self.chunk_len


@dataclass
class StepPlan:
    admissions: list[str] = field(default_factory=list)
    prefills: list[PrefillItem] = field(default_factory=list)
    decodes: list[str] = field(default_factory=list)
    step_token_budget: int = 0
    fast_path: bool = False
    metrics: dict = field(default_factory=dict)

    @property
    def is_empty(self) -> bool:
        return not (self.admissions or self.prefills or self.decodes)

    @property
    def num_tokens(self) -> int:
        return sum(p.chunk_len for p in self.prefills) + len(self.decodes)

    def to_wire(self) -> dict:
        """Compact form broadcast from rank 0 to worker ranks each step."""
        return {"a": self.admissions, "p": [(p.request_id, p.start, p.chunk_len) for p in self.prefills],
                "d": self.decodes, "b": self.step_token_budget, "f": self.fast_path}

    @classmethod
    def from_wire(cls, w: dict) -> "StepPlan":
        return cls(admissions=list(w["a"]), prefills=[PrefillItem(*t) for t in w["p"]],
                   decodes=list(w["d"]), step_token_budget=int(w["b"]), fast_path=bool(w["f"]))
