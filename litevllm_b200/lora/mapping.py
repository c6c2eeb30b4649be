"""Token -> adapter mapping of one batch (reference: vllm/lora/mapping.py)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class LoRAMapping:
    segments: list[tuple[str | None, int, int]]   # (adapter name or None, first token row, n rows)

    @classmethod
    def from_segments(cls, names: list[str | None], lengths: list[int]) -> "LoRAMapping":
        segs, off = [], 0
        for name, n in zip(names, lengths):
            segs.append((name, off, n))
            off += n
        return cls(segs)

    @property
    def adapters(self) -> set[str]:
        return {n for n, _, _ in self.segments if n}

    @property
    def is_mixed(self) -> bool:
        return len({n for n, _, _ in self.segments}) > 1

    def rows_of(self, name: str) -> list[tuple[int, int]]:
        """Merged contiguous (start, n) row ranges of one adapter."""
        out: list[tuple[int, int]] = []
        for n, start, cnt in self.segments:
            if n != name or cnt == 0:
                continue
            if out and out[-1][0] + out[-1][1] == start:
                out[-1] = (out[-1][0], out[-1][1] + cnt)
            else:
                out.append((start, cnt))
        return out
