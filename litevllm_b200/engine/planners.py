"""Planning stages of one step: admission, token budget, prefill/decode selection.

Policy (reference: vllm/engine/planners/{admission_planner,budget_computer,decode_prefill_planner}.py):
FIFO admission capped per step; decode tokens are budgeted first; waiting prefills get a catch-up
share of the remaining budget that grows with the backlog; a prefill batch is a *varlen* group of up
to ``microbatch`` requests, each contributing ``min(remaining, chunk, budget left)`` tokens (the
reference's rectangular batches required equal processed lengths and a common chunk length; the
flattened token layout removes that restriction).
"""
from __future__ import annotations

from dataclasses import dataclass

from .request_state import RequestState
from .step_plan import PrefillItem


class AdmissionPlanner:
    def __init__(self, max_admit_per_step: int):
        self.max_admit_per_step = max(1, max_admit_per_step)

    def plan(self, queued_ids, free_slots: int) -> list[str]:
        n = min(self.max_admit_per_step, free_slots, len(queued_ids))
        return [queued_ids[i] for i in range(n)]


@dataclass
class Budget:
    total: int
    decode_tokens: int
    prefill_tokens: int
    starvation_override: bool = False


class BudgetComputer:
    def __init__(self, step_token_budget: int, decode_priority: bool = True, catchup_ratio: float = 0.25,
                 reserved_tokens: int = 0, reserve_backlog: int = 2, min_chunk: int = 128):
        self.step_token_budget = step_token_budget
        self.decode_priority = decode_priority
        self.catchup_ratio = catchup_ratio
        self.reserved_tokens = reserved_tokens
        self.reserve_backlog = reserve_backlog
        self.min_chunk = min_chunk

    def compute(self, n_decode: int, n_prefill: int, backlog: int, force_prefill: bool) -> Budget:
        total = self.step_token_budget
        decode_tokens = min(n_decode, total)
        rest = total - decode_tokens
        if n_prefill == 0:
            return Budget(total, decode_tokens, 0)
        if n_decode == 0 or not self.decode_priority or force_prefill:
            return Budget(total, decode_tokens, rest, starvation_override=force_prefill and n_decode > 0)
        ratio = self.catchup_ratio
        if backlog > self.reserve_backlog:
            ratio = min(1.0, ratio * (1 + backlog - self.reserve_backlog))
        share = max(self.reserved_tokens, self.min_chunk, int(total * ratio))
        return Budget(total, decode_tokens, min(rest, share))


class DecodePrefillPlanner:
    def __init__(self, chunk_size: int, microbatch: int, min_chunk: int = 128, max_chunk: int | None = None,
                 verified_decode_batch_sizes: tuple[int, ...] | None = None):
        self.chunk_size = chunk_size
        self.microbatch = max(1, microbatch)
        self.min_chunk = min_chunk
        self.max_chunk = max_chunk
        self.verified_decode_batch_sizes = tuple(sorted(verified_decode_batch_sizes)) if verified_decode_batch_sizes else None

    def build_prefill_plan(self, prefill_reqs: list[RequestState], budget_tokens: int) -> list[PrefillItem]:
        items: list[PrefillItem] = []
        left = budget_tokens
        chunk_cap = self.chunk_size if self.max_chunk is None else min(self.chunk_size, self.max_chunk)
        for st in prefill_reqs:
            if len(items) >= self.microbatch or left <= 0:
                break
            remaining = st.remaining_prefill
            if remaining <= 0:
                continue
            n = min(remaining, chunk_cap, left)
            # do not shred a prompt into slivers unless it is the tail of the prompt
            if n < min(self.min_chunk, remaining) and items:
                break
            items.append(PrefillItem(st.request_id, st.seq_len, n))
            left -= n
        return items

    def build_decode_plan(self, decode_reqs: list[RequestState], budget_tokens: int) -> list[str]:
        ids = [st.request_id for st in decode_reqs[:max(0, budget_tokens)]]
        if self.verified_decode_batch_sizes and ids:
            ok = [b for b in self.verified_decode_batch_sizes if b <= len(ids)]
            ids = ids[: (ok[-1] if ok else 1)]
        return ids
