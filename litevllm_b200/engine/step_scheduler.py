"""Builds one :class:`StepPlan` per engine step from the scheduler state.

Starvation guards: after ``max_decode_streak`` decode-only steps with a prefill waiting, or once a
prefill has been deferred ``max_prefill_deferrals`` times, the prefill is forced with the full
remaining budget.  Reference: vllm/engine/step_scheduler.py:53-157.
"""
from __future__ import annotations

from ..config.runtime_policy import SchedulerRuntimePolicy
from .planners import AdmissionPlanner, BudgetComputer, DecodePrefillPlanner
from .request_scheduler import RequestScheduler
from .step_plan import StepPlan


class StepScheduler:
    def __init__(self, step_token_budget: int, prefill_chunk_size: int, prefill_microbatch: int,
                 policy: SchedulerRuntimePolicy | None = None, decode_priority: bool = True,
                 catchup_ratio: float = 0.25, reserved_tokens: int = 0, reserve_backlog: int = 2,
                 min_chunk: int = 128, max_chunk: int | None = None,
                 verified_decode_batch_sizes: tuple[int, ...] | None = None, max_active: int = 16):
        self.policy = policy or SchedulerRuntimePolicy()
        self.admission = AdmissionPlanner(min(self.policy.max_admit_per_step, max_active) if max_active < 8
                                          else max(self.policy.max_admit_per_step, max_active))
        self.budget = BudgetComputer(step_token_budget, decode_priority, catchup_ratio, reserved_tokens,
                                     reserve_backlog, min_chunk)
        self.planner = DecodePrefillPlanner(prefill_chunk_size, prefill_microbatch, min_chunk, max_chunk,
                                            verified_decode_batch_sizes)
        self.decode_streak = 0

    def build_plan(self, sched: RequestScheduler) -> StepPlan:
        # fast path: exactly one running request in decode and nothing waiting
        if len(sched.running) == 1 and not sched.queued:
            st = sched.requests[sched.running[0]]
            if not st.is_prefill:
                self.decode_streak = 0
                return StepPlan(decodes=[st.request_id], step_token_budget=self.budget.step_token_budget,
                                fast_path=True, metrics={"fast_path": True})
        admissions = self.admission.plan(sched.queued, len(sched.free_slots))
        prefill, decode = sched.classify_requests()
        # requests admitted this step start prefilling in the same step
        admitted_states = [sched.requests[r] for r in admissions]
        prefill = prefill + admitted_states
        starving = any(st.prefill_deferrals >= self.policy.max_prefill_deferrals for st in prefill)
        force = bool(prefill) and (self.decode_streak >= self.policy.max_decode_streak or starving)
        b = self.budget.compute(len(decode), len(prefill), len(sched.queued) - len(admissions) + len(prefill), force)
        decodes = self.planner.build_decode_plan(decode, b.decode_tokens)
        prefills = self.planner.build_prefill_plan(prefill, b.prefill_tokens)
        planned = {p.request_id for p in prefills}
        for st in prefill:
            if st.request_id in planned:
                st.prefill_deferrals = 0
            else:
                st.prefill_deferrals += 1
        if decodes and not prefills and prefill:
            self.decode_streak += 1
        else:
            self.decode_streak = 0
        return StepPlan(admissions=admissions, prefills=prefills, decodes=decodes,
                        step_token_budget=b.total,
                        metrics={"starvation_override": b.starvation_override or force,
                                 "decode_streak": self.decode_streak, "prefill_budget": b.prefill_tokens})
