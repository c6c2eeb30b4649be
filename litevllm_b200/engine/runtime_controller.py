"""One engine step: expire queued requests, plan, admit, grow KV, execute.
Reference: vllm/engine/runtime_controller.py:47-191 (``ExecutionBackend`` protocol :15-36)."""
from __future__ import annotations

import time
from typing import Protocol

from .errors import RequestRejectedError
from .step_plan import StepPlan


class ExecutionBackend(Protocol):
    def ensure_kv_blocks(self, plan: StepPlan) -> None: ...
    def register_admitted(self, st) -> None: ...
    def maybe_apply_prefix_cache(self, st) -> None: ...
    def run_prefills(self, plan: StepPlan) -> list: ...
    def run_decodes(self, plan: StepPlan) -> list: ...
    def decode_step_sync(self, request_id: str) -> list: ...
    def release_request(self, request_id: str) -> None: ...
    def stats(self) -> dict: ...


class RuntimeController:
    def __init__(self, scheduler, step_scheduler, backend: ExecutionBackend, observer, plan_hook=None):
        self.scheduler = scheduler
        self.step_scheduler = step_scheduler
        self.backend = backend
        self.observer = observer
        self.plan_hook = plan_hook      # multi-GPU: rank 0 broadcasts the plan to the workers here
        self.steps = 0
        self.last_plan: StepPlan | None = None

    def _reject_expired(self) -> None:
        for st in self.scheduler.expire_queued():
            err = RequestRejectedError(
                f"request {st.request_id} waited longer than {self.scheduler.queue_timeout_s:g} s in the queue (queue timeout)",
                "queue_timeout")
            self.scheduler.publish_output(st.request_id, err)
            self.observer.on_request_rejected(st.request_id, "queue_timeout")
            self.backend.release_request(st.request_id)

    def _admit(self, plan: StepPlan) -> None:
        now = time.monotonic()
        for rid in plan.admissions:
            st = self.scheduler.admit(rid)
            self.backend.register_admitted(st)
            self.backend.maybe_apply_prefix_cache(st)
            self.observer.on_request_admitted(rid, now - st.arrival_time)
            if st.seq_len > 0:   # a cached prefix moved the start of this request's first chunk
                for it in plan.prefills:
                    if it.request_id == rid:
                        end = max(it.end, min(st.prompt_len, st.seq_len + it.chunk_len))
                        it.start = st.seq_len
                        it.chunk_len = max(0, min(end, st.prompt_len) - st.seq_len)

    def step(self) -> list:
        self._reject_expired()
        plan = self.step_scheduler.build_plan(self.scheduler)
        if self.plan_hook is not None:
            plan = self.plan_hook(plan)
        self.last_plan = plan
        if plan.is_empty:
            return []
        self._admit(plan)
        self.backend.ensure_kv_blocks(plan)
        self.observer.on_step_started(plan)
        self.steps += 1
        if plan.fast_path and len(plan.decodes) == 1:
            return self.backend.decode_step_sync(plan.decodes[0])
        outs = self.backend.run_prefills(plan)
        outs += self.backend.run_decodes(plan)
        return outs

    def stats(self, extra: dict | None = None) -> dict:
        s = {"steps": self.steps, "scheduler": self.scheduler.gauges(), "observer": self.observer.stats(),
             "backend": self.backend.stats()}
        if extra:
            s.update(extra)
        return s
