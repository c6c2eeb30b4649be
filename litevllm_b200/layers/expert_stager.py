"""Routed-expert weights that do not fit the device: host-resident payloads with a byte-budgeted set of device slots.

A checkpoint whose routed experts exceed what one GPU should spend on them keeps the raw expert payloads (GGUF
blocks, packed int4, any tensor with a leading expert dimension) in pinned host memory.  The device holds a slab of
``slots`` expert-sized entries per tensor.  Before a MoE block runs, the experts that the step's routes name are
made resident: hits are refreshed in a least-recently-used order, misses are copied into a free slot or over the
least recently used entry, and experts marked hot are never evicted.  The block then runs on the slab with the
routes renumbered to slot numbers.  A step that names more experts than there are slots runs in waves; every
route is served in exactly one wave.

Copies are issued on the launching stream from immutable pinned memory, so a slot is never overwritten while a
kernel that reads it is still queued in front of the copy.

Behavioural contract (byte budget, least-recently-used eviction, pinned hot experts, raw-payload staging):
vllm/model_executor/models/deepseek_v4_flash/gpu_weight_staging.py:76-793 and the dense-expert cache of
vllm/model_executor/models/gemma4/moe.py:331-392 of the reference.
"""
from __future__ import annotations

import os
from collections import OrderedDict
from collections.abc import Iterable, Sequence

import torch


def budget_bytes_from_env(default: float | None = None) -> int | None:
    """``FI_EXPERT_STAGING_GB``: device bytes that all routed experts of the model together may occupy.
    Unset or empty: everything stays resident."""
    raw = os.environ.get("FI_EXPERT_STAGING_GB", "")
    if not raw.strip():
        return None if default is None else int(default * 2 ** 30)
    value = float(raw)
    if value <= 0:
        raise ValueError("FI_EXPERT_STAGING_GB must be positive")
    return int(value * 2 ** 30)


def auto_pin_from_env() -> tuple[int, int]:
    """``FI_EXPERT_STAGING_PIN_HOT="n"`` or ``"n@steps"``: after ``steps`` staged steps of a block (default 64)
    its ``n`` most used experts are pinned.  (0, 0): no automatic pinning."""
    raw = os.environ.get("FI_EXPERT_STAGING_PIN_HOT", "").strip()
    if not raw:
        return 0, 0
    n, _, after = raw.partition("@")
    n, after = int(n), int(after or 64)
    if n < 0 or after < 1:
        raise ValueError("FI_EXPERT_STAGING_PIN_HOT: expected n or n@steps with n >= 0 and steps >= 1")
    return n, after


class ExpertStager:
    """Device slots for the experts of one MoE block.

    ``host``: name -> tensor ``[E, ...]`` (kept by reference; pinned by the caller where the device is a GPU).
    ``budget_bytes``: device bytes this block may use for expert payloads; at least ``min_slots`` slots are
    allocated whatever the budget says, and never more than ``E``.
    """

    def __init__(self, host: dict[str, torch.Tensor], device, budget_bytes: int, min_slots: int = 1):
        if not host:
            raise ValueError("no expert tensors to stage")
        self.names = sorted(host)
        counts = {int(host[k].shape[0]) for k in self.names}
        if len(counts) != 1:
            raise ValueError(f"expert tensors disagree on the number of experts: {sorted(counts)}")
        self.num_experts = counts.pop()
        self.host = host
        self.device = torch.device(device)
        self.bytes_per_expert = sum(int(host[k][0].numel()) * host[k].element_size() for k in self.names)
        self.slots = int(max(min_slots, min(self.num_experts, budget_bytes // max(1, self.bytes_per_expert))))
        self.slab = {k: torch.zeros((self.slots, *host[k].shape[1:]), dtype=host[k].dtype, device=self.device)
                     for k in self.names}
        self._slot_of: dict[int, int] = {}
        self._lru: OrderedDict[int, None] = OrderedDict()       # resident and evictable, oldest first
        self._free = list(range(self.slots - 1, -1, -1))
        self._pinned: set[int] = set()
        self.use_counts = [0] * self.num_experts
        self.stats = {"hits": 0, "misses": 0, "evictions": 0, "bytes_staged": 0, "waves": 0, "steps": 0}
        self.auto_pin = auto_pin_from_env()

    def begin_step(self) -> None:
        """Counts a step of the block and applies the automatic pinning once its step count is reached."""
        self.stats["steps"] += 1
        n, after = self.auto_pin
        if n and self.stats["steps"] == after + 1:
            self.pin_hot(n)

    # ---- residency ------------------------------------------------------------------------------------------
    @property
    def device_bytes(self) -> int:
        return self.slots * self.bytes_per_expert

    def resident(self) -> list[int]:
        return sorted(self._slot_of)

    def pinned(self) -> list[int]:
        return sorted(self._pinned)

    def slot_of(self, expert: int) -> int:
        return self._slot_of.get(expert, -1)

    def pin(self, experts: Iterable[int]) -> None:
        """Make ``experts`` resident for good.  At least one slot stays evictable, so that any step can run."""
        experts = [int(e) for e in experts if int(e) not in self._pinned]
        if len(self._pinned) + len(experts) > self.slots - 1 and self.slots < self.num_experts:
            raise ValueError(f"cannot pin {len(self._pinned) + len(experts)} experts in {self.slots} slots: "
                             "one slot has to stay evictable")
        for e in experts:
            self._check(e)
            self._make_resident(e, keep=set(experts) | self._pinned)
            self._lru.pop(e, None)
            self._pinned.add(e)

    def unpin(self, experts: Iterable[int] | None = None) -> None:
        for e in list(self._pinned if experts is None else experts):
            if e in self._pinned:
                self._pinned.discard(e)
                self._lru[e] = None

    def pin_hot(self, n: int) -> list[int]:
        """Pin the ``n`` most used experts so far (ties by expert number); returns them."""
        n = max(0, min(n, self.slots - 1 if self.slots < self.num_experts else self.slots))
        order = sorted(range(self.num_experts), key=lambda e: (-self.use_counts[e], e))[:n]
        self.unpin()
        self.pin(order)
        return order

    def _check(self, e: int) -> None:
        if not 0 <= e < self.num_experts:
            raise IndexError(f"expert {e} outside 0..{self.num_experts - 1}")

    def _make_resident(self, e: int, keep: set[int]) -> int:
        slot = self._slot_of.get(e)
        if slot is not None:
            self.stats["hits"] += 1
            if e in self._lru:
                self._lru.move_to_end(e)
            return slot
        self.stats["misses"] += 1
        if self._free:
            slot = self._free.pop()
        else:
            victim = next((v for v in self._lru if v not in keep), None)
            if victim is None:
                raise RuntimeError("no evictable slot: the wave names more experts than there are slots")
            del self._lru[victim]
            slot = self._slot_of.pop(victim)
            self.stats["evictions"] += 1
        with torch.inference_mode():        # the slab may have been allocated inside the engine's inference mode
            for k in self.names:
                self.slab[k][slot].copy_(self.host[k][e], non_blocking=True)
        self.stats["bytes_staged"] += self.bytes_per_expert
        self._slot_of[e] = slot
        self._lru[e] = None
        return slot

    # ---- a step ---------------------------------------------------------------------------------------------
    def waves(self, experts: Sequence[int]) -> list[list[int]]:
        """Split the experts of one step into groups that fit the slots together.  Resident experts come first,
        so a step that fits needs no eviction of what it is about to use."""
        need = sorted({int(e) for e in experts})
        for e in need:
            self._check(e)
        hot = [e for e in need if e in self._pinned]
        rest = sorted((e for e in need if e not in self._pinned), key=lambda e: (e not in self._slot_of, e))
        room = self.slots - len(self._pinned)
        if rest and room <= 0:
            raise RuntimeError("every slot is pinned")
        groups = [rest[i:i + room] for i in range(0, len(rest), room)] if rest else []
        if not groups:
            return [hot] if hot else []
        groups[0] = hot + groups[0]
        return groups

    def stage(self, wave: Sequence[int]) -> dict[int, int]:
        """Make every expert of ``wave`` resident at once; returns expert -> slot."""
        keep = set(wave) | self._pinned
        if len(keep) > self.slots:
            raise RuntimeError(f"a wave of {len(wave)} experts plus {len(self._pinned - set(wave))} pinned ones "
                               f"exceeds {self.slots} slots")
        self.stats["waves"] += 1
        out = {}
        for e in wave:
            self.use_counts[e] += 1
            out[e] = self._make_resident(e, keep)
        return out

    def slot_ids(self, ids: torch.Tensor, placed: dict[int, int], e_lo: int = 0) -> torch.Tensor:
        """Routes renumbered for one wave: the slot of experts in ``placed``, -1 for every other route (served
        by another wave or another rank).  ``ids`` hold global expert numbers, this block owns
        ``[e_lo, e_lo + num_experts)``."""
        E = self.num_experts
        table = torch.full((E + 1,), -1, dtype=torch.int32)
        if placed:
            table[torch.tensor(list(placed.keys()), dtype=torch.long)] = torch.tensor(list(placed.values()), dtype=torch.int32)
        table = table.to(ids.device)
        local = ids.long() - e_lo
        local = torch.where((local < 0) | (local >= E), torch.full_like(local, E), local)
        return table[local].to(ids.dtype) if ids.dtype in (torch.int32, torch.int64) else table[local]

    def snapshot(self) -> dict:
        s = dict(self.stats)
        total = s["hits"] + s["misses"]
        s.update(slots=self.slots, experts=self.num_experts, resident=len(self._slot_of), pinned=len(self._pinned),
                 device_bytes=self.device_bytes, host_bytes=self.num_experts * self.bytes_per_expert,
                 hit_rate=(s["hits"] / total) if total else 0.0)
        return s


def stagers_of(model) -> list[ExpertStager]:
    """Every live stager of a model: attributes named ``stager`` of its modules, and of the ``routed`` members of
    its layers (model-owned data planes keep their expert blocks outside the module tree)."""
    found = []
    holders = list(model.modules()) if hasattr(model, "modules") else []
    holders += [getattr(l, "routed", None) for l in getattr(model, "layers", [])]
    for h in holders:
        st = getattr(h, "stager", None)
        if isinstance(st, ExpertStager) and all(st is not f for f in found):
            found.append(st)
    return found


def summary(model) -> dict:
    """Totals over the model's stagers; empty when nothing is staged."""
    sts = stagers_of(model)
    if not sts:
        return {}
    keys = ("hits", "misses", "evictions", "bytes_staged", "waves", "steps")
    out = {k: sum(st.stats[k] for st in sts) for k in keys}
    total = out["hits"] + out["misses"]
    out.update(blocks=len(sts), slots_per_block=sts[0].slots, experts_per_block=sts[0].num_experts,
               pinned=sum(len(st.pinned()) for st in sts), device_bytes=sum(st.device_bytes for st in sts),
               host_bytes=sum(st.num_experts * st.bytes_per_expert for st in sts),
               hit_rate=(out["hits"] / total) if total else 0.0)
    return out


def pin_hot_experts(model, per_block: int) -> int:
    """Pin each block's ``per_block`` most used experts (by the traffic seen so far); returns how many were pinned."""
    return sum(len(st.pin_hot(per_block)) for st in stagers_of(model))
