"""EPIPE: readiness-aware ordering of expert groups (host decisions only).

The reference classifies the expert segments a rank has to execute by whether
their weights are usable now, starts the copy of ONE unusable expert on a side
stream, computes the usable segments meanwhile, waits for the copy and then
computes the rest (utils/eval_core.py:11867-12167 upfront scan for decode
without a predictor; 12169-12512 residual scan for decode with RS prefetch;
gating at 5585-5598, 12228-12254, 13264-13334).

Here a "segment" is an expert id with rows in this pass; executing a set of
segments is one launch of the grouped GEMM whose slot map marks every other
expert as "skip", so the ordering costs two GEMM launches and no per-expert
Python loop.  This module only decides the order; `store.py` carries it out.

Readiness classes
  ready   resident and no copy pending
  late    resident (admitted by the prefetcher) but its copy event has not completed
  demand  not resident
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Iterable, List, Optional, Sequence, Tuple


@dataclass
class EpipePlan:
    first: List[int]                 # experts computed while the residual's copy runs
    residual: int                    # the one expert whose copy is overlapped
    residual_kind: str               # "late" (copy already in flight) | "demand" (copy started now)
    rest: List[int] = field(default_factory=list)   # everything else, after the residual


def classify(needed: Sequence[int], is_resident: Callable[[int], bool],
             copy_pending: Callable[[int], bool]) -> Tuple[List[int], List[int], List[int]]:
    """(ready, late, demand) in the order of `needed` (ascending expert id)."""
    ready, late, demand = [], [], []
    for e in needed:
        if not is_resident(e):
            demand.append(e)
        elif copy_pending(e):
            late.append(e)
        else:
            ready.append(e)
    return ready, late, demand


def plan_upfront_scan(needed: Sequence[int], is_resident: Callable[[int], bool]) -> Optional[EpipePlan]:
    """Decode without a predictor: overlap the first missing expert's copy with
    all resident experts.  None (= run the plain executor) unless there is at
    least one resident expert to hide the copy behind and one missing expert."""
    ready = [e for e in needed if is_resident(e)]
    missing = [e for e in needed if not is_resident(e)]
    if not ready or not missing:
        return None
    return EpipePlan(first=ready, residual=missing[0], residual_kind="demand", rest=missing[1:])


def plan_residual_scan(needed: Sequence[int], is_resident: Callable[[int], bool],
                       copy_pending: Callable[[int], bool], handle_late: bool = True,
                       handle_demand: bool = True, min_buffer_groups: int = 1) -> Optional[EpipePlan]:
    """Decode with RS prefetch: the residual is the first late expert, else the
    first demand miss; it needs at least `min_buffer_groups` ready experts in
    front of it."""
    ready, late, demand = classify(needed, is_resident, copy_pending)
    if len(ready) < max(1, min_buffer_groups):
        return None
    if late and handle_late:
        residual, kind = late[0], "late"
    elif demand and handle_demand:
        residual, kind = demand[0], "demand"
    else:
        return None
    rest = [e for e in needed if e not in ready and e != residual]
    return EpipePlan(first=ready, residual=residual, residual_kind=kind, rest=rest)


class RollingGate:
    """Skip EPIPE attempts for a while when they rarely find anything to overlap:
    over the last `window` decode steps fewer than `min_triggers` plans -> skip the
    next `skip_steps` steps (utils/eval_core.py:4989-4992, 12228-12254)."""

    def __init__(self, window: int = 16, min_triggers: int = 1, skip_steps: int = 8):
        self.window, self.min_triggers, self.skip_steps = int(window), int(min_triggers), int(skip_steps)
        self.history: Deque[int] = deque(maxlen=max(1, self.window))
        self.skip_left = 0

    def should_attempt(self) -> bool:
        if self.skip_left > 0:
            self.skip_left -= 1
            return False
        return True

    def record(self, triggered: bool) -> None:
        self.history.append(1 if triggered else 0)
        if len(self.history) == self.history.maxlen and sum(self.history) < self.min_triggers:
            self.skip_left = self.skip_steps
            self.history.clear()
