"""Ownership rules for speculative expert staging (no CUDA in this file).

Counterpart of the reference's `utils/rs_staging.py:11-118`:
  * a `Transfer` is one expert payload copied (or being copied) into a staging
    slot, with the event that marks the copy's completion;
  * a `StagingJob` collects the transfers issued for ONE target layer.  A worker
    thread may publish transfers until the layer's demand path closes the job;
    publication and closing exclude each other, so after `close()` returns no
    further copy can be submitted for that layer and every issued copy is
    visible to the demand path - an expert is never loaded twice;
  * a `DemandView` lets the demand path see staged payloads next to the
    resident cache without speculation ever touching LRU state; only payloads
    the demand path really used are remembered, for admission afterwards;
  * `select_candidates` scores predicted experts.
Speculation never writes the resident cache.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Sequence


@dataclass
class Transfer:
    expert: int
    payload: object      # what the demand path consumes (a slab slot in this package)
    event: object        # completion event of the copy
    slot: object         # staging slot to give back afterwards
    nbytes: int
    used: bool = False
    retained: bool = False


class StagingJob:
    """Transfers published for one target layer under one ticket."""

    def __init__(self, ticket, slots):
        self.ticket, self.slots = ticket, slots
        self.transfers: Dict[int, Transfer] = {}
        self.closed = False
        self.lock = threading.Lock()
        self.future = None
        self.plan_count = None

    def publish(self, expert: int, submit: Callable[[], Transfer]) -> bool:
        """Run `submit` (enqueue-only: no event wait, no allocation, no planning)
        and record its transfer, unless the job is already closed."""
        with self.lock:
            if self.closed:
                return False
            tr = submit()
            if tr.expert != expert or expert in self.transfers:
                raise AssertionError("a staging job takes each expert once")
            self.transfers[expert] = tr
            return True

    def close(self) -> Dict[int, Transfer]:
        """Stop publication and hand over what was issued so far."""
        with self.lock:
            self.closed = True
            return dict(self.transfers)


# The reference's name for the same object.
TargetJob = StagingJob


class DemandView:
    """Resident cache plus the staged transfers of the current layer.

    `has` is true for payloads that exist, possibly still in flight; `get` marks
    a staged transfer as used (once) and remembers the order of first use;
    `peek` changes nothing.  Everything else is forwarded to the resident cache.
    """

    def __init__(self, resident):
        self.resident = resident
        self.staged: Dict[int, Transfer] = {}
        self.used_in_order: List[Transfer] = []

    def __getattr__(self, name):
        return getattr(self.resident, name)

    def has(self, expert) -> bool:
        return self.resident.has(expert) or int(expert) in self.staged

    def get(self, expert):
        hit = self.resident.get(expert)
        if hit is not None:
            return hit
        tr = self.staged.get(int(expert))
        if tr is None:
            return None
        if not tr.used:
            tr.used = True
            self.used_in_order.append(tr)
        return tr.payload

    def peek(self, expert):
        hit = self.resident.peek(expert)
        if hit is not None:
            return hit
        tr = self.staged.get(int(expert))
        return tr.payload if tr is not None else None

    def resident_ids(self):
        return self.resident.resident_ids()


DemandCacheView = DemandView


def candidate_scores(ids: Iterable[int], weights: Iterable[float], allowed, resident,
                     diagnostics: Optional[dict] = None) -> Dict[int, float]:
    """score(e) = sum_p * (1 + 0.15*(count-1)) + 0.05 * max_p over the predictions
    of expert e, skipping experts this rank may not hold and experts already
    resident (utils/eval_core.py:10104-10106, utils/rs_staging.py:112-113)."""
    total: Dict[int, float] = {}
    hits: Dict[int, int] = {}
    peak: Dict[int, float] = {}
    foreign = present = 0
    for e, p in zip(ids, weights):
        e, p = int(e), float(p)
        if e not in allowed:
            foreign += 1
        elif e in resident:
            present += 1
        else:
            total[e] = total.get(e, 0.0) + p
            hits[e] = hits.get(e, 0) + 1
            peak[e] = max(peak.get(e, 0.0), p)
    scores = {e: total[e] * (1 + .15 * (hits[e] - 1)) + .05 * peak[e] for e in total}
    if diagnostics is not None:
        diagnostics["nonlocal_entries"] = foreign
        diagnostics["resident_entries"] = present
        diagnostics["scored"] = len(scores)
    return scores


def select_candidates(ids: Sequence[int], weights: Sequence[float], *, allowed, resident,
                      minimum: float, budget: int, diagnostics: Optional[dict] = None) -> List[int]:
    """Best-scoring predicted experts, at most `budget`, each scoring >= `minimum`."""
    scores = candidate_scores(ids, weights, allowed, resident, diagnostics)
    if diagnostics is not None:
        diagnostics["below_threshold"] = sum(1 for v in scores.values() if v < minimum)
    ranked = sorted(scores, key=scores.get, reverse=True)
    return [e for e in ranked if scores[e] >= minimum][:budget]
