"""Per-layer LRU of expert weights that are resident in slab slots.

Same observable behaviour as the reference's `ExpertWeightCache`
(utils/eval_core.py:3661-3882): passive LRU on demand accesses, pinned entries
for prefetches, "prefill transient" entries that are evicted first, and an
active-replacement admission path for the prefetch planner.  Here a payload is
whatever the caller stores (the slab slot index in this package); the cache
never touches device memory.

Eviction order when over capacity (first class that has a member, oldest
member of that class):
  1. not pinned, not protected, prefill-transient
  2. not pinned, not protected
  3. not pinned, prefill-transient
  4. not pinned
  5. the oldest entry
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Any, Dict, Iterable, List, Optional, Set


class _Entry:
    __slots__ = ("payload", "pinned", "transient")

    def __init__(self, payload: Any, pinned: bool, transient: bool):
        self.payload, self.pinned, self.transient = payload, pinned, transient


class ExpertWeightCache:
    def __init__(self, capacity: int):
        self.capacity = int(capacity)
        self._order: "OrderedDict[int, _Entry]" = OrderedDict()   # oldest first
        self._last_evicted_transient = False
        self.last_evicted_payload: Any = None

    # -- lookups ------------------------------------------------------------------
    def has(self, expert_id: int) -> bool:
        return expert_id in self._order

    def peek(self, expert_id: int):
        """Payload without touching recency."""
        if self.capacity <= 0:
            return None
        ent = self._order.get(int(expert_id))
        return ent.payload if ent is not None else None

    def get(self, expert_id: int):
        """Payload of a demand access; makes the entry the most recent."""
        if self.capacity <= 0:
            return None
        ent = self._order.get(expert_id)
        if ent is None:
            return None
        self._order.move_to_end(expert_id)
        return ent.payload

    def resident_ids(self) -> List[int]:
        return list(self._order)

    def prefetch_free_slots(self) -> int:
        return max(0, self.capacity - len(self._order))

    def evictable_prefetch_ids(self, protect_ids: Optional[Set[int]] = None) -> List[int]:
        guard = protect_ids or set()
        return [int(k) for k, ent in self._order.items() if not ent.pinned and k not in guard]

    # -- mutation -----------------------------------------------------------------
    def _victim(self, guard: Set[int]) -> int:
        best_key, best_class = None, 5
        for k, ent in self._order.items():           # oldest first: first hit of a class wins
            if ent.pinned:
                continue
            free = int(k) not in guard
            cls = (1 if free else 3) if ent.transient else (2 if free else 4)
            if cls < best_class:
                best_key, best_class = k, cls
                if cls == 1:
                    break
        if best_key is None:
            best_key = next(iter(self._order))
        return best_key

    def put(self, expert_id: int, weights, pinned: bool = False, prefer_hot: bool = False,
            protect_ids: Optional[Set[int]] = None, prefill_scp_transient: bool = False) -> Optional[int]:
        """Insert or refresh after a demand load.  Returns the expert evicted to
        make room (its payload is then in `last_evicted_payload`), or None."""
        if self.capacity <= 0:
            return None
        ent = self._order.get(expert_id)
        if ent is not None:
            ent.payload = weights
            ent.pinned = ent.pinned or bool(pinned)
            ent.transient = ent.transient or bool(prefill_scp_transient)
            self._order.move_to_end(expert_id)
            return None
        self._order[expert_id] = _Entry(weights, bool(pinned), bool(prefill_scp_transient))
        evicted, was_transient = None, False
        guard = protect_ids or set()
        while len(self._order) > self.capacity:
            k = self._victim(guard)
            gone = self._order.pop(k)
            evicted, was_transient = int(k), gone.transient
            self.last_evicted_payload = gone.payload
        self._last_evicted_transient = was_transient
        return evicted

    def admit_prefetch(self, expert_id: int, weights, *, protect_ids: Optional[Set[int]] = None,
                       preferred_victim: Optional[int] = None) -> bool:
        """Admission of a prefetched expert: the entry is pinned until the next
        `unpin_all`.  With a full cache a victim is replaced (the preferred one if
        it may be evicted, else the oldest evictable); False if nothing may go."""
        if self.capacity <= 0:
            return False
        ent = self._order.get(expert_id)
        if ent is not None:
            ent.payload, ent.pinned = weights, True
            self._order.move_to_end(expert_id)
            return True
        if len(self._order) >= self.capacity:
            candidates = self.evictable_prefetch_ids(protect_ids)
            if not candidates:
                return False
            victim = candidates[0]
            if preferred_victim is not None and int(preferred_victim) in candidates:
                victim = int(preferred_victim)
            gone = self._order.pop(victim, None)
            if gone is not None:
                self.last_evicted_payload = gone.payload
        self._order[expert_id] = _Entry(weights, True, False)
        return True

    def discard(self, expert_id: int) -> bool:
        gone = self._order.pop(int(expert_id), None)
        if gone is not None:
            self.last_evicted_payload = gone.payload
        return gone is not None

    def clear(self) -> None:
        self._order.clear()
        self._last_evicted_transient = False

    def unpin(self, expert_id: int) -> None:
        ent = self._order.get(expert_id)
        if ent is not None:
            ent.pinned = False

    def unpin_all(self) -> None:
        for ent in self._order.values():
            ent.pinned = False

    def promote_hot(self, expert_id: int) -> None:
        if expert_id in self._order:
            self._order.move_to_end(expert_id)

    def reset_request_metadata(self, *, unpin: bool = True, demote_hot: bool = False) -> None:
        if unpin:
            self.unpin_all()

    # -- prefill-transient bookkeeping (SCP prefill placement) -------------------------
    def last_evicted_was_prefill_scp_transient(self) -> bool:
        return bool(self._last_evicted_transient)

    def is_prefill_scp_transient(self, expert_id: int) -> bool:
        ent = self._order.get(int(expert_id))
        return bool(ent is not None and ent.transient)

    def clear_prefill_scp_transient(self, expert_id: int) -> bool:
        ent = self._order.get(int(expert_id))
        if ent is None or not ent.transient:
            return False
        ent.transient = False
        return True

    def prefill_scp_transient_ids(self) -> List[int]:
        return [int(k) for k, ent in self._order.items() if ent.transient]

    def demote_prefill_scp_transients(self) -> int:
        """At the prefill->decode boundary: transient entries become the oldest,
        unpinned, so ordinary eviction takes them first."""
        ids = self.prefill_scp_transient_ids()
        for k in ids:
            self._order.move_to_end(k, last=False)
            self._order[k].pinned = False
        return len(ids)

    def occupancy(self) -> Dict[str, int]:
        n = len(self._order)
        return {"capacity": self.capacity, "resident": n, "hot": 0, "transient_demand": n,
                "transient_prefetch": 0, "prefill_scp_transient": len(self.prefill_scp_transient_ids())}


class SlotPool:
    """Free list of slab slots for one layer's cache."""

    def __init__(self, slots: Iterable[int]):
        self._free = list(slots)
        self.total = len(self._free)

    def take(self) -> Optional[int]:
        return self._free.pop() if self._free else None

    def give(self, slot: int) -> None:
        self._free.append(int(slot))

    def __len__(self) -> int:
        return len(self._free)
