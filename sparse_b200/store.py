"""Expert weight residency on one GPU: slab slots, the LRU, and the copy streams.

The reference keeps every expert's weights in pinned host memory
(`expert_offload="cpu"`), a per-layer LRU of device payloads, and loads a missing
expert with three `.to(device, non_blocking=True)` copies on the compute stream
(utils/eval_core.py:11388-11435), or ahead of time on `prefetch_stream`
(9970-9984, 10433-10527) or `epipe_stream` (11626-11633).  Here the device side
is a preallocated slab of slots (`LayerWeights.w13/w2`), a payload is a slot
index, and a copy is two `sb_slot_copy_async` calls (gate/up slab row, down slab
row) from pinned host memory or from the owner GPU's slab over NVLink.  Nothing
is allocated after construction.

Cross-stream safety: a slot is overwritten by a side-stream copy only after the
side stream has waited for the compute stream's last GEMM that could read it
(`note_compute_done`), and a consumer waits for the slot's copy event before its
GEMM (`wait_ready`).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Set, Tuple

import torch

from . import _lib, ops
from ._lib import DECODE_MAX_TOKENS
from .cache import ExpertWeightCache, SlotPool
from .config import BlockConfig
from .context import Metrics, SparseContext
from .epipe import EpipePlan, RollingGate, plan_residual_scan, plan_upfront_scan
from .layer import LayerWeights, pack_w13

SLOT_SKIP = -2      # slot_of_expert value: not part of this GEMM launch
SLOT_ABSENT = -1    # slot_of_expert value: not resident (routing to it is an error)


class HostExperts:
    """Pinned host copies of expert weights in slab layout: w13 [2I,H], w2 [H,I] per expert."""

    def __init__(self, hidden: int, inter: int):
        self.hidden, self.inter = hidden, inter
        self.w13: Dict[int, torch.Tensor] = {}
        self.w2: Dict[int, torch.Tensor] = {}

    def add(self, expert: int, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, pin: bool = True) -> None:
        w13 = pack_w13(gate.to(torch.bfloat16), up.to(torch.bfloat16)).contiguous()
        w2 = down.to(torch.bfloat16).contiguous()
        if pin and torch.cuda.is_available():
            w13, w2 = w13.pin_memory(), w2.pin_memory()
        self.w13[expert], self.w2[expert] = w13, w2

    def __contains__(self, expert: int) -> bool:
        return expert in self.w13

    def nbytes(self, expert: int) -> int:
        return self.w13[expert].numel() * 2 + self.w2[expert].numel() * 2


class ExpertStore:
    """Residency manager of one layer on one GPU."""

    def __init__(self, weights: LayerWeights, host: HostExperts, cache_capacity: int,
                 staging_slots: int = 1, resident: Sequence[int] = (), cfg: Optional[BlockConfig] = None,
                 metrics: Optional[Metrics] = None, layer_idx: int = 0, peers=None):
        """`peers`: a `peer_cache.PeerExperts` naming, for experts without a host
        copy here, the owner GPU's slab rows to copy from over NVLink."""
        need = len(resident) + cache_capacity + staging_slots
        if weights.n_slots < need:
            raise RuntimeError("slab has %d slots, need %d (resident %d + cache %d + staging %d)" % (
                weights.n_slots, need, len(resident), cache_capacity, staging_slots))
        self.w, self.host, self.cfg = weights, host, cfg or BlockConfig()
        self.peers = peers
        self.metrics, self.layer_idx = metrics, layer_idx
        self.device = weights.device
        self.num_experts = weights.num_experts
        self.cache = ExpertWeightCache(cache_capacity)
        self.fixed: Dict[int, int] = {e: s for s, e in enumerate(resident)}     # never evicted
        base = len(resident)
        self.pool = SlotPool(range(base, base + cache_capacity))
        self.staging = SlotPool(range(base + cache_capacity, base + cache_capacity + staging_slots))
        self.events: Dict[int, torch.cuda.Event] = {}       # expert -> copy completion event
        self.prefetched_this_group: Set[int] = set()
        self.used_this_group: Set[int] = set()
        self.access_freq: Dict[int, int] = {}
        self.last_used_decode_step: Dict[int, int] = {}
        on_gpu = self.device.type == "cuda"
        self.prefetch_stream = torch.cuda.Stream(device=self.device) if on_gpu else None
        self.epipe_stream = torch.cuda.Stream(device=self.device) if on_gpu else None
        self._compute_done: Optional[torch.cuda.Event] = None
        self.view = None        # DemandView installed by the bounded stager
        # host mirror of slot_of_expert, pushed to the device before a GEMM launch
        self._ring = [torch.empty((self.num_experts,), dtype=torch.int32).pin_memory() if on_gpu
                      else torch.empty((self.num_experts,), dtype=torch.int32) for _ in range(16)]
        self._ring_events: List[Optional[torch.cuda.Event]] = [None] * len(self._ring)
        self._ring_pos = 0
        self.gate = RollingGate(self.cfg.epipe_gate_window, self.cfg.epipe_gate_min_triggers,
                                self.cfg.epipe_gate_skip_steps)

    # -- queries ------------------------------------------------------------------
    def slot_of(self, expert: int) -> Optional[int]:
        if expert in self.fixed:
            return self.fixed[expert]
        return self.cache.peek(expert)

    def is_resident(self, expert: int) -> bool:
        if expert in self.fixed or self.cache.has(expert):
            return True
        return self.view is not None and expert in self.view.staged

    def copy_pending(self, expert: int) -> bool:
        ev = self.events.get(expert)
        return ev is not None and not ev.query()

    # -- copies -------------------------------------------------------------------
    def _copy_into(self, slot: int, expert: int, stream: torch.cuda.Stream, prefetch: bool) -> None:
        if expert not in self.host:
            if self.peers is None or expert not in self.peers:
                raise RuntimeError("expert %d has neither a host copy nor a peer copy on this rank" % expert)
            # owner GPU's slab rows -> this slot, two plain async copies over NVLink
            n = self.peers.copy_into(self.w, slot, expert, stream)
            if self.metrics is not None:
                self.metrics.expert_weight_peer_bytes += n
                if prefetch:
                    self.metrics.expert_weight_peer_prefetch_bytes += n
                else:
                    self.metrics.expert_weight_peer_demand_bytes += n
            return
        ops.slot_copy_async(self.w.w13[slot], self.host.w13[expert], stream, _lib.SB_COPY_HOST_TO_DEVICE)
        ops.slot_copy_async(self.w.w2[slot], self.host.w2[expert], stream, _lib.SB_COPY_HOST_TO_DEVICE)
        if self.metrics is not None:
            n = self.host.nbytes(expert)
            self.metrics.expert_weight_h2d_bytes += n
            if prefetch:
                self.metrics.expert_weight_h2d_prefetch_bytes += n
            else:
                self.metrics.expert_weight_h2d_demand_bytes += n

    def note_compute_done(self) -> None:
        """Record, on the compute stream, that every GEMM launched so far has been enqueued."""
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self._compute_done = ev

    def _side_stream_may_overwrite(self, stream: torch.cuda.Stream) -> None:
        if self._compute_done is not None:
            stream.wait_event(self._compute_done)

    def wait_ready(self, expert: int) -> None:
        """Make the compute stream wait for the expert's copy, if one is in flight."""
        ev = self.events.get(expert)
        if ev is None:
            return
        if ev.query():
            if self.metrics is not None and expert in self.prefetched_this_group:
                self.metrics.prefetch_complete_before_use_count += 1
        else:
            torch.cuda.current_stream(self.device).wait_event(ev)
            if self.metrics is not None:
                self.metrics.prefetch_late_count += 1
        self.events.pop(expert, None)

    # -- demand path --------------------------------------------------------------
    def _take_cache_slot(self, expert: int, protect: Set[int], transient: bool,
                         wave: Set[int]) -> Optional[int]:
        slot = self.pool.take()
        if slot is not None:
            self.cache.put(expert, slot, protect_ids=protect, prefill_scp_transient=transient)
            return slot
        # Full.  The reference may evict an expert it has just used because it runs
        # one expert at a time; a grouped launch needs all experts of the launch
        # resident together, so an eviction that would hit the current launch
        # group ("wave") is refused and the caller flushes the group first.
        victim = self.cache._victim(protect)
        if victim in wave:
            return None
        evicted = self.cache.put(expert, -1, protect_ids=protect, prefill_scp_transient=transient)
        if evicted is None or evicted == expert:
            raise RuntimeError("expert cache of layer %d cannot make room (capacity %d)" % (
                self.layer_idx, self.cache.capacity))
        slot = int(self.cache.last_evicted_payload)
        pending = self.events.pop(evicted, None)
        if pending is not None and not pending.query():
            # a speculative copy into this slot is still in flight: order our copy after it
            torch.cuda.current_stream(self.device).wait_event(pending)
        self.prefetched_this_group.discard(evicted)
        self.cache.put(expert, slot)
        return slot

    def demand(self, expert: int, protect: Optional[Set[int]] = None, transient: bool = False,
               wave: Optional[Set[int]] = None) -> Optional[int]:
        """Slot of `expert` for immediate use; loads it on the compute stream on a
        miss.  `wave` = experts already made resident for the GEMM launch being
        assembled; returns None if room could only be made by evicting one of
        them (the caller launches what it has and starts a new wave)."""
        self.access_freq[expert] = self.access_freq.get(expert, 0) + 1
        if SparseContext.current_phase == "decode":
            self.last_used_decode_step[expert] = SparseContext.runtime_call_id
        if expert in self.fixed:
            return self.fixed[expert]
        slot = self.cache.get(expert)
        if slot is not None:
            if self.metrics is not None:
                self.metrics.cache_hit_count += 1
            if expert in self.prefetched_this_group:
                self.used_this_group.add(expert)
            self.wait_ready(expert)
            return int(slot)
        if self.view is not None and expert in self.view.staged:
            # issued speculatively into a staging slot; use it there, LRU admission comes later
            slot = self.view.get(expert)
            if self.metrics is not None:
                self.metrics.cache_hit_count += 1
            self.used_this_group.add(expert)
            self.wait_ready(expert)
            return int(slot)
        if self.cache.capacity <= 0:
            raise RuntimeError("expert %d of layer %d is not resident and the cache has no capacity" % (
                expert, self.layer_idx))
        slot = self._take_cache_slot(expert, protect or set(), transient, wave or set())
        if slot is None:
            self.access_freq[expert] -= 1
            return None
        if self.metrics is not None:
            self.metrics.cache_miss_count += 1
        stream = torch.cuda.current_stream(self.device)
        timing = self.metrics is not None and self.cfg.demand_h2d_timing
        if timing:
            t0 = torch.cuda.Event(enable_timing=True)
            t0.record(stream)
        self._copy_into(slot, expert, stream, prefetch=False)
        if timing:
            t1 = torch.cuda.Event(enable_timing=True)
            t1.record(stream)
            self.metrics.pending_events.append(("demand_h2d", SparseContext.current_phase or "prefill", t0, t1))
        return slot

    # -- prefetch path ------------------------------------------------------------
    def protect_ids(self) -> Set[int]:
        """Residents the planner may not evict: prefetched or used in this group, and
        experts used within the last `recent_protect_steps` decode steps
        (utils/eval_core.py:9651-9665)."""
        guard = set(self.prefetched_this_group) | set(self.used_this_group)
        steps = self.cfg.recent_protect_steps
        if steps > 0 and SparseContext.current_phase == "decode" and SparseContext.runtime_call_id >= 0:
            now = SparseContext.runtime_call_id
            guard.update(e for e, s in self.last_used_decode_step.items() if now - s <= steps)
        return guard

    def keep_bias(self, expert: int) -> float:
        bias = 0.02 * float(min(self.access_freq.get(expert, 0), 16))
        if expert in self.prefetched_this_group:
            bias += 0.10
        return bias

    def admit_prefetch_plan(self, plan: Sequence[Tuple[int, Optional[int]]]) -> int:
        """Issue the planned copies on the prefetch stream and admit them (pinned)
        into the LRU.  Returns the number admitted."""
        if not plan:
            return 0
        if self.metrics is not None:
            self.metrics.prefetch_issued_count += len(plan)
        admitted = 0
        protect = self.protect_ids()
        for expert, victim in plan:
            if self.cache.has(expert):
                if self.cache.admit_prefetch(expert, self.cache.get(expert), protect_ids=protect,
                                             preferred_victim=victim):
                    self.prefetched_this_group.add(expert)
                    protect.add(expert)
                    admitted += 1
                continue
            if victim is not None and self.cache.has(victim):
                self.cache.discard(victim)
                self.pool.give(int(self.cache.last_evicted_payload))
                self.events.pop(victim, None)
            slot = self.pool.take()
            if slot is None:
                continue
            self._side_stream_may_overwrite(self.prefetch_stream)
            self._copy_into(slot, expert, self.prefetch_stream, prefetch=True)
            ev = torch.cuda.Event()
            ev.record(self.prefetch_stream)
            if not self.cache.admit_prefetch(expert, slot, protect_ids=protect, preferred_victim=None):
                self.pool.give(slot)
                continue
            self.events[expert] = ev
            self.prefetched_this_group.add(expert)
            protect.add(expert)
            admitted += 1
        if self.metrics is not None:
            self.metrics.prefetch_admitted_count += admitted
        return admitted

    def end_prefetch_group(self) -> None:
        """New planning cycle: prefetch pins are dropped and unused prefetches counted."""
        if self.metrics is not None:
            self.metrics.prefetch_wasted_count += len(self.prefetched_this_group - self.used_this_group)
            self.metrics.prefetch_completed_count += len(self.prefetched_this_group)
        self.cache.unpin_all()
        self.prefetched_this_group.clear()
        self.used_this_group.clear()

    # -- slot map -----------------------------------------------------------------
    def push_slot_map(self, active: Optional[Iterable[int]] = None, needed: Optional[Iterable[int]] = None,
                      overrides: Optional[Dict[int, int]] = None) -> None:
        """Write slot_of_expert for the next GEMM launch on the compute stream.
        `active` = experts this launch computes (others that are `needed` become
        SLOT_SKIP); None = every resident expert is active.  `overrides` maps
        experts to slots outside the LRU (a transient staging slot)."""
        i = self._ring_pos
        self._ring_pos = (i + 1) % len(self._ring)
        if self._ring_events[i] is not None:
            self._ring_events[i].synchronize()
        row = self._ring[i]
        row.fill_(SLOT_ABSENT)
        for e, s in self.fixed.items():
            row[e] = s
        for e in self.cache.resident_ids():
            row[e] = int(self.cache.peek(e))
        if self.view is not None:
            for e, tr in self.view.staged.items():
                if tr.used and not self.cache.has(e):
                    row[e] = int(tr.payload)
        for e, slot in (overrides or {}).items():
            row[e] = slot
        if active is not None:
            act = set(active)
            for e in (needed if needed is not None else range(self.num_experts)):
                if e not in act:
                    row[e] = SLOT_SKIP
        self.w.slot_of_expert.copy_(row, non_blocking=True)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._ring_events[i] = ev

    def stage_transient(self, expert: int) -> Tuple[int, torch.cuda.Event]:
        """Copy `expert` into a staging slot on the EPIPE stream without touching
        the LRU.  Returns (slot, completion event)."""
        slot = self.staging.take()
        if slot is None:
            raise RuntimeError("no staging slot free in layer %d" % self.layer_idx)
        self._side_stream_may_overwrite(self.epipe_stream)
        self._copy_into(slot, expert, self.epipe_stream, prefetch=False)
        ev = torch.cuda.Event()
        ev.record(self.epipe_stream)
        return slot, ev

    def clear(self) -> None:
        for e in self.cache.resident_ids():
            self.pool.give(int(self.cache.peek(e)))
        self.cache.clear()
        self.events.clear()
        self.prefetched_this_group.clear()
        self.used_this_group.clear()


class CachedLayerRunner:
    """Layer pass with offloaded experts: router -> permute -> (read back which
    experts have rows) -> make them resident, ordered by readiness -> grouped
    GEMM(s) -> shared expert -> combine.

    The one host synchronisation is the read-back of the E+1 expert offsets
    (the reference synchronises on `.tolist()` of the unique expert ids and once
    more per segment, utils/eval_core.py:13204-13208, 13257-13258)."""

    def __init__(self, store: ExpertStore, top_k: int, renorm: bool = False, fp32_logits: bool = False):
        self.store, self.top_k, self.renorm, self.fp32_logits = store, top_k, renorm, fp32_logits
        w = store.w
        self.status = torch.zeros((1,), dtype=torch.int32, device=w.device)
        self._offsets_host = torch.empty((w.num_experts + 1,), dtype=torch.int32).pin_memory()
        self.last_plan: Optional[EpipePlan] = None
        self.last_needed: List[int] = []
        self.launches = 0

    def _needed_experts(self, expert_offsets: torch.Tensor) -> List[int]:
        self._offsets_host.copy_(expert_offsets, non_blocking=True)
        torch.cuda.current_stream(self.store.device).synchronize()
        off = self._offsets_host.tolist()
        return [e for e in range(len(off) - 1) if off[e + 1] > off[e]]

    def _epipe_plan(self, needed: List[int], stage: str) -> Optional[EpipePlan]:
        st, cfg = self.store, self.store.cfg
        if not cfg.epipe_enable:
            return None
        if stage == "prefill" and not cfg.epipe_prefill_enable:
            return None
        if stage != "decode" and cfg.epipe_decode_only:
            return None
        metrics = st.metrics
        if metrics is not None:
            metrics.epipe_attempt_count += 1
        use_rs = cfg.epipe_decode_rs_mode == "residual_scan" and bool(st.prefetched_this_group or st.events)
        if cfg.epipe_rolling_gate and not st.gate.should_attempt():
            return None
        if use_rs:
            plan = plan_residual_scan(needed, st.is_resident, st.copy_pending,
                                      cfg.epipe_handle_late_prefetch, cfg.epipe_handle_demand_miss)
        else:
            plan = plan_upfront_scan(needed, st.is_resident)
        if cfg.epipe_rolling_gate:
            st.gate.record(plan is not None)
        if metrics is not None:
            if plan is None:
                metrics.epipe_fallback_count += 1
            else:
                metrics.epipe_trigger_count += 1
                metrics.epipe_ready_group_count += len(plan.first)
        return plan

    def run_routed(self, needed: List[int], gemm, plan: Optional[EpipePlan]) -> None:
        """Make the `needed` experts resident and call `gemm()` (a grouped launch
        over the current slot map) on them: one launch when the cache holds them
        all, several waves otherwise, in readiness order when `plan` says so."""
        st, w = self.store, self.store.w
        protect = set(needed)
        self.launch_groups = 0

        def run_group(experts, overrides=None):
            """Make `experts` resident and launch the grouped GEMM on them, in as
            few launches as the cache capacity allows (normally one)."""
            wave: List[int] = []
            for e in experts:
                if overrides and e in overrides:
                    wave.append(e)
                    continue
                slot = st.demand(e, protect, wave=set(wave))
                if slot is None:
                    st.push_slot_map(active=wave, needed=needed, overrides=overrides)
                    gemm()
                    self.launch_groups += 1
                    wave = []
                    slot = st.demand(e, protect, wave=set())
                    if slot is None:
                        raise RuntimeError("expert cache of layer %d cannot hold a single expert" % st.layer_idx)
                wave.append(e)
            if wave:
                st.push_slot_map(active=wave, needed=needed, overrides=overrides)
                gemm()
                self.launch_groups += 1

        if plan is None:
            run_group(needed)
        else:
            staged_slot = None
            stage_event = None
            if plan.residual_kind == "demand":
                staged_slot, stage_event = st.stage_transient(plan.residual)
                if st.metrics is not None:
                    st.metrics.epipe_staged_expert_count += 1
            run_group(plan.first)                         # resident experts: recency updates only
            # the residual: the compute stream waits for its copy, then everything else runs
            if plan.residual_kind == "demand":
                torch.cuda.current_stream(w.device).wait_event(stage_event)
                # the transient payload lives in a staging slot outside the LRU
                run_group([plan.residual] + plan.rest, overrides={plan.residual: staged_slot})
                if st.cfg.epipe_demand_commit:
                    st.access_freq[plan.residual] = st.access_freq.get(plan.residual, 0) + 1
                st.staging.give(staged_slot)
            else:
                run_group([plan.residual] + plan.rest)    # a hit that waits for the prefetch event
        st.note_compute_done()

    def forward(self, x: torch.Tensor, stage: str = "") -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        st, w, k = self.store, self.store.w, self.top_k
        t = x.shape[0]
        stage = stage or SparseContext.stage(1 if t == 1 else t)
        idx, wts, logits, shared_scale = ops.router_topk(
            x, w.router_w, k, bias=w.router_bias, w_shared_gate=w.shared_gate_w, renorm=self.renorm,
            fp32_logits=self.fp32_logits)
        p = ops.permute(x, idx.reshape(-1), w.num_experts, k, item_scale=wts.reshape(-1))
        needed = self._needed_experts(p.expert_offsets)
        self.last_needed = needed
        plan = self._epipe_plan(needed, stage)
        self.last_plan = plan
        hbuf = torch.empty((p.r_cap, w.inter), dtype=torch.bfloat16, device=w.device)
        y = torch.empty((p.r_cap, w.hidden), dtype=torch.bfloat16, device=w.device)

        # Up to DECODE_MAX_TOKENS rows take the same weight-streaming kernels the
        # resident layer uses at that size, so both stay bit-identical; the
        # shared expert rides in the first of those launches.
        decode = t <= DECODE_MAX_TOKENS
        shared_h = shared_dec = None
        if decode and w.shared_inter:
            shared_h = torch.empty((t, w.shared_inter), dtype=torch.bfloat16, device=w.device)
            shared_dec = torch.empty((t, w.hidden), dtype=torch.bfloat16, device=w.device)
        shared_pending = [decode and bool(w.shared_inter)]

        def gemm():
            stream = torch.cuda.current_stream(w.device).cuda_stream
            if decode:
                with_shared = shared_pending[0]
                shared_pending[0] = False
                _lib.check(_lib.lib.sb_decode_experts(
                    x.data_ptr(), p.item_of_slot.data_ptr(), k, p.tile_table.data_ptr(),
                    w.slot_of_expert.data_ptr(), w.w13.data_ptr(), w.w2.data_ptr(), p.slot_scale.data_ptr(),
                    w.hidden, w.inter, w.n_slots, hbuf.data_ptr(), y.data_ptr(),
                    w.shared_w13.data_ptr() if with_shared else 0, w.shared_w2.data_ptr() if with_shared else 0,
                    shared_scale.data_ptr() if with_shared and shared_scale is not None else 0,
                    w.shared_inter if with_shared else 0, t,
                    shared_h.data_ptr() if with_shared else 0, shared_dec.data_ptr() if with_shared else 0,
                    self.status.data_ptr(), stream), "sb_decode_experts")
                return
            _lib.check(_lib.lib.sb_grouped_swiglu(
                p.rows.data_ptr(), p.tile_table.data_ptr(), 0, w.w13.data_ptr(), w.w2.data_ptr(),
                w.slot_of_expert.data_ptr(), p.slot_scale.data_ptr(), p.r_cap, w.hidden, w.inter, w.n_slots,
                hbuf.data_ptr(), y.data_ptr(), self.status.data_ptr(), stream), "sb_grouped_swiglu")

        self.run_routed(needed, gemm, plan)
        shared_out = None
        if decode and w.shared_inter:
            if shared_pending[0]:                         # no routed launch happened (cannot occur with top_k >= 1)
                gemm()
            shared_out = shared_dec
        elif w.shared_inter:
            shared_out, _ = ops.grouped_swiglu(x, w.shared_w13, w.shared_w2, dense_rows=t, row_scale=shared_scale,
                                               status=self.status)
        out = ops.combine(y, p.slot_of_item, idx, shared_out, t)
        return out, idx, wts, logits
