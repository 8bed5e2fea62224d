"""Bounded next-layer staging: prediction and copies off the critical path.

Counterpart of the reference's opt-in `BoundedRS` adapter
(utils/rs_overlap.py:58-497).  Rules kept from there:
  * a fixed pool of staging slots (>= 2, default 4), reserved up front; a target
    layer may use at most min(top_m, slots // 2) of them;
  * the predictor of layer L+1 runs as a CUDA graph on a side stream during
    layer L (decode only), its top-k goes to pinned host buffers asynchronously;
  * ONE worker thread waits for that read-back, picks candidates from a
    snapshot of the target's resident set (`select_candidates`) and enqueues
    host->slot copies on a copy stream through `StagingJob.publish`;
  * when layer L+1 reaches its demand path it closes the job (no later
    publication), sees the issued transfers through a `DemandView`, and waits
    for a transfer only where it actually uses it, on that transfer's event;
  * speculation never touches the LRU: after the layer's kernels are enqueued,
    transfers that were USED are committed into the LRU by exchanging slot
    ownership (the evicted resident's slot becomes the next staging slot, no
    bytes move); unused ones are counted as wasted and their slots recycled
    once their copy event has completed;
  * a slot is reused only after the event recorded behind its last consumer.
Staging slots are slab slots here, so a "payload" is a slot index.
"""
from __future__ import annotations

import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Optional, Tuple

import torch

from . import _lib, ops
from .context import SparseContext
from .staging import DemandView, StagingJob, Transfer, select_candidates


class GraphPredictor:
    """Predictor MLP + top-k captured as a CUDA graph for a fixed input shape."""

    def __init__(self, model, batch: int, width: int, k: int, device: torch.device):
        self.model, self.k = model, k
        self.input = torch.zeros((batch, width), device=device, dtype=torch.float32)
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side), torch.inference_mode():
            for _ in range(3):
                self._compute(self.input)
        side.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=side), torch.inference_mode():
            self.ids, self.values = self._compute(self.input)
        torch.cuda.current_stream(device).wait_stream(side)

    def _compute(self, x):
        values, ids = torch.topk(self.model(x).float(), k=self.k, dim=-1)
        return ids.to(torch.int64), values

    def __call__(self, x):
        self.input.copy_(x)
        self.graph.replay()
        return self.ids, self.values


class _Slot:
    __slots__ = ("index", "busy", "retire", "event")

    def __init__(self, index: int, device):
        self.index, self.busy, self.retire = index, False, None
        self.event = torch.cuda.Event()


class BoundedStager:
    """Drives speculative staging for a stack of cached-mode MoE blocks."""

    def __init__(self, blocks: Dict[int, object], slots: int = 4):
        if slots < 2:
            raise ValueError("the staging pool needs at least 2 slots")
        self.blocks = blocks
        self.slot_count = slots
        self.pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="rs-staging")
        self.owner = threading.get_ident()
        self.jobs: Dict[int, StagingJob] = {}
        self.retired: List[Tuple[StagingJob, Dict[int, Transfer]]] = []
        self.views: Dict[int, DemandView] = {}
        self.slots: Dict[int, List[_Slot]] = {}       # per layer: slab slots reserved for staging
        self.graphs: Dict[Tuple[int, int], GraphPredictor] = {}
        self.buffers: Dict[Tuple[int, int], tuple] = {}
        self.stream: Optional[torch.cuda.Stream] = None
        self.copy_stream: Optional[torch.cuda.Stream] = None
        self.epoch = 0
        self.enabled = False
        self.stats = dict(predictions=0, issued=0, used=0, wasted=0, retained=0, recycled=0,
                          skipped_slots=0, closed_before_publish=0, worker_ms=0.0, readback_wait_ms=0.0)

    # -- set-up (between requests) -----------------------------------------------------
    def install(self, batch: int) -> None:
        """Reserve staging slots in every cached block's slab and capture the predictors."""
        any_block = next(iter(self.blocks.values()))
        dev = any_block.device
        self.stream = torch.cuda.Stream(device=dev)
        self.copy_stream = torch.cuda.Stream(device=dev)
        for layer, blk in self.blocks.items():
            store = blk.store
            if store is None:
                continue
            taken = []
            while len(taken) < self.slot_count:
                s = store.staging.take()
                if s is None:
                    break
                taken.append(_Slot(s, dev))
            if len(taken) < 2:
                raise RuntimeError("layer %d: slab has %d staging slots, the bounded stager needs >= 2" % (
                    layer, len(taken)))
            self.slots[layer] = taken
            self.views[layer] = DemandView(store.cache)
            store.view = self.views[layer]
        bank = SparseContext.rs_bank
        for layer, blk in self.blocks.items():
            target = layer + 1
            if bank is None or target not in self.blocks or self.blocks[target].store is None:
                continue
            k = min(blk.num_experts, self.blocks[target]._rs_prefetch_predict_topk())
            self.graphs[layer, k] = GraphPredictor(bank[target], batch, blk.hidden_size, k, dev)
            self.buffers[layer, k] = (torch.empty((batch, k), dtype=torch.int64).pin_memory(),
                                      torch.empty((batch, k), dtype=torch.float32).pin_memory(),
                                      torch.cuda.Event())
        self.enabled = True

    # -- slot bookkeeping ----------------------------------------------------------------
    def _collect(self) -> None:
        keep = []
        for job, transferred in self.retired:
            if not job.future.done():
                keep.append((job, transferred))
                continue
            row = job.future.result()
            self.stats["worker_ms"] += row["worker_ms"]
            self.stats["readback_wait_ms"] += row["readback_wait_ms"]
            used = {id(t.slot) for t in transferred.values()}
            for slot in job.slots:
                if id(slot) not in used:
                    slot.busy, slot.retire = False, None
        self.retired = keep

    def _reserve(self, layer: int, budget: int) -> List[_Slot]:
        self._collect()
        free = [s for s in self.slots[layer] if not s.busy and (s.retire is None or s.retire.query())]
        got = free[:budget]
        for s in got:
            s.busy, s.retire = True, None
        return got

    # -- worker thread --------------------------------------------------------------------
    def _work(self, job: StagingJob, target, ids, weights, readback, resident, minimum, allowed):
        t0 = time.perf_counter()
        store = target.store
        with torch.cuda.device(target.device):
            w0 = time.perf_counter()
            readback.synchronize()
            waited = (time.perf_counter() - w0) * 1e3
            if not job.closed:
                chosen = select_candidates(ids.reshape(-1).tolist(), weights.reshape(-1).tolist(),
                                           allowed=allowed, resident=resident, minimum=minimum,
                                           budget=len(job.slots))
                job.plan_count = len(chosen)
                for expert, slot in zip(chosen, job.slots):
                    def submit(expert=expert, slot=slot):
                        ops.slot_copy_async(store.w.w13[slot.index], store.host.w13[expert], self.copy_stream,
                                            _lib.SB_COPY_HOST_TO_DEVICE)
                        ops.slot_copy_async(store.w.w2[slot.index], store.host.w2[expert], self.copy_stream,
                                            _lib.SB_COPY_HOST_TO_DEVICE)
                        slot.event.record(self.copy_stream)
                        return Transfer(expert, slot.index, slot.event, slot, store.host.nbytes(expert))
                    if not job.publish(expert, submit):
                        break
        return dict(worker_ms=(time.perf_counter() - t0) * 1e3, readback_wait_ms=waited)

    # -- hooks called by the serving loop ----------------------------------------------------
    def predict(self, layer: int, x: torch.Tensor) -> None:
        """During layer `layer` (decode, one token per sequence): start the
        prediction for layer+1 and hand the planning to the worker."""
        if not self.enabled or threading.get_ident() != self.owner:
            raise RuntimeError("BoundedStager.predict must be called by the thread that built it, after install()")
        target_layer = layer + 1
        target = self.blocks.get(target_layer)
        if target is None or target.store is None:
            return
        self._collect()
        if target_layer in self.jobs or any(j.ticket[2] == target_layer for j, _ in self.retired):
            self.stats["skipped_slots"] += 1
            return
        budget = min(int(target._effective_rs_prefetch_top_m()), self.slot_count // 2)
        if budget <= 0:
            return
        slots = self._reserve(target_layer, budget)
        if not slots:
            self.stats["skipped_slots"] += 1
            return
        blk = self.blocks[layer]
        k = min(blk.num_experts, target._rs_prefetch_predict_topk())
        graph = self.graphs[layer, k]
        host_ids, host_w, event = self.buffers[layer, k]
        cur = torch.cuda.current_stream(blk.device)
        self.stream.wait_stream(cur)
        x.record_stream(self.stream)
        with torch.cuda.stream(self.stream), torch.inference_mode():
            ids, w = graph(x)
            host_ids.copy_(ids, non_blocking=True)
            host_w.copy_(w, non_blocking=True)
            event.record(self.stream)
        # the copy stream must not overwrite a staging slot a GEMM may still read
        target.store._side_stream_may_overwrite(self.copy_stream)
        job = StagingJob((self.epoch, int(SparseContext.runtime_call_id), target_layer), slots)
        self.jobs[target_layer] = job
        resident = frozenset(self.views[target_layer].resident_ids())
        lo, _, _ = target.cfg.effective_planner_thresholds()
        job.future = self.pool.submit(self._work, job, target, host_ids, host_w, event, resident, float(lo),
                                      frozenset(target._local_eid_set))
        self.stats["predictions"] += 1

    def activate(self, layer: int) -> DemandView:
        """At layer `layer`'s demand time: close publication and expose what was issued."""
        view = self.views[layer]
        job = self.jobs.pop(layer, None)
        if job is None:
            return view
        transfers = job.close()
        if job.ticket[:2] != (self.epoch, int(SparseContext.runtime_call_id)):
            raise AssertionError("stale prediction crossed a request/step boundary")
        self.retired.append((job, transfers))
        if not transfers:
            self.stats["closed_before_publish"] += 1
        view.staged = transfers
        store = self.blocks[layer].store
        for expert, tr in transfers.items():
            store.events[expert] = tr.event
            store.prefetched_this_group.add(expert)
            if store.metrics is not None:
                store.metrics.expert_weight_h2d_bytes += tr.nbytes
                store.metrics.expert_weight_h2d_prefetch_bytes += tr.nbytes
                store.metrics.prefetch_issued_count += 1
                store.metrics.prefetch_admitted_count += 1
            self.stats["issued"] += 1
        return view

    def release(self, layer: int) -> None:
        """After layer `layer`'s kernels are enqueued: commit used transfers into the
        LRU by swapping slot ownership, recycle the rest."""
        view = self.views[layer]
        store = self.blocks[layer].store
        used = [t for t in view.staged.values() if t.used]
        done = None
        if used:
            done = torch.cuda.Event()
            done.record(torch.cuda.current_stream(store.device))
        for tr in view.used_in_order:
            cache = view.resident
            evicted = cache.put(tr.expert, tr.payload)
            if cache.has(tr.expert):
                if evicted is not None:
                    tr.slot.index = int(cache.last_evicted_payload)   # victim's slot becomes the scratch slot
                    store.events.pop(evicted, None)
                    self.stats["recycled"] += 1
                else:
                    free = store.pool.take()
                    if free is None:
                        raise RuntimeError("LRU accepted an entry without evicting but the slot pool is empty")
                    tr.slot.index = free
                tr.retained = True
                self.stats["retained"] += 1
        for expert, tr in view.staged.items():
            tr.slot.busy = False
            tr.slot.retire = done if tr.used else tr.event
            self.stats["used" if tr.used else "wasted"] += 1
            if not tr.used and store.metrics is not None:
                store.metrics.prefetch_wasted_count += 1
            store.events.pop(expert, None)
            store.prefetched_this_group.discard(expert)
            store.used_this_group.discard(expert)
        view.staged = {}
        view.used_in_order = []

    def finish(self) -> dict:
        """Drain at the end of a request: close open jobs, wait for the worker, sync the side streams."""
        for layer, job in list(self.jobs.items()):
            transfers = job.close()
            self.retired.append((job, transfers))
            for tr in transfers.values():
                tr.slot.busy, tr.slot.retire = False, tr.event
        self.jobs.clear()
        for job, _ in self.retired:
            job.future.result(timeout=30)
        self._collect()
        if self.stream is not None:
            self.stream.synchronize()
            self.copy_stream.synchronize()
        for layer, view in self.views.items():
            if view.staged:
                self.release(layer)
        self.epoch += 1
        return dict(self.stats)

    def close(self) -> None:
        self.finish()
        self.pool.shutdown(wait=True)
        for layer, slots in self.slots.items():
            store = self.blocks[layer].store
            for s in slots:
                store.staging.give(s.index)
            store.view = None
        self.slots, self.enabled = {}, False
