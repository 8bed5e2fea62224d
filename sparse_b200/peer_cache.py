"""Non-owned experts in local cache slots, filled from the owners' GPUs.

Under expert parallelism every expert has an owner rank whose slab holds its
weights.  With spare HBM a rank can also keep copies of experts it does not own
in a few cache slots and run its own tokens' rows for them locally instead of
sending the rows to the owner and waiting for the result ("run locally if the
weights are here, else at the owner": the reference's `_light_destinations`,
utils/eval_core.py:6396-6411, over its local-only materialisation
utils/eval_core.py:9970-9984).  The copies come from the owner GPU's slab over
NVLink (plain `cudaMemcpyAsync` between mapped allocations on a side stream,
one call per tensor) into preallocated slots; nothing is allocated per step.

    PeerSlab         a layer's weight slabs in memory every rank has mapped
    PeerExperts      expert -> (owner rank, slot at the owner) -> source pointers
    LocalCacheEpLayer  the decode-sized expert-parallel step with local execution
                     of cached non-owned experts, a reactive LRU and an optional
                     next-layer prefetch plan

Policies of a step (`LocalCacheEpLayer.miss` / `.late`):
    miss = "load"   a selected non-owned expert that is not cached is copied now,
                    on the compute stream (the reference's reactive demand load:
                    the copy time is exposed), then run locally
    miss = "owner"  its rows go to the owner this step (nothing is waited for)
    late = "wait"   a cached expert whose prefetch copy is still in flight makes
                    the compute stream wait for it (exposed)
    late = "owner"  its rows go to the owner this step (readiness scheduling)
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Sequence, Set, Tuple

import torch

from . import _lib
from ._lib import lib, check
from .cache import ExpertWeightCache
from .context import Metrics
from .ep import ExpertParallelLayer
from .layer import LayerWeights
from .rs import build_prefetch_plan
from .store import ExpertStore, HostExperts, SLOT_SKIP


class _RawCuda:
    """A device allocation presented through __cuda_array_interface__ (int16 view)."""

    def __init__(self, ptr: int, n_elems: int):
        self.__cuda_array_interface__ = {"shape": (n_elems,), "typestr": "<i2", "data": (ptr, False), "version": 3}


def _wrap(ptr: int, shape: Tuple[int, ...], device: torch.device) -> torch.Tensor:
    n = 1
    for d in shape:
        n *= d
    t = torch.as_tensor(_RawCuda(ptr, n), device=device)
    return t.view(torch.bfloat16).view(*shape)


class PeerSlab:
    """w13 [S,2I,H] and w2 [S,H,I] of one layer in exportable device memory, and
    the addresses of every peer's slabs as mapped on this GPU."""

    def __init__(self, hidden: int, inter: int, n_slots: int, ep: int, rank: int, device: torch.device):
        self.hidden, self.inter, self.n_slots, self.ep, self.rank, self.device = hidden, inter, n_slots, ep, rank, device
        self.bytes13 = n_slots * 2 * inter * hidden * 2
        self.bytes2 = n_slots * hidden * inter * 2
        self._owned: List[int] = []
        self._imported: List[int] = []
        with torch.cuda.device(device):
            p13, p2 = C.c_void_p(), C.c_void_p()
            check(lib.sb_peer_alloc(self.bytes13, C.byref(p13)), "sb_peer_alloc")
            check(lib.sb_peer_alloc(self.bytes2, C.byref(p2)), "sb_peer_alloc")
        self._owned = [int(p13.value), int(p2.value)]
        self.w13 = _wrap(int(p13.value), (n_slots, 2 * inter, hidden), device)
        self.w2 = _wrap(int(p2.value), (n_slots, hidden, inter), device)
        self.peer13: List[int] = [0] * ep
        self.peer2: List[int] = [0] * ep
        self.peer13[rank], self.peer2[rank] = int(p13.value), int(p2.value)

    def export_handles(self) -> bytes:
        out = b""
        for p in self._owned:
            buf = C.create_string_buffer(64)
            check(lib.sb_ipc_export(p, buf), "sb_ipc_export")
            out += buf.raw
        return out

    def import_handles(self, peer: int, blob: bytes) -> None:
        ptrs = []
        for i in range(2):
            p = C.c_void_p()
            h = C.create_string_buffer(blob[64 * i:64 * (i + 1)], 64)
            check(lib.sb_ipc_import(h, C.byref(p)), "sb_ipc_import")
            ptrs.append(int(p.value))
            self._imported.append(int(p.value))
        self.peer13[peer], self.peer2[peer] = ptrs

    def adopt_local_peer(self, peer: int, other: "PeerSlab") -> None:
        """Simulated ranks inside one process."""
        self.peer13[peer], self.peer2[peer] = other.peer13[other.rank], other.peer2[other.rank]

    def exchange(self, group) -> None:
        import torch.distributed as dist
        blobs: List[Optional[bytes]] = [None] * self.ep
        dist.all_gather_object(blobs, self.export_handles(), group=group)
        for peer, blob in enumerate(blobs):
            if peer != self.rank:
                self.import_handles(peer, blob)

    def close(self) -> None:
        for p in self._imported:
            lib.sb_ipc_close(p)
        for p in self._owned:
            lib.sb_peer_free(p)
        self._imported, self._owned = [], []


class PeerExperts:
    """Source of a non-owned expert's weights: rows of its owner's slab."""

    def __init__(self, slab: PeerSlab, owner_of: Sequence[int], slot_at_owner: Sequence[int]):
        self.slab = slab
        self.owner_of = [int(r) for r in owner_of]
        self.slot_at_owner = [int(s) for s in slot_at_owner]
        self.stride13 = 2 * slab.inter * slab.hidden * 2
        self.stride2 = slab.hidden * slab.inter * 2

    def __contains__(self, expert: int) -> bool:
        return 0 <= expert < len(self.owner_of) and self.owner_of[expert] != self.slab.rank

    def copy_into(self, weights: LayerWeights, slot: int, expert: int, stream: torch.cuda.Stream) -> int:
        """Two async copies (gate/up rows, down rows) from the owner GPU; returns the bytes."""
        r, s = self.owner_of[expert], self.slot_at_owner[expert]
        dev = weights.device.index
        check(lib.sb_slot_copy_async(weights.w13[slot].data_ptr(), self.slab.peer13[r] + s * self.stride13,
                                     self.stride13, _lib.SB_COPY_PEER_TO_DEVICE, dev, stream.cuda_stream),
              "sb_slot_copy_async(peer w13)")
        check(lib.sb_slot_copy_async(weights.w2[slot].data_ptr(), self.slab.peer2[r] + s * self.stride2,
                                     self.stride2, _lib.SB_COPY_PEER_TO_DEVICE, dev, stream.cuda_stream),
              "sb_slot_copy_async(peer w2)")
        return self.stride13 + self.stride2


def owned_slots(owner_of: Sequence[int], ep: int) -> Tuple[List[List[int]], List[int]]:
    """(experts owned by each rank in ascending id, slot of every expert at its owner)."""
    owned: List[List[int]] = [[] for _ in range(ep)]
    slot_at_owner = [0] * len(owner_of)
    for e, r in enumerate(owner_of):
        slot_at_owner[e] = len(owned[r])
        owned[r].append(e)
    return owned, slot_at_owner


def build_rank_layer(w, device: torch.device, rank: int, ep: int, owner_of: Sequence[int], cache_slots: int,
                     slab: Optional[PeerSlab] = None) -> Tuple[LayerWeights, PeerSlab, List[int], List[int]]:
    """Weights of one rank: owned experts in slots 0..n_owned-1 of a peer-mapped
    slab, `cache_slots` empty slots behind them.  `w` is a `synth.BlockWeights`.
    Returns (weights, slab, owned experts, slot of every expert at its owner)."""
    s = w.shape
    owned, slot_at_owner = owned_slots(owner_of, ep)
    mine = owned[rank]
    n_slots = max(1, max(len(o) for o in owned) + cache_slots)       # same slab size on every rank
    if slab is None:
        slab = PeerSlab(s.hidden, s.inter, n_slots, ep, rank, device)
    lw = LayerWeights(s.hidden, s.inter, s.num_experts, n_slots, s.shared_inter, device, w13=slab.w13, w2=slab.w2)
    lw.set_router(w.router, w.router_bias)
    slot_of = [-1] * s.num_experts
    for slot, e in enumerate(mine):
        lw.load_expert(slot, w.gate[e], w.up[e], w.down[e])
        slot_of[e] = slot
    lw.set_slot_map(slot_of)
    if s.shared_inter:
        lw.set_shared(w.sh_gate, w.sh_up, w.sh_down, w.sh_scalar_gate)
    return lw, slab, mine, slot_at_owner


class LocalCacheEpLayer(ExpertParallelLayer):
    """Expert-parallel layer whose decode-sized steps run cached non-owned experts locally.

    The slab holds this rank's owned experts (fixed slots) and `cache_slots` LRU
    slots for copies of other ranks' experts.  A decode-sized step reads back
    which experts this rank's tokens selected (one host synchronisation, as the
    reference's per-layer `.tolist()`), decides per expert where it runs, and
    tells the exchange kernel (`sb_ep_exchange_dispatch_local`) which experts
    stay here; their rows are computed by the weight-streaming kernels out of
    the cache slots and written where the combine expects them.  Larger batches
    take the owner-routed path of the base class."""

    def __init__(self, weights: LayerWeights, slab: PeerSlab, owned: Sequence[int], slot_at_owner: Sequence[int],
                 owner_of: Sequence[int], top_k: int, max_tokens: int, rank: int, ep: int, process_group,
                 cache_slots: int, miss: str = "load", late: str = "wait", metrics: Optional[Metrics] = None,
                 layer_idx: int = 0, renorm: bool = False, fp32_logits: bool = False):
        if miss not in ("load", "owner") or late not in ("wait", "owner"):
            raise ValueError("miss must be load or owner, late must be wait or owner")
        super().__init__(weights, top_k, max_tokens, rank, ep, process_group, owner=list(owner_of),
                         renorm=renorm, fp32_logits=fp32_logits)
        self.miss, self.late = miss, late
        self.metrics = metrics if metrics is not None else Metrics()
        self.owned_set: Set[int] = set(int(e) for e in owned)
        self.peers = PeerExperts(slab, owner_of, slot_at_owner)
        self.store = ExpertStore(weights, HostExperts(weights.hidden, weights.inter), cache_slots, staging_slots=0,
                                 resident=list(owned), metrics=self.metrics, layer_idx=layer_idx, peers=self.peers)
        dev, e = weights.device, weights.num_experts
        n = max(1, _lib.DECODE_MAX_TOKENS * top_k)
        i32 = torch.int32
        self.local_map = torch.full((e,), -1, dtype=i32, device=dev)           # exchange: >= 0 stays here
        self.local_slots = torch.full((e,), SLOT_SKIP, dtype=i32, device=dev)  # local GEMM: slot or skip
        self.local_dst = torch.zeros((n,), dtype=torch.int64, device=dev)
        self.local_hbuf = torch.empty((n, weights.inter), dtype=torch.bfloat16, device=dev)
        self._maps_host = [torch.empty((2, e), dtype=i32).pin_memory() for _ in range(8)]
        self._maps_events: List[Optional[torch.cuda.Event]] = [None] * len(self._maps_host)
        self._maps_pos = 0
        self._idx_host = torch.empty((_lib.DECODE_MAX_TOKENS, top_k), dtype=i32).pin_memory()
        self.last_local: List[int] = []
        self.last_to_owner: List[int] = []

    # -- prefetch --------------------------------------------------------------------------
    def prefetch(self, scores: Dict[int, float], budget: int, min_score: float = 0.0) -> int:
        """Start copies (owner GPU -> cache slot, side stream) for the best-scored
        non-owned experts that are not cached yet; returns how many were admitted.
        Call it while an earlier layer computes; `begin_step` ends the cycle."""
        st = self.store
        want = {int(e): float(s) for e, s in scores.items() if int(e) not in self.owned_set}
        plan = build_prefetch_plan(want, st.cache, protect_ids=st.protect_ids(), budget=budget,
                                   min_score=min_score, replace_advantage=0.0, replace_margin=1.0,
                                   allow_active_replace=True, is_local=lambda e: True, keep_bias=st.keep_bias)
        return st.admit_prefetch_plan(plan)

    def begin_step(self) -> None:
        """A new decode step begins: prefetch pins of the previous one are dropped."""
        self.store.end_prefetch_group()

    # -- one step --------------------------------------------------------------------------
    def _push_maps(self, local: Dict[int, int]) -> None:
        i = self._maps_pos
        self._maps_pos = (i + 1) % len(self._maps_host)
        if self._maps_events[i] is not None:
            self._maps_events[i].synchronize()
        row = self._maps_host[i]
        row[0].fill_(-1)
        row[1].fill_(SLOT_SKIP)
        for e, slot in local.items():
            row[0, e] = slot
            row[1, e] = slot
        self.local_map.copy_(row[0], non_blocking=True)
        self.local_slots.copy_(row[1], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.r.device))
        self._maps_events[i] = ev

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, stage: Optional[str] = None) -> torch.Tensor:
        r, st, m = self.r, self.store, self.metrics
        t = x.shape[0]
        if t > _lib.DECODE_MAX_TOKENS or t == 0 or not r.scatter_return:
            return super().forward(x, out, stage)
        if stage is not None and stage != r.stage:
            r.use_stage(stage)
        r.launches = 0
        stream = torch.cuda.current_stream(r.device)
        with torch.cuda.device(r.device):
            r.stage_route(x)
            self._idx_host[:t].copy_(r.topk_idx[:t], non_blocking=True)
            stream.synchronize()                                    # the one host synchronisation
            chosen = self._idx_host[:t].reshape(-1).tolist()
            counts: Dict[int, int] = {}
            for e in chosen:
                if 0 <= e < r.w.num_experts and e not in self.owned_set:
                    counts[e] = counts.get(e, 0) + 1
            selected = set(counts)
            local: Dict[int, int] = {}
            to_owner: List[int] = []
            t0 = None
            for e in sorted(counts):
                cached = st.cache.has(e)
                if cached and st.copy_pending(e) and self.late == "owner":
                    to_owner.append(e)                               # not ready: the owner runs it this step
                    continue
                if not cached and self.miss == "owner":
                    to_owner.append(e)
                    m.cache_miss_count += 1
                    continue
                if not cached and len(st.pool) == 0 and not st.cache.evictable_prefetch_ids(selected):
                    to_owner.append(e)                               # every slot holds an expert of this step
                    m.cache_miss_count += 1
                    continue
                if t0 is None and (not cached or st.copy_pending(e)):
                    t0 = torch.cuda.Event(enable_timing=True)        # from here the stream may wait for copies
                    t0.record(stream)
                slot = st.demand(e, protect=selected)
                if slot is None:
                    to_owner.append(e)                               # no evictable slot: fall back to the owner
                    continue
                local[e] = int(slot)
            if t0 is not None:
                t1 = torch.cuda.Event(enable_timing=True)
                t1.record(stream)
                m.pending_events.append(("load_exposed", "decode", t0, t1))
            m.local_cached_item_count += sum(counts[e] for e in local)
            m.owner_fallback_item_count += sum(counts[e] for e in to_owner)
            self.last_local, self.last_to_owner = sorted(local), to_owner
            self._push_maps(local)
            b, w, k = r.bufs, r.w, r.top_k
            check(lib.sb_ep_exchange_dispatch_local(
                r.local_offsets.data_ptr(), b.ptr_array("ctl"), b.ptr_array("ctl", b.flags_offset),
                b.local["ctl"] + b.epoch_offset, r.owner.data_ptr(), w.num_experts, r.rank, r.ep,
                b.recv_cap, r.dst_base.data_ptr(), r.recv_offsets.data_ptr(), r.recv_tiles.data_ptr(),
                x.data_ptr(), r.topk_idx.data_ptr(), r.topk_w.data_ptr(), r.slot_of_item.data_ptr(),
                t * k, k, w.hidden, b.ptr_array("rows"), b.ptr_array("scale"), r.item_rank.data_ptr(),
                r.item_row.data_ptr(), b.ptr_array("meta"), b.ptr_array("ret"), b.ret_rows,
                r.row_dst.data_ptr(), self.local_map.data_ptr(), r.item_of_slot.data_ptr(),
                self.local_dst.data_ptr(), r.status.data_ptr(), stream.cuda_stream),
                "sb_ep_exchange_dispatch_local")
            r.launches += 1
            r._scattered = True
            if local:
                check(lib.sb_decode_experts_to(
                    x.data_ptr(), r.item_of_slot.data_ptr(), k, r.local_tiles.data_ptr(),
                    self.local_slots.data_ptr(), w.w13.data_ptr(), w.w2.data_ptr(), r.local_scale.data_ptr(),
                    w.hidden, w.inter, w.n_slots, self.local_hbuf.data_ptr(), self.local_dst.data_ptr(), t,
                    r.status.data_ptr(), stream.cuda_stream), "sb_decode_experts_to")
                r.launches += 2
            r.stage_experts_and_shared()
            self._barrier()
            res = r.stage_combine(out)
            st.note_compute_done()
        m.finalize_events()
        self.last_launches = r.launches
        return res
