"""Expert-parallel layer pass: tokens sharded by rank, experts sharded by owner,
rows moved by this library's own kernels over NVLink peer memory.

One process per GPU.  Each rank allocates six exportable buffers (receive rows,
receive route weights, return addresses of the received rows, expert outputs,
the return buffer its own results come back into, counts + flags), exchanges
their CUDA IPC handles once through `torch.distributed` (the only use of the
process group on this path), and from then on a layer pass is a fixed sequence
of kernel launches with no host synchronisation:

    router -> local sort -> publish counts -> barrier -> plan -> dispatch (rows,
    weights, return addresses) -> barrier -> resolve return addresses
           -> grouped SwiGLU on the received rows, result rows stored straight
              into the senders' return buffers -> barrier -> local combine

The shared expert runs on the caller's stream beside the exchange (side stream);
decode-sized steps use a shorter single-stream sequence with fused launches.
The buffers are reused by every layer; the barriers order the reuse (a rank
cannot start writing into a peer's buffer for the next pass before that peer
has passed the previous pass's last barrier).

`EpRank.stage_*` are the individual steps; `ExpertParallelLayer.forward` strings
them together with barriers.  The stages can also be driven for several
simulated ranks inside one process (all "peer" buffers on one GPU, no barrier
kernels, the caller steps the ranks in lockstep), which is how the index
arithmetic is tested on a single GPU.
"""
from __future__ import annotations

import os

import ctypes as C
from typing import List, Optional, Sequence

import torch

from . import _lib
from ._lib import lib, check
from .layer import LayerWeights

_TILE = _lib.SB_TILE_M


def _round_up(v: int, a: int) -> int:
    return (v + a - 1) // a * a


def recv_capacity(max_tokens: int, top_k: int, ep: int) -> int:
    """Rows a rank must be able to receive: every item of every rank."""
    return _round_up(max(1, max_tokens * top_k * ep), _TILE)


def owner_table(owner, ep: int, num_experts: int) -> torch.Tensor:
    """Destination table int32 [ep][E] from either one ownership row [E] or a
    per-source table [ep][E] (e.g. `Placement.dest_table`)."""
    t = torch.as_tensor(owner, dtype=torch.int32)
    if t.dim() == 1:
        t = t.unsqueeze(0).expand(ep, -1)
    if tuple(t.shape) != (ep, num_experts):
        raise ValueError("owner table must be [E] or [ep,E] = [%d,%d], got %s" % (ep, num_experts, tuple(t.shape)))
    if int(t.min()) < 0 or int(t.max()) >= ep:
        raise ValueError("owner table holds a rank outside [0,%d)" % ep)
    return t.contiguous()


def plan_layout_reference(counts_all: torch.Tensor, owner: torch.Tensor, rank: int):
    """Host mirror of `sb_ep_plan` (integer arithmetic on CPU tensors), used by the
    debug checks and the CPU tests.  counts_all int [ep,E]; owner int [E] or
    [ep,E] (owner[s][e] = destination of expert e for source s).
    Returns (dst_base [E], recv_offsets [E+1], seg_begin [ep,E]): rows of expert e
    coming from source s sit, in rank d = owner[s][e]'s receive buffer, at
    seg_begin[d][e] + (rows of e from sources s' < s that also go to d); a buffer
    is ordered by expert id, then source rank, then the source's stable item order."""
    counts_all = counts_all.to(torch.long)
    ep, e = counts_all.shape
    own = owner_table(owner, ep, e).to(torch.long)
    tot = torch.zeros((ep, e), dtype=torch.long)
    for s in range(ep):
        tot[own[s], torch.arange(e)] += counts_all[s]
    seg_begin = torch.cumsum(tot, 1) - tot
    dst = own[rank]
    before = torch.zeros(e, dtype=torch.long)
    for s in range(rank):
        before += torch.where(own[s] == dst, counts_all[s], torch.zeros_like(counts_all[s]))
    dst_base = seg_begin[dst, torch.arange(e)] + before
    recv_offsets = torch.zeros(e + 1, dtype=torch.long)
    recv_offsets[:e] = seg_begin[rank]
    recv_offsets[e] = int(tot[rank].sum())
    return dst_base, recv_offsets, seg_begin


class PeerBuffers:
    """This rank's exportable buffers and the pointers of every rank's copies."""

    NAMES = ("rows", "scale", "y", "ctl", "meta", "ret")

    def __init__(self, hidden: int, num_experts: int, recv_cap: int, ep: int, rank: int, ret_rows: int = 0):
        self.hidden, self.num_experts, self.recv_cap, self.ep, self.rank = hidden, num_experts, recv_cap, ep, rank
        # rows of the return buffer: this rank's own items (tokens * top_k)
        self.ret_rows = ret_rows if ret_rows > 0 else max(1, recv_cap // ep)
        self.sizes = {
            "rows": recv_cap * hidden * 2,
            "scale": _round_up(recv_cap * 2, 256),
            "y": recv_cap * hidden * 2,
            # return address of every received row, and the buffer the owners write results back into
            "meta": _round_up(recv_cap * 4, 256),
            "ret": self.ret_rows * hidden * 2,
            # counts matrix int32 [ep][E] followed (at a 256-byte boundary) by the barrier flags uint32 [ep]
            "ctl": _round_up(ep * num_experts * 4, 256) + 256,
        }
        self.flags_offset = _round_up(ep * num_experts * 4, 256)
        # this rank's barrier epoch counter (uint32, touched by no peer) sits behind the flags
        self.epoch_offset = self.flags_offset + 128
        self.local = {}
        self.peers = {n: [0] * ep for n in self.NAMES}
        self._owned: List[int] = []
        self._imported: List[int] = []

    def allocate_local(self) -> None:
        for n in self.NAMES:
            p = C.c_void_p()
            check(lib.sb_peer_alloc(self.sizes[n], C.byref(p)), "sb_peer_alloc")
            self.local[n] = int(p.value)
            self._owned.append(int(p.value))
            self.peers[n][self.rank] = int(p.value)

    def export_handles(self) -> bytes:
        out = b""
        for n in self.NAMES:
            buf = C.create_string_buffer(64)
            check(lib.sb_ipc_export(self.local[n], buf), "sb_ipc_export")
            out += buf.raw
        return out

    def import_handles(self, peer: int, blob: bytes) -> None:
        for i, n in enumerate(self.NAMES):
            p = C.c_void_p()
            h = C.create_string_buffer(blob[64 * i:64 * (i + 1)], 64)
            check(lib.sb_ipc_import(h, C.byref(p)), "sb_ipc_import")
            self.peers[n][peer] = int(p.value)
            self._imported.append(int(p.value))

    def adopt_local_peer(self, peer: int, other: "PeerBuffers") -> None:
        """Simulated ranks inside one process: the peer's buffers are ordinary local pointers."""
        for n in self.NAMES:
            self.peers[n][peer] = other.local[n]

    def ptr_array(self, name: str, offset: int = 0):
        arr = (C.c_void_p * self.ep)()
        for i, p in enumerate(self.peers[name]):
            arr[i] = p + offset
        return arr

    def close(self) -> None:
        for p in self._imported:
            lib.sb_ipc_close(p)
        for p in self._owned:
            lib.sb_peer_free(p)
        self._imported, self._owned = [], []


def exchange_handles(bufs: PeerBuffers, group) -> None:
    """All ranks swap IPC handles through the process group (set-up time only)."""
    import torch.distributed as dist
    blobs: List[Optional[bytes]] = [None] * bufs.ep
    dist.all_gather_object(blobs, bufs.export_handles(), group=group)
    for peer, blob in enumerate(blobs):
        if peer != bufs.rank:
            bufs.import_handles(peer, blob)


class EpRank:
    """State and stages of one rank's layer pass."""

    def __init__(self, weights: LayerWeights, top_k: int, max_tokens: int, rank: int, ep: int,
                 owner: Sequence[int], bufs: PeerBuffers, renorm: bool = False,
                 fp32_logits: bool = False, owner_decode: Optional[Sequence[int]] = None):
        self.w, self.top_k, self.rank, self.ep = weights, top_k, rank, ep
        self.renorm, self.fp32_logits = renorm, fp32_logits
        self.bufs = bufs
        dev = weights.device
        self.device = dev
        e, h = weights.num_experts, weights.hidden
        self.max_tokens = max_tokens
        n = max_tokens * top_k
        i32, bf = torch.int32, torch.bfloat16
        # Destination tables [ep][E], one per stage: the reference picks the table
        # of the current stage on every forward (utils/eval_core.py:6736-6769) and
        # its launchers keep decode on round-robin while prefill follows the
        # placement (SPARSE_SCP_APPLY_DECODE=0).  `use_stage` switches between them.
        pre = owner_table(owner, ep, e).to(dev)
        dec = pre if owner_decode is None else owner_table(owner_decode, ep, e).to(dev)
        self._owners = {"prefill": (pre, pre[rank].contiguous()), "decode": (dec, dec[rank].contiguous())}
        self.stage = "prefill"
        self.owner, self.owner_row = self._owners["prefill"]        # [ep][E]; this rank's destinations
        self.topk_idx = torch.empty((max_tokens, top_k), dtype=i32, device=dev)
        self.topk_w = torch.empty((max_tokens, top_k), dtype=bf, device=dev)
        self.logits = torch.empty((max_tokens, e), dtype=torch.float32 if fp32_logits else bf, device=dev)
        self.shared_scale = torch.empty((_round_up(max_tokens, _TILE),), dtype=bf, device=dev)
        self.local_offsets = torch.empty((e + 1,), dtype=i32, device=dev)
        self.slot_of_item = torch.empty((max(n, 1),), dtype=i32, device=dev)
        self.item_of_slot = torch.empty((max(n, 1),), dtype=i32, device=dev)
        self.local_tiles = torch.empty((lib.sb_tile_table_ints(n, e),), dtype=i32, device=dev)
        self.sort_ws = torch.empty((lib.sb_permute_workspace_bytes(n, e),), dtype=torch.uint8, device=dev)
        self.dst_base = torch.empty((e,), dtype=i32, device=dev)
        self.recv_offsets = torch.empty((e + 1,), dtype=i32, device=dev)
        self.recv_tiles = torch.empty((lib.sb_tile_table_ints(bufs.recv_cap, e),), dtype=i32, device=dev)
        self.item_rank = torch.empty((max(n, 1),), dtype=i32, device=dev)
        self.item_row = torch.empty((max(n, 1),), dtype=i32, device=dev)
        self.hbuf = torch.empty((bufs.recv_cap, weights.inter), dtype=bf, device=dev)
        t_cap = _round_up(max_tokens, _TILE)
        self.shared_h = self.shared_out = None
        if weights.shared_inter:
            self.shared_h = torch.empty((t_cap, weights.shared_inter), dtype=bf, device=dev)
            self.shared_out = torch.empty((t_cap, h), dtype=bf, device=dev)
        self.out = torch.empty((max_tokens, h), dtype=bf, device=dev)
        self.status = torch.zeros((1,), dtype=i32, device=dev)
        self.launches = 0
        self._x = None
        self._t = 0
        self._scattered = False
        # Batches of at most DECODE_MAX_TOKENS rows take the decode-sized kernels
        # (per-row router, single-CTA sort, weight-streaming expert kernels).
        self.small_batch_kernels = True
        # Owners write result rows straight into the senders' return buffers from
        # the down GEMM's epilogue (needs the CTA-pair kernel); otherwise senders
        # read the owners' output buffers after the GEMM.
        self.scatter_return = bool(lib.sb_w13_interleaved())
        self.row_dst = torch.zeros((bufs.recv_cap,), dtype=torch.int64, device=dev)
        self.route_ws = torch.empty((_lib.DECODE_MAX_TOKENS * e,), dtype=torch.float32, device=dev)
        self.local_scale = torch.empty((max(_lib.DECODE_MAX_TOKENS * top_k, 1),), dtype=bf, device=dev)

    def use_stage(self, stage: str) -> None:
        """Route this and the following passes by the destination table of `stage`
        ("prefill" or "decode"); every rank must switch at the same pass."""
        if stage not in self._owners:
            raise ValueError("stage must be prefill or decode, got %r" % (stage,))
        self.stage = stage
        self.owner, self.owner_row = self._owners[stage]

    def _s(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _small(self) -> bool:
        return self.small_batch_kernels and 0 < self._t <= _lib.DECODE_MAX_TOKENS

    # -- stages -------------------------------------------------------------------
    def begin(self, x: torch.Tensor) -> None:
        """Names the batch of this pass (every stage below works on it)."""
        if x.shape[0] > self.max_tokens:
            raise RuntimeError("EP layer was sized for %d tokens, got %d" % (self.max_tokens, x.shape[0]))
        self._x, self._t = x, x.shape[0]

    def stage_route(self, x: Optional[torch.Tensor] = None, part: str = "both") -> None:
        """Router and local expert sort; above the decode size `part` = "router" /
        "sort" runs only that launch group (the sort is one CTA and can sit beside
        a GEMM, the router wants the machine)."""
        if x is not None:
            self.begin(x)
        w, x, t, k = self.w, self._x, self._t, self.top_k
        if self._small():
            check(lib.sb_route_decode(
                x.data_ptr(), w.router_w.data_ptr(),
                w.router_bias.data_ptr() if w.router_bias is not None else None,
                w.shared_gate_w.data_ptr() if w.shared_gate_w is not None else None,
                t, w.hidden, w.num_experts, k, int(self.renorm), int(self.fp32_logits),
                self.route_ws.data_ptr(), self.topk_idx.data_ptr(), self.topk_w.data_ptr(),
                self.logits.data_ptr(),
                self.shared_scale.data_ptr() if w.shared_gate_w is not None else None,
                self.local_offsets.data_ptr(), self.slot_of_item.data_ptr(), self.item_of_slot.data_ptr(),
                self.local_scale.data_ptr(), self.local_tiles.data_ptr(), self._s()), "sb_route_decode")
            self.launches += 2
            return
        if part in ("both", "router"):
            check(lib.sb_router_topk(
                x.data_ptr(), w.router_w.data_ptr(),
                w.router_bias.data_ptr() if w.router_bias is not None else None,
                w.shared_gate_w.data_ptr() if w.shared_gate_w is not None else None,
                t, w.hidden, w.num_experts, k, int(self.renorm), _lib.SB_DTYPE_BF16, int(self.fp32_logits),
                self.topk_idx.data_ptr(), self.topk_w.data_ptr(), self.logits.data_ptr(),
                self.shared_scale.data_ptr() if w.shared_gate_w is not None else None, self._s()),
                "sb_router_topk")
            self.launches += 1
        if part in ("both", "sort"):
            check(lib.sb_permute(
                None, self.topk_idx.data_ptr(), None, t * k, k, w.hidden, w.num_experts,
                self.sort_ws.data_ptr(), self.sort_ws.numel(), None, self.local_offsets.data_ptr(),
                self.slot_of_item.data_ptr(), self.item_of_slot.data_ptr(), None,
                self.local_tiles.data_ptr(), self._s()), "sb_permute")
            self.launches += 3

    def stage_publish(self) -> None:
        check(lib.sb_ep_publish_counts(self.local_offsets.data_ptr(), self.w.num_experts, self.rank,
                                       self.ep, self.bufs.ptr_array("ctl"), self._s()),
              "sb_ep_publish_counts")
        self.launches += 1

    # Wait limit of the cross-rank barriers in nanoseconds (None = the library's 2 s).
    barrier_limit_ns: Optional[int] = None

    def stage_barrier(self) -> None:
        b = self.bufs
        if self.barrier_limit_ns is None:
            check(lib.sb_ep_barrier_seq(b.ptr_array("ctl", b.flags_offset), self.rank, self.ep,
                                        b.local["ctl"] + b.epoch_offset, self.status.data_ptr(), self._s()),
                  "sb_ep_barrier_seq")
        else:
            check(lib.sb_ep_barrier_timed(b.ptr_array("ctl", b.flags_offset), self.rank, self.ep,
                                          b.local["ctl"] + b.epoch_offset, int(self.barrier_limit_ns),
                                          self.status.data_ptr(), self._s()), "sb_ep_barrier_timed")
        self.launches += 1

    def check_status(self) -> None:
        """Host-synchronising read of the device status word; raises on a non-zero value."""
        s = int(self.status.item())
        if s != 0:
            self.status.zero_()
            raise RuntimeError("sparse_b200 EP device status %d (1: GEMM wait expired, 2: expert "
                               "without a weight slot, 3: peer barrier wait expired)" % s)

    def stage_exchange_dispatch(self) -> None:
        """publish + barrier + plan + dispatch + barrier as one launch (decode-sized steps)."""
        b, w, t, k = self.bufs, self.w, self._t, self.top_k
        check(lib.sb_ep_exchange_dispatch(
            self.local_offsets.data_ptr(), b.ptr_array("ctl"), b.ptr_array("ctl", b.flags_offset),
            b.local["ctl"] + b.epoch_offset, self.owner.data_ptr(), w.num_experts, self.rank, self.ep,
            b.recv_cap, self.dst_base.data_ptr(), self.recv_offsets.data_ptr(), self.recv_tiles.data_ptr(),
            self._x.data_ptr(), self.topk_idx.data_ptr(), self.topk_w.data_ptr(), self.slot_of_item.data_ptr(),
            t * k, k, w.hidden, b.ptr_array("rows"), b.ptr_array("scale"), self.item_rank.data_ptr(),
            self.item_row.data_ptr(), b.ptr_array("meta") if self.scatter_return else None,
            b.ptr_array("ret") if self.scatter_return else None, b.ret_rows,
            self.row_dst.data_ptr() if self.scatter_return else None, self.status.data_ptr(), self._s()),
            "sb_ep_exchange_dispatch")
        self.launches += 1
        self._scattered = self.scatter_return

    def stage_experts_and_shared(self) -> None:
        """Routed groups and the shared expert in one pair of weight-streaming launches.

        The row bound handed to the library is the whole receive buffer: the
        streaming kernels sweep a group of any size 16 rows at a time, so a peer
        that sends a prefill-sized batch in the same step (ranks may mix the two
        branches) gets every row computed, only slower than the tile kernel would."""
        w, b, t = self.w, self.bufs, self._t
        has_shared = bool(w.shared_inter) and t > 0
        check(lib.sb_grouped_swiglu_mixed(
            b.local["rows"], self.recv_tiles.data_ptr(), w.w13.data_ptr(), w.w2.data_ptr(),
            w.slot_of_expert.data_ptr(), b.local["scale"], b.recv_cap, w.hidden, w.inter, w.n_slots,
            self.hbuf.data_ptr(), b.local["y"], b.recv_cap,
            self._x.data_ptr() if has_shared else None,
            w.shared_w13.data_ptr() if has_shared else None, w.shared_w2.data_ptr() if has_shared else None,
            self.shared_scale.data_ptr() if has_shared and w.shared_gate_w is not None else None,
            w.shared_inter if has_shared else 0, t if has_shared else 0,
            self.shared_h.data_ptr() if has_shared else None, self.shared_out.data_ptr() if has_shared else None,
            self.row_dst.data_ptr() if self._scattered else None, self.status.data_ptr(), self._s()),
            "sb_grouped_swiglu_mixed")
        self.launches += 2

    def stage_plan(self) -> None:
        check(lib.sb_ep_plan(self.bufs.local["ctl"], self.owner.data_ptr(), self.w.num_experts,
                             self.rank, self.ep, self.bufs.recv_cap, self.dst_base.data_ptr(),
                             self.recv_offsets.data_ptr(), self.recv_tiles.data_ptr(), self._s()),
              "sb_ep_plan")
        self.launches += 1

    def stage_dispatch(self) -> None:
        w, t, k = self.w, self._t, self.top_k
        check(lib.sb_ep_dispatch(
            self._x.data_ptr(), self.topk_idx.data_ptr(), self.topk_w.data_ptr(),
            self.slot_of_item.data_ptr(), self.local_offsets.data_ptr(), self.dst_base.data_ptr(),
            self.owner_row.data_ptr(), t * k, k, w.hidden, self.ep, self.bufs.recv_cap,
            self.bufs.ptr_array("rows"), self.bufs.ptr_array("scale"), self.item_rank.data_ptr(),
            self.item_row.data_ptr(), self.rank, self.bufs.ptr_array("meta") if self.scatter_return else None,
            self._s()), "sb_ep_dispatch")
        self.launches += 1
        self._scattered = self.scatter_return

    def stage_shared(self, passes: int = 3, stages: int = 0) -> None:
        """The shared expert on this rank's own tokens; `passes` 1 / 2 run only its
        gate/up or only its down pass (batches above the decode size), `stages`
        names the GEMM pipeline (-1 leaves room for a router CTA on each SM)."""
        w, t = self.w, self._t
        if not w.shared_inter or t == 0:
            return
        if passes != 3 and not self._small():
            check(lib.sb_grouped_swiglu_passes(
                self._x.data_ptr(), None, t, w.shared_w13.data_ptr(), w.shared_w2.data_ptr(), None,
                self.shared_scale.data_ptr() if w.shared_gate_w is not None else None, t, w.hidden,
                w.shared_inter, 1, self.shared_h.data_ptr(), self.shared_out.data_ptr(), passes, stages,
                self.status.data_ptr(), self._s()), "sb_grouped_swiglu_passes(shared)")
            self.launches += 1
            return
        if passes == 2 and self._small():
            return                          # the decode-sized kernels did both passes in the first call
        if self._small():
            check(lib.sb_decode_experts(
                self._x.data_ptr(), None, 1, None, None, None, None, None, w.hidden, w.inter, 1, None, None,
                w.shared_w13.data_ptr(), w.shared_w2.data_ptr(),
                self.shared_scale.data_ptr() if w.shared_gate_w is not None else None, w.shared_inter, t,
                self.shared_h.data_ptr(), self.shared_out.data_ptr(), self.status.data_ptr(), self._s()),
                "sb_decode_experts(shared)")
            self.launches += 2
            return
        check(lib.sb_grouped_swiglu(
            self._x.data_ptr(), None, t, w.shared_w13.data_ptr(), w.shared_w2.data_ptr(), None,
            self.shared_scale.data_ptr() if w.shared_gate_w is not None else None, t, w.hidden,
            w.shared_inter, 1, self.shared_h.data_ptr(), self.shared_out.data_ptr(),
            self.status.data_ptr(), self._s()), "sb_grouped_swiglu(shared)")
        self.launches += 2

    def stage_resolve(self) -> None:
        """After every rank's rows (and return addresses) have landed."""
        if not self._scattered:
            return
        b = self.bufs
        check(lib.sb_ep_resolve_return(b.local["meta"], self.recv_offsets.data_ptr(), self.w.num_experts,
                                       b.ptr_array("ret"), self.ep, b.ret_rows, self.w.hidden, b.recv_cap,
                                       self.row_dst.data_ptr(), self._s()), "sb_ep_resolve_return")
        self.launches += 1

    def stage_return(self) -> None:
        """Push the finished rows of `y` to their senders (after stage_experts(fused=False))."""
        if not self._scattered:
            return
        b = self.bufs
        check(lib.sb_ep_return_rows(b.local["y"], self.row_dst.data_ptr(), self.recv_offsets.data_ptr(),
                                    self.w.num_experts, self.w.hidden, b.recv_cap, self._s()), "sb_ep_return_rows")
        self.launches += 1

    def stage_experts(self, fused: bool = True) -> None:
        """Routed experts over the received rows.  With return addresses
        (`_scattered`) the rows go back to their senders either from the down GEMM's
        own epilogue (`fused`) or, written to the local `y` first, by stage_return."""
        w, b = self.w, self.bufs
        dst = self.row_dst.data_ptr() if (self._scattered and fused) else None
        if self._small():
            # few rows per expert arrive in a decode step, whatever the peers sent
            check(lib.sb_grouped_swiglu_mixed(
                b.local["rows"], self.recv_tiles.data_ptr(), w.w13.data_ptr(), w.w2.data_ptr(),
                w.slot_of_expert.data_ptr(), b.local["scale"], b.recv_cap, w.hidden, w.inter, w.n_slots,
                self.hbuf.data_ptr(), b.local["y"], 0, None, None, None, None, 0, 0, None, None,
                dst, self.status.data_ptr(), self._s()), "sb_grouped_swiglu_mixed(routed)")
            self.launches += 4
            return
        if self._scattered and fused:
            check(lib.sb_grouped_swiglu_scatter(
                b.local["rows"], self.recv_tiles.data_ptr(), w.w13.data_ptr(), w.w2.data_ptr(),
                w.slot_of_expert.data_ptr(), b.local["scale"], b.recv_cap, w.hidden, w.inter, w.n_slots,
                self.hbuf.data_ptr(), dst, self.status.data_ptr(), self._s()), "sb_grouped_swiglu_scatter")
            self.launches += 2
            return
        check(lib.sb_grouped_swiglu(
            b.local["rows"], self.recv_tiles.data_ptr(), 0, w.w13.data_ptr(), w.w2.data_ptr(),
            w.slot_of_expert.data_ptr(), b.local["scale"], b.recv_cap, w.hidden, w.inter, w.n_slots,
            self.hbuf.data_ptr(), b.local["y"], self.status.data_ptr(), self._s()),
            "sb_grouped_swiglu(routed)")
        self.launches += 2

    def stage_combine(self, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        w, t, k = self.w, self._t, self.top_k
        dst = self.out[:t] if out is None else out
        if self._scattered:
            # every row of this rank's items is already here, in item order; with
            # return addresses the dispatch wrote item_row[i] = i, or -1 for an item
            # that was never sent (expert id out of range, no room), which the
            # combine then skips instead of adding a stale row
            check(lib.sb_combine(self.bufs.local["ret"], self.item_row.data_ptr(), self.topk_idx.data_ptr(),
                                 self.shared_out.data_ptr() if w.shared_inter else None, t, w.hidden, k,
                                 dst.data_ptr(), self._s()), "sb_combine")
            self.launches += 1
            return dst
        check(lib.sb_ep_combine(
            self.bufs.ptr_array("y"), self.item_rank.data_ptr(), self.item_row.data_ptr(),
            self.topk_idx.data_ptr(), self.shared_out.data_ptr() if w.shared_inter else None, t,
            w.hidden, k, self.ep, dst.data_ptr(), self._s()), "sb_ep_combine")
        self.launches += 1
        return dst


class ExpertParallelLayer:
    """One rank of a multi-process expert-parallel layer."""

    _shared_bufs = {}     # (device, hidden, experts, recv_cap, ep) -> PeerBuffers, reused by all layers

    def __init__(self, weights: LayerWeights, top_k: int, max_tokens: int, rank: int, ep: int,
                 process_group, owner: Optional[Sequence[int]] = None, renorm: bool = False,
                 fp32_logits: bool = False, owner_decode: Optional[Sequence[int]] = None):
        if owner is None:
            owner = [e % ep for e in range(weights.num_experts)]
        cap = recv_capacity(max_tokens, top_k, ep)
        key = (str(weights.device), weights.hidden, weights.num_experts, cap, ep)
        bufs = self._shared_bufs.get(key)
        if bufs is None:
            with torch.cuda.device(weights.device):
                bufs = PeerBuffers(weights.hidden, weights.num_experts, cap, ep, rank)
                bufs.allocate_local()
                exchange_handles(bufs, process_group)
            self._shared_bufs[key] = bufs
        self.bufs = bufs
        self.r = EpRank(weights, top_k, max_tokens, rank, ep, owner, bufs, renorm, fp32_logits,
                        owner_decode=owner_decode)
        self.last_launches = 0
        self.overlap = True
        self.router_first = os.environ.get("SPARSE_B200_EP_ROUTER_FIRST", "1") != "0"
        with torch.cuda.device(weights.device):
            self._side = torch.cuda.Stream(device=weights.device)
            self._fork = torch.cuda.Event()
            self._mid = torch.cuda.Event()
            self._join = torch.cuda.Event()
        self._graphs = {}

    @property
    def logits(self):
        return self.r.logits

    @property
    def topk_idx(self):
        return self.r.topk_idx

    @property
    def topk_w(self):
        return self.r.topk_w

    def _barrier(self) -> None:
        self.r.stage_barrier()

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                stage: Optional[str] = None) -> torch.Tensor:
        """One layer pass; `stage` ("prefill" / "decode") picks the destination
        table, None keeps the one in use."""
        r = self.r
        if stage is not None and stage != r.stage:
            r.use_stage(stage)
        r.launches = 0
        marks = self.stage_events
        stream = torch.cuda.current_stream(r.device)

        def mark(name):
            if marks is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(stream)
                marks.append((name, ev))

        with torch.cuda.device(r.device):
            if marks is not None or not self.overlap:
                # one stream, stage after stage: what the per-stage timing marks measure
                mark("begin")
                r.stage_route(x)
                mark("router+sort")
                r.stage_publish()
                self._barrier()
                mark("publish+barrier")
                r.stage_plan()
                r.stage_dispatch()
                mark("plan+dispatch")
                r.stage_shared()
                mark("shared_swiglu")
                self._barrier()
                r.stage_resolve()
                mark("barrier(rows landed)")
            elif x.shape[0] <= _lib.DECODE_MAX_TOKENS and r.small_batch_kernels:
                # Decode-sized step: launch-bound, so one stream, the fewest
                # launches, nothing that a CUDA graph capture could not record.
                # Ranks may take different branches in the same step: every branch
                # runs three barriers and uses the same return protocol.
                r.stage_route(x)
                r.stage_exchange_dispatch()
                r.stage_experts_and_shared()
                self._barrier()
                res = r.stage_combine(out)
                self.last_launches = r.launches
                return res
            else:
                # The router and the sort run first, alone: beside a GEMM a router
                # CTA gets one slot per SM and a share of the issue cycles, takes
                # 190 us instead of 73 us, and everything that follows it (counts,
                # plan, dispatch, the barriers, and the shared expert's down pass,
                # which needs the scalar gate) starts that much later.  Then the
                # send side (counts, plan, dispatch, "rows landed" barrier) runs on
                # the side stream beside both passes of the shared expert.
                # `router_first = False` gives the other order: router beside the
                # shared gate/up pass (what the single-GPU layer does, where there
                # is no send side to wait for).
                tl = self.timeline

                def stamp(name, st):
                    if tl is not None:
                        ev = torch.cuda.Event(enable_timing=True)
                        ev.record(st)
                        tl.append((name, ev))

                r.begin(x)
                has_shared = bool(r.w.shared_inter)
                stamp("begin", stream)
                if self.router_first:
                    r.stage_route(part="router")
                    stamp("main: router done", stream)
                self._fork.record(stream)
                if has_shared and not self.router_first:
                    r.stage_shared(1, stages=-1)
                    stamp("main: shared gate/up done", stream)
                with torch.cuda.stream(self._side):
                    self._side.wait_event(self._fork)
                    if self.router_first:
                        r.stage_route(part="sort")
                        stamp("side: sort done", self._side)
                    else:
                        r.stage_route()
                        stamp("side: router+sort done", self._side)
                        self._mid.record(self._side)
                    r.stage_publish()
                    self._barrier()
                    stamp("side: counts exchanged", self._side)
                    r.stage_plan()
                    r.stage_dispatch()
                    stamp("side: rows dispatched", self._side)
                    self._barrier()
                    r.stage_resolve()
                    stamp("side: rows landed", self._side)
                    self._join.record(self._side)
                if has_shared and self.router_first:
                    r.stage_shared(1)
                    stamp("main: shared gate/up done", stream)
                if not self.router_first:
                    stream.wait_event(self._mid)        # the scalar gate of the shared expert is known
                if has_shared:
                    r.stage_shared(2)
                    stamp("main: shared down done", stream)
                stream.wait_event(self._join)
            fused = marks is None          # the timing marks time the GEMM and the return push separately
            r.stage_experts(fused=fused)
            mark("routed_swiglu")
            if self.timeline is not None and marks is None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(stream)
                self.timeline.append(("main: routed GEMM + return done", ev))
            if not fused:
                r.stage_return()
                mark("return rows")
            self._barrier()
            mark("barrier(outputs ready)")
            res = r.stage_combine(out)
            mark("combine")
            if self.timeline is not None and marks is None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(stream)
                self.timeline.append(("main: combined", ev))
        self.last_launches = r.launches
        return res

    def forward_graphed(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                        stage: Optional[str] = None) -> torch.Tensor:
        """`forward` replayed from a CUDA graph: the first call with a given input
        and output buffer records the step's launches (two streams, device-side
        barrier epochs, nothing baked in that changes from step to step), later
        calls cost the host one graph launch instead of some twenty kernel
        launches.  Recording executes nothing, so every rank must make the same
        sequence of calls (as with `forward`); call `forward` once before the first
        recording so that one-time set-up is not captured."""
        r = self.r
        if stage is not None and stage != r.stage:
            r.use_stage(stage)
        dst = r.out[:x.shape[0]] if out is None else out
        key = (x.data_ptr(), x.shape[0], dst.data_ptr(), r.stage)
        ent = self._graphs.get(key)
        if ent is None:
            if len(self._graphs) >= 32:
                self._graphs.clear()
            stream = torch.cuda.current_stream(r.device)
            cap = torch.cuda.Stream(device=r.device)
            cap.wait_stream(stream)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(cap):
                with torch.cuda.graph(graph, stream=cap, capture_error_mode="thread_local"):
                    self.forward(x, dst)
            stream.wait_stream(cap)
            ent = (graph, self.last_launches, x, dst)       # keeps the buffers alive
            self._graphs[key] = ent
        ent[0].replay()
        self.last_launches = ent[1]
        return ent[3]

    # When set to a list, forward() appends (stage name, CUDA event) marks to it.
    stage_events = None
    # When set to a list, the overlapped (two-stream) path appends (point, CUDA event)
    # stamps on both streams: where each stream stands when, in the real schedule.
    timeline = None

    def check_status(self) -> None:
        self.r.check_status()


class CachedExpertParallelLayer(ExpertParallelLayer):
    """Expert-parallel layer whose owned experts live in pinned host memory with
    an LRU of device slots (`store.ExpertStore`), as the reference runs with
    `expert_offload="cpu"` under EP (utils/eval_core.py:13156-13372 over
    11338-11435).  The received rows are known on the device only, so after the
    "rows landed" barrier the E+1 receive offsets are read back once (the
    reference synchronises per segment) and the experts with rows are made
    resident and run in as few grouped launches as the cache allows, in EPIPE's
    readiness order when that is enabled.  One stream, stage after stage."""

    def __init__(self, cached_runner, top_k: int, max_tokens: int, rank: int, ep: int, process_group,
                 owner=None, renorm: bool = False, fp32_logits: bool = False, owner_decode=None):
        super().__init__(cached_runner.store.w, top_k, max_tokens, rank, ep, process_group, owner=owner,
                         renorm=renorm, fp32_logits=fp32_logits, owner_decode=owner_decode)
        self.cached = cached_runner
        self.r.status = cached_runner.status          # one status word for both
        self.overlap = False

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, stage: str = "") -> torch.Tensor:
        from .context import SparseContext
        r, c = self.r, self.cached
        r.launches = 0
        t = x.shape[0]
        stage = stage or SparseContext.stage(1 if t == 1 else t)
        if stage in r._owners and stage != r.stage:
            r.use_stage(stage)
        with torch.cuda.device(r.device):
            r.stage_route(x)
            r.stage_publish()
            self._barrier()
            r.stage_plan()
            r.stage_dispatch()
            r.stage_shared()
            self._barrier()
            r.stage_resolve()
            needed = c._needed_experts(r.recv_offsets)      # the one host synchronisation
            c.last_needed = needed
            plan = c._epipe_plan(needed, stage)
            c.last_plan = plan
            c.run_routed(needed, r.stage_experts, plan)
            self._barrier()
            res = r.stage_combine(out)
        self.last_launches = r.launches
        return res
