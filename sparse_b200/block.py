"""Block-level API of the B200 MoE layer.

`B200MoeBlock` is the object a serving loop holds per MoE layer: it owns the
layer's device weights, the scratch of the layer pass and (for expert
parallelism) the peer-memory buffers, and exposes

    forward_device(x_dev)          -> out_dev            inputs already in HBM
    forward_host(x_pinned, out_pinned)                    host buffers, copies included
    forward(hidden_states[B,S,H])  -> (out, router_logits) | out
                                      the `DistributedSparseMoeBlock.forward`
                                      contract (utils/eval_core.py:16418-16563)

Everything it computes goes through the C ABI; there is no eager fallback.
"""
from __future__ import annotations

from typing import Optional

import torch

from .layer import LayerRunner, LayerWeights


class B200MoeBlock:
    def __init__(self, weights: LayerWeights, top_k: int, max_tokens: int,
                 norm_topk_prob: bool = False, fp32_router_logits: bool = False,
                 return_router_logits: bool = True, ep_rank: int = 0, ep_size: int = 1,
                 process_group=None, owner=None, use_graphs: bool = False):
        self.weights = weights
        self.device = weights.device
        self.top_k = top_k
        self.ep_rank, self.ep_size = ep_rank, ep_size
        self.return_router_logits = return_router_logits
        self.runner = LayerRunner(weights, top_k, max_tokens, renorm=norm_topk_prob,
                                  fp32_logits=fp32_router_logits, want_logits=True)
        self._ep = None
        if ep_size > 1:
            from .ep import ExpertParallelLayer
            self._ep = ExpertParallelLayer(weights, top_k, max_tokens, ep_rank, ep_size,
                                           process_group, owner=owner, renorm=norm_topk_prob,
                                           fp32_logits=fp32_router_logits)
        self._x_stage: Optional[torch.Tensor] = None
        self.last_launches = 0
        # Replay each (input buffer, output buffer) pair's step from a CUDA graph
        # (see `forward_device`); off by default because a graph pins its buffers.
        self.use_graphs = use_graphs
        self._graphs = {}

    @classmethod
    def from_block_weights(cls, w, device: torch.device, ep_rank: int = 0, ep_size: int = 1,
                           max_tokens: int = 4096, process_group=None, placement=None,
                           layer_idx: int = 0, stage: str = "prefill",
                           use_graphs: bool = False) -> "B200MoeBlock":
        """Build from seeded `synth.BlockWeights`; at ep_size > 1 only the
        experts this rank serves are loaded: round-robin (e % ep_size) by default,
        or every expert a `placement.Placement` lists `ep_rank` as a replica of,
        with that placement's per-source destination table."""
        s = w.shape
        owner = None
        if ep_size == 1:
            lw = LayerWeights.from_block_weights(w, device)
        else:
            if placement is not None:
                owned = sorted(placement.receive_experts(layer_idx, ep_rank, stage))
                owner = placement.dest_table(layer_idx, stage)
            else:
                owned = [e for e in range(s.num_experts) if e % ep_size == ep_rank]
            lw = LayerWeights(s.hidden, s.inter, s.num_experts, max(1, len(owned)), s.shared_inter, device)
            lw.set_router(w.router, w.router_bias)
            slot_of = [-1] * s.num_experts
            for slot, e in enumerate(owned):
                lw.load_expert(slot, w.gate[e], w.up[e], w.down[e])
                slot_of[e] = slot
            lw.set_slot_map(slot_of)
            if s.shared_inter:
                lw.set_shared(w.sh_gate, w.sh_up, w.sh_down, w.sh_scalar_gate)
        return cls(lw, s.top_k, max_tokens, norm_topk_prob=s.norm_topk_prob,
                   fp32_router_logits=not s.shared_gate and s.num_experts == 64,
                   ep_rank=ep_rank, ep_size=ep_size, process_group=process_group, owner=owner,
                   use_graphs=use_graphs)

    # -- the three entry points -----------------------------------------------------
    def forward_device(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One layer pass on device-resident rows.  With `use_graphs` the launches
        of a pass are recorded once per (input buffer, row count, output buffer)
        and replayed afterwards: a serving loop that cycles through a few fixed
        buffers pays one graph launch per step instead of ten to twenty kernel
        launches from Python.  The first pass on new buffers runs un-recorded
        (one-time set-up must not be captured); under expert parallelism every
        rank has to make the same sequence of calls."""
        if self._ep is not None:
            if self.use_graphs and self._warm:
                res = self._ep.forward_graphed(x, out)
            else:
                res = self._ep.forward(x, out)
                self._warm = True
            self.last_launches = self._ep.last_launches
            return res
        if self.use_graphs and self._warm and x.shape[0] <= self.runner.max_tokens:
            return self._forward_graphed_local(x, out)
        res, _, _, _ = self.runner.forward(x, out)
        self._warm = True
        self.last_launches = self.runner.last_launches
        return res

    _warm = False

    def _forward_graphed_local(self, x: torch.Tensor, out: Optional[torch.Tensor]) -> torch.Tensor:
        dst = self.runner.out[:x.shape[0]] if out is None else out
        key = (x.data_ptr(), x.shape[0], dst.data_ptr())
        ent = self._graphs.get(key)
        if ent is None:
            if len(self._graphs) >= 32:
                self._graphs.clear()
            stream = torch.cuda.current_stream(self.device)
            cap = torch.cuda.Stream(device=self.device)
            cap.wait_stream(stream)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(cap):
                with torch.cuda.graph(graph, stream=cap, capture_error_mode="thread_local"):
                    self.runner.forward(x, dst)
            stream.wait_stream(cap)
            ent = (graph, self.runner.last_launches, x, dst)
            self._graphs[key] = ent
        ent[0].replay()
        self.last_launches = ent[1]
        return ent[3]

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """x_host, out_host: pinned bf16 [T,H].  Copies in, runs the layer, copies
        the result out; returns when `out_host` is valid."""
        t, h = x_host.shape
        if self._x_stage is None or self._x_stage.shape[0] < t:
            self._x_stage = torch.empty((max(t, self.runner.max_tokens), h), dtype=torch.bfloat16,
                                        device=self.device)
        xd = self._x_stage[:t]
        xd.copy_(x_host, non_blocking=True)
        out = self.forward_device(xd)
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()

    def host_pipeline(self, depth: int = 3) -> "HostPipeline":
        """A queue for host-resident batches: copy-in, layer and copy-out of
        successive batches overlap (see `HostPipeline`)."""
        return HostPipeline(self, depth)

    def forward(self, hidden_states: torch.Tensor):
        b, s, h = hidden_states.shape
        x = hidden_states.reshape(-1, h)
        if x.dtype != torch.bfloat16:
            raise RuntimeError("B200MoeBlock computes in bf16; got %s" % x.dtype)
        out = torch.empty_like(x)
        self.forward_device(x.contiguous(), out)
        out = out.view(b, s, h)
        if not self.return_router_logits:
            return out
        return out, self.router_logits(x.shape[0])

    def router_logits(self, tokens: int) -> torch.Tensor:
        src = self._ep.logits if self._ep is not None else self.runner.logits
        return src[:tokens]

    def topk(self, tokens: int):
        r = self._ep if self._ep is not None else self.runner
        return r.topk_idx[:tokens], r.topk_w[:tokens]

    def check_status(self) -> None:
        (self._ep or self.runner).check_status()


class HostPipeline:
    """Streams host batches through a block: batch i+1 is copied to the device
    and batch i-1 is copied back while batch i is in the layer.

    `submit(x_host, out_host)` enqueues one batch (pinned bf16 [T,H] buffers) and
    returns at once; `out_host` is valid after `wait(ticket)` or `drain()`.  Each
    of `depth` slots owns a device input and output buffer; a slot is reused only
    after its copy-out has finished (an event wait on the copy-in stream, not a
    host sync).  The layer itself runs on the stream that was current when the
    pipeline was built."""

    def __init__(self, block: B200MoeBlock, depth: int = 3):
        if depth < 2:
            raise ValueError("a pipeline needs at least 2 slots")
        self.block = block
        dev = block.device
        t, h = block.runner.max_tokens, block.weights.hidden
        with torch.cuda.device(dev):
            self.compute = torch.cuda.current_stream(dev)
            self.h2d = torch.cuda.Stream(device=dev)
            self.d2h = torch.cuda.Stream(device=dev)
            self.x_dev = [torch.empty((t, h), dtype=torch.bfloat16, device=dev) for _ in range(depth)]
            self.out_dev = [torch.empty((t, h), dtype=torch.bfloat16, device=dev) for _ in range(depth)]
            self.ev_in = [torch.cuda.Event() for _ in range(depth)]
            self.ev_done = [torch.cuda.Event() for _ in range(depth)]
            self.ev_out = [torch.cuda.Event() for _ in range(depth)]
        self.depth = depth
        self.count = 0

    def submit(self, x_host: torch.Tensor, out_host: torch.Tensor) -> int:
        t = x_host.shape[0]
        if t > self.x_dev[0].shape[0]:
            raise RuntimeError("pipeline was sized for %d rows, got %d" % (self.x_dev[0].shape[0], t))
        slot = self.count % self.depth
        xd, od = self.x_dev[slot][:t], self.out_dev[slot][:t]
        if self.count >= self.depth:
            self.h2d.wait_event(self.ev_out[slot])          # the slot's previous result has left the device
        with torch.cuda.stream(self.h2d):
            xd.copy_(x_host, non_blocking=True)
            self.ev_in[slot].record(self.h2d)
        self.compute.wait_event(self.ev_in[slot])
        with torch.cuda.stream(self.compute):
            self.block.forward_device(xd, od)
            self.ev_done[slot].record(self.compute)
        self.d2h.wait_event(self.ev_done[slot])
        with torch.cuda.stream(self.d2h):
            out_host.copy_(od, non_blocking=True)
            self.ev_out[slot].record(self.d2h)
        self.count += 1
        return self.count - 1

    def wait(self, ticket: int) -> None:
        """Blocks until the result of `submit` number `ticket` is in its host buffer
        (only the last `depth` tickets can still be waited for)."""
        if ticket < self.count - self.depth or ticket >= self.count:
            raise ValueError("ticket %d is not in flight" % ticket)
        self.ev_out[ticket % self.depth].synchronize()

    def drain(self) -> None:
        self.d2h.synchronize()
        self.compute.synchronize()
