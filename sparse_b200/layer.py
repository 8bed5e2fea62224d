"""Device-resident weights of one MoE layer and the single-call layer pass.

HBM layout (bf16 everywhere):
  routed experts   w13 slab [S, 2I, H]  (per slot: I gate rows, then I up rows)
                   w2  slab [S, H, I]
                   slot_of_expert int32[E]  (expert id -> slab slot, -1 = absent)
  shared expert    w13 [1, 2Is, H], w2 [1, H, Is]
  router           [E, H] (+ fp32 bias [E]), shared scalar gate [H]
A slab addresses every slot through one TMA tensor map, so swapping which
expert sits in a slot only rewrites `slot_of_expert` and the slot's bytes.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from . import _lib
from ._lib import lib, check, MoeLayer


def pack_w13(gate: torch.Tensor, up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gate and up matrices [I,H] -> one slab entry [2I,H] in the row order the
    loaded library expects: stacked (gate rows, then up rows) for the single-CTA
    GEMM, interleaved (g0,u0,g1,u1,...) for the CTA-pair GEMM."""
    i, h = gate.shape
    if out is None:
        out = torch.empty((2 * i, h), dtype=torch.bfloat16, device=gate.device)
    if lib.sb_w13_interleaved():
        out[0::2].copy_(gate)
        out[1::2].copy_(up)
    else:
        out[:i].copy_(gate)
        out[i:].copy_(up)
    return out


class LayerWeights:
    """Weights of one MoE layer on one GPU."""

    def __init__(self, hidden: int, inter: int, num_experts: int, n_slots: int,
                 shared_inter: int, device: torch.device, w13: Optional[torch.Tensor] = None,
                 w2: Optional[torch.Tensor] = None):
        """`w13` / `w2`: slabs the caller already owns (e.g. memory that peer GPUs
        have mapped, `peer_cache.PeerSlab`); allocated here when omitted."""
        self.hidden, self.inter, self.num_experts = hidden, inter, num_experts
        self.n_slots, self.shared_inter = n_slots, shared_inter
        self.device = device
        bf = torch.bfloat16
        if (w13 is None) != (w2 is None):
            raise ValueError("w13 and w2 slabs go together")
        if w13 is not None and (tuple(w13.shape) != (n_slots, 2 * inter, hidden) or
                                tuple(w2.shape) != (n_slots, hidden, inter) or w13.dtype != bf or w2.dtype != bf):
            raise ValueError("external slabs must be bf16 [S,2I,H] and [S,H,I]")
        self.w13 = w13 if w13 is not None else torch.empty((n_slots, 2 * inter, hidden), dtype=bf, device=device)
        self.w2 = w2 if w2 is not None else torch.empty((n_slots, hidden, inter), dtype=bf, device=device)
        self.slot_of_expert = torch.full((num_experts,), -1, dtype=torch.int32, device=device)
        self.router_w: Optional[torch.Tensor] = None
        self.router_bias: Optional[torch.Tensor] = None      # fp32 [E], bf16-rounded values
        self.shared_gate_w: Optional[torch.Tensor] = None    # [H]
        self.shared_w13: Optional[torch.Tensor] = None
        self.shared_w2: Optional[torch.Tensor] = None
        if shared_inter:
            self.shared_w13 = torch.empty((1, 2 * shared_inter, hidden), dtype=bf, device=device)
            self.shared_w2 = torch.empty((1, hidden, shared_inter), dtype=bf, device=device)

    # -- loading ----------------------------------------------------------------
    def set_router(self, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        self.router_w = w.to(device=self.device, dtype=torch.bfloat16).contiguous()
        self.router_bias = None
        if bias is not None:
            self.router_bias = bias.to(torch.bfloat16).to(device=self.device, dtype=torch.float32).contiguous()

    def set_shared(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor,
                   scalar_gate: Optional[torch.Tensor]) -> None:
        pack_w13(gate, up, self.shared_w13[0])
        self.shared_w2[0].copy_(down)
        self.shared_gate_w = None
        if scalar_gate is not None:
            self.shared_gate_w = scalar_gate.reshape(-1).to(device=self.device, dtype=torch.bfloat16).contiguous()

    def load_expert(self, slot: int, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> None:
        """Synchronous (setup-time) load of one expert's three matrices into a slot."""
        pack_w13(gate, up, self.w13[slot])
        self.w2[slot].copy_(down)

    def set_slot_map(self, slot_of_expert: Sequence[int]) -> None:
        self.slot_of_expert.copy_(torch.tensor(list(slot_of_expert), dtype=torch.int32))

    def clone(self) -> "LayerWeights":
        """A second layer with its own copies of every device tensor."""
        import copy
        other = copy.copy(self)
        for name, value in vars(self).items():
            if isinstance(value, torch.Tensor):
                setattr(other, name, value.clone())
        return other

    @classmethod
    def from_block_weights(cls, w, device: torch.device) -> "LayerWeights":
        """All experts resident, slot = expert id.  `w` is a `synth.BlockWeights`."""
        s = w.shape
        lw = cls(s.hidden, s.inter, s.num_experts, s.num_experts, s.shared_inter, device)
        lw.set_router(w.router, w.router_bias)
        for e in range(s.num_experts):
            lw.load_expert(e, w.gate[e], w.up[e], w.down[e])
        lw.set_slot_map(range(s.num_experts))
        if s.shared_inter:
            lw.set_shared(w.sh_gate, w.sh_up, w.sh_down, w.sh_scalar_gate)
        return lw


class LayerRunner:
    """Owns the scratch of one layer pass and calls `sb_moe_layer_forward`."""

    def __init__(self, weights: LayerWeights, top_k: int, max_tokens: int,
                 renorm: bool = False, fp32_logits: bool = False, want_logits: bool = True):
        self.w = weights
        self.top_k, self.renorm, self.fp32_logits = top_k, renorm, fp32_logits
        self.want_logits = want_logits
        self.max_tokens = 0
        self.status = torch.zeros((1,), dtype=torch.int32, device=weights.device)
        dev_index = weights.device.index if weights.device.index is not None else torch.cuda.current_device()
        _lib.init_device(dev_index)
        self._reserve(max_tokens)

    def _reserve(self, tokens: int) -> None:
        w, dev = self.w, self.w.device
        tokens = max(int(tokens), 1)
        self.max_tokens = tokens
        nbytes = lib.sb_moe_layer_workspace_bytes(tokens, w.hidden, w.num_experts, self.top_k,
                                                  w.inter, w.shared_inter)
        # over-allocate so the base can be rounded up to 1024 bytes
        self._ws_raw = torch.empty((nbytes + 1024,), dtype=torch.uint8, device=dev)
        base = self._ws_raw.data_ptr()
        self._ws_ptr = (base + 1023) // 1024 * 1024
        self._ws_bytes = nbytes
        self.out = torch.empty((tokens, w.hidden), dtype=torch.bfloat16, device=dev)
        self.topk_idx = torch.empty((tokens, self.top_k), dtype=torch.int32, device=dev)
        self.topk_w = torch.empty((tokens, self.top_k), dtype=torch.bfloat16, device=dev)
        self.logits = None
        if self.want_logits:
            self.logits = torch.empty((tokens, w.num_experts),
                                      dtype=torch.float32 if self.fp32_logits else torch.bfloat16,
                                      device=dev)

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None):
        """x [T,H] bf16 on the layer's device -> (out [T,H], topk_idx, topk_w, logits).
        Returned tensors are views of buffers this runner reuses on the next call."""
        w = self.w
        if x.dtype != torch.bfloat16 or not x.is_cuda or not x.is_contiguous():
            raise RuntimeError("LayerRunner.forward needs a contiguous CUDA bf16 tensor")
        t = x.shape[0]
        if t > self.max_tokens:
            self._reserve(t)
        dst = self.out[:t] if out is None else out
        L = MoeLayer()
        L.T, L.H, L.E, L.K, L.I, L.I_shared = t, w.hidden, w.num_experts, self.top_k, w.inter, w.shared_inter
        L.renorm, L.n_slots = int(self.renorm), w.n_slots
        L.router_fp32_logits = int(self.fp32_logits)
        L.x = x.data_ptr()
        L.router_w = w.router_w.data_ptr()
        L.router_bias = w.router_bias.data_ptr() if w.router_bias is not None else None
        L.shared_gate_w = w.shared_gate_w.data_ptr() if w.shared_gate_w is not None else None
        L.w13, L.w2 = w.w13.data_ptr(), w.w2.data_ptr()
        L.slot_of_expert = w.slot_of_expert.data_ptr()
        L.shared_w13 = w.shared_w13.data_ptr() if w.shared_w13 is not None else None
        L.shared_w2 = w.shared_w2.data_ptr() if w.shared_w2 is not None else None
        L.out = dst.data_ptr()
        L.logits = self.logits.data_ptr() if self.logits is not None else None
        L.topk_idx, L.topk_w = self.topk_idx.data_ptr(), self.topk_w.data_ptr()
        L.ws, L.ws_bytes = self._ws_ptr, self._ws_bytes
        with torch.cuda.device(w.device):
            stream = torch.cuda.current_stream(w.device).cuda_stream
            check(lib.sb_moe_layer_forward(C.byref(L), self.status.data_ptr(), stream),
                  "sb_moe_layer_forward")
        self.last_launches = int(lib.sb_last_launch_count())
        logits = self.logits[:t] if self.logits is not None else None
        return dst, self.topk_idx[:t], self.topk_w[:t], logits

    def check_status(self) -> None:
        """Host-synchronising check of the device status word (tests, debug)."""
        s = int(self.status.item())
        if s != 0:
            self.status.zero_()
            raise RuntimeError(
                "sparse_b200 device status %d: %s" % (
                    s, "a bounded device-side wait gave up" if s == 1 else
                    "an expert without a resident weight slot was routed to"))
