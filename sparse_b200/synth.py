"""Seeded synthetic weights and inputs for the MoE-block workloads.

Real checkpoints and prompt datasets are not available offline, so every
measurement and parity case uses random-init weights N(0, 0.02) and hidden
states N(0, 1) of the published block shapes.  All tensors are drawn on the
CPU generator in a fixed order so that the same seeds give the same bits in
the golden-vector generator, in the tests and in the benchmark.

Draw order for the weights (seed `weight_seed`): router gate, then for every
routed expert gate_proj, up_proj, down_proj, then the shared expert
gate/up/down, then the shared scalar gate.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch


@dataclass(frozen=True)
class BlockShape:
    """Shape of one MoE block."""
    hidden: int
    num_experts: int
    inter: int
    top_k: int
    shared_inter: int          # 0 = no shared expert
    shared_gate: bool          # sigmoid scalar gate on the shared expert
    norm_topk_prob: bool = False

    @property
    def routed_expert_bytes_bf16(self) -> int:
        return 3 * self.hidden * self.inter * 2

    def flops_per_token(self) -> int:
        h, e, i, k = self.hidden, self.num_experts, self.inter, self.top_k
        f = 2 * h * e + k * (2 * h * 2 * i + 2 * i * h)
        if self.shared_inter:
            f += 2 * 3 * h * self.shared_inter
        if self.shared_gate:
            f += 2 * h
        return f


QWEN_MOE = BlockShape(hidden=2048, num_experts=60, inter=1408, top_k=4,
                      shared_inter=5632, shared_gate=True)
DEEPSEEK_V2_LITE = BlockShape(hidden=2048, num_experts=64, inter=1408, top_k=6,
                              shared_inter=2816, shared_gate=False)
# Small ragged shape for fast tests (all dims still legal for the kernels).
TINY = BlockShape(hidden=256, num_experts=8, inter=192, top_k=2,
                  shared_inter=320, shared_gate=True)


@dataclass
class BlockWeights:
    """fp32 master weights in nn.Linear layout ([out, in])."""
    shape: BlockShape
    router: torch.Tensor                      # [E, H]
    router_bias: Optional[torch.Tensor]       # [E] or None
    gate: List[torch.Tensor] = field(default_factory=list)   # E x [I, H]
    up: List[torch.Tensor] = field(default_factory=list)     # E x [I, H]
    down: List[torch.Tensor] = field(default_factory=list)   # E x [H, I]
    sh_gate: Optional[torch.Tensor] = None    # [Is, H]
    sh_up: Optional[torch.Tensor] = None      # [Is, H]
    sh_down: Optional[torch.Tensor] = None    # [H, Is]
    sh_scalar_gate: Optional[torch.Tensor] = None  # [1, H]


def make_weights(shape: BlockShape, weight_seed: int = 0, std: float = 0.02,
                 zipf_s: float = 0.0, zipf_seed: int = 7) -> BlockWeights:
    """Draw the block's weights.  `zipf_s > 0` adds a router bias of
    log(Zipf(s) weight) over a seeded random expert permutation, which gives
    skewed, co-activated expert popularity."""
    g = torch.Generator(device="cpu")
    g.manual_seed(int(weight_seed))

    def draw(*size):
        return torch.randn(*size, generator=g, dtype=torch.float32) * std

    h, e, i = shape.hidden, shape.num_experts, shape.inter
    w = BlockWeights(shape=shape, router=draw(e, h), router_bias=None)
    for _ in range(e):
        w.gate.append(draw(i, h))
        w.up.append(draw(i, h))
        w.down.append(draw(h, i))
    if shape.shared_inter:
        w.sh_gate = draw(shape.shared_inter, h)
        w.sh_up = draw(shape.shared_inter, h)
        w.sh_down = draw(h, shape.shared_inter)
    if shape.shared_gate:
        w.sh_scalar_gate = draw(1, h)
    if zipf_s > 0.0:
        w.router_bias = zipf_router_bias(e, zipf_s, zipf_seed)
    return w


def zipf_router_bias(num_experts: int, s: float, seed: int) -> torch.Tensor:
    """bias[perm[r]] = log(normalised Zipf weight of rank r+1)."""
    ranks = torch.arange(1, num_experts + 1, dtype=torch.float64)
    wts = ranks.pow(-float(s))
    wts = wts / wts.sum()
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))
    perm = torch.randperm(num_experts, generator=g)
    bias = torch.empty(num_experts, dtype=torch.float64)
    bias[perm] = wts.log()
    return bias.to(torch.float32)


def make_hidden(tokens: int, hidden: int, seed: int = 1) -> torch.Tensor:
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))
    return torch.randn(tokens, hidden, generator=g, dtype=torch.float32)


def expected_distinct_experts(shape: BlockShape, tokens: int) -> float:
    e, k = shape.num_experts, shape.top_k
    return e * (1.0 - math.pow(1.0 - k / e, tokens))
