"""CPU oracle for the MoE-block hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU with plain torch / numpy ops, what the
reference's MoE block computes for one layer pass.  It is the checker for the
CUDA path: only the tests, the smoke check and the benchmark's CPU-baseline /
reference arm may import it.  Nothing in the `sparse_b200` package imports it
and the product path never falls back to it.

Parity status: PINNED.  `tests/golden/make_golden.py` runs the reference's own
`DistributedSparseMoeBlock` (imported from the reference checkout, CPU,
world=1) on seeded inputs and stores its outputs under `tests/golden/`;
`tests/test_oracle_golden.py` checks every function here against those files.

Reference anchors (paths inside the reference project):
  router            utils/eval_core.py:9519-9520, 9591-9595
  world=1 experts   utils/eval_core.py:14690-14721
  expert SwiGLU     utils/eval_core.py:11767-11793
  shared expert     utils/eval_core.py:9455-9463
  combine           utils/eval_core.py:523-538
  EP dispatch       utils/eval_core.py:14865-14900, 15048-15060
  local executor    utils/eval_core.py:13240-13253
  destinations      utils/eval_core.py:6736-6769, 4573-4576

Two deliberate, documented choices where the reference leaves the bits to the
library it happens to run on:

* top-k ties.  `torch.topk` does not define which of several equal
  probabilities it returns and the CPU and CUDA implementations disagree.  The
  oracle uses "larger probability first, then smaller expert id", which is what
  a stable descending sort gives.  Exact ties only occur with bf16 logits.
* router accumulation order.  The reference's logits come from a library GEMM
  whose fp32 summation order is unspecified.  `router_logits_fixed_order`
  defines one (per lane an even and an odd partial sum over interleaved groups
  of 8 elements, then an xor-butterfly) that the CUDA kernel follows bit for bit;
  `router_logits_library` is the reference's literal `F.linear` call.  The two
  differ only by rare 1-ulp roundings of a logit.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------
# Router  (utils/eval_core.py:9519-9520, 9591-9595)
# --------------------------------------------------------------------------

def router_logits_library(x: torch.Tensor, wg: torch.Tensor,
                          bias: Optional[torch.Tensor]) -> torch.Tensor:
    """`router_logits = self.gate(x)` exactly as the reference calls it: one
    library GEMM in the model dtype (utils/eval_core.py:9519)."""
    return F.linear(x, wg, bias)


def _fixed_order_dot(xf: np.ndarray, wf: np.ndarray) -> np.ndarray:
    """fp32 dot products of every row of xf [T,H] with every row of wf [R,H]
    in the summation order the CUDA router kernel uses.

    The H elements are cut into groups of 8.  Lane `l` (0..31) takes groups
    l, l+32, l+64, ... in increasing order and keeps two partial sums, one over
    the even and one over the odd elements of its groups, each step
    `p = fl(p + fl(x*w))`; its lane sum is `fl(p_even + p_odd)`.  The 32 lane
    sums are then combined by an xor-butterfly with offsets 16, 8, 4, 2, 1."""
    t, h = xf.shape
    r = wf.shape[0]
    assert h % 8 == 0
    groups = h // 8
    part = np.zeros((2, t, r, 32), dtype=np.float32)
    steps = (groups + 31) // 32
    for j in range(steps):
        nl = min(32, groups - j * 32)
        base = (j * 32 + np.arange(nl)) * 8
        for i in range(8):
            cols = base + i
            prod = xf[:, None, cols] * wf[None, :, cols]                  # fl(x*w)
            part[i & 1][:, :, :nl] = part[i & 1][:, :, :nl] + prod        # fl(p + .)
    acc = part[0] + part[1]
    lanes = np.arange(32)
    for off in (16, 8, 4, 2, 1):
        acc = acc + acc[:, :, lanes ^ off]
    return acc[:, :, 0]


def router_logits_fixed_order(x: torch.Tensor, wg: torch.Tensor,
                              bias: Optional[torch.Tensor]) -> torch.Tensor:
    """Router logits in the model dtype with the defined summation order: fp32
    accumulate, add the bias in fp32, round once to the model dtype."""
    dt = x.dtype
    acc = _fixed_order_dot(x.float().numpy(), wg.to(dt).float().numpy())
    if bias is not None:
        acc = acc + bias.to(dt).float().numpy()[None, :]
    return torch.from_numpy(acc).to(dt)


def softmax_topk(logits: torch.Tensor, top_k: int, norm_topk_prob: bool,
                 out_dtype: torch.dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    """softmax in fp32 over the model-dtype logits, top-k, optional
    renormalisation, cast of the weights to the activation dtype
    (utils/eval_core.py:9520, 9591-9595).  Ties: smaller expert id first."""
    probs = torch.softmax(logits, dim=-1, dtype=torch.float32)
    sv, si = torch.sort(probs, dim=-1, descending=True, stable=True)
    topv = sv[:, :top_k].contiguous()
    topi = si[:, :top_k].contiguous()
    if norm_topk_prob:
        topv = topv / topv.sum(dim=-1, keepdim=True).clamp_min(1e-12)
    return topv.to(out_dtype), topi.to(torch.long)


def tie_rows(logits: torch.Tensor, top_k: int) -> torch.Tensor:
    """bool[T]: rows whose top-(k+1) probabilities contain an exact tie, i.e.
    rows where the library's unspecified tie-breaking can change the selected
    set or the slot order."""
    probs = torch.softmax(logits, dim=-1, dtype=torch.float32)
    sv, _ = torch.sort(probs, dim=-1, descending=True, stable=True)
    kk = min(top_k + 1, sv.shape[1])
    head = sv[:, :kk]
    return (head[:, 1:] == head[:, :-1]).any(dim=-1)


# --------------------------------------------------------------------------
# Experts  (utils/eval_core.py:11767-11793, 14690-14721, 9455-9463)
# --------------------------------------------------------------------------

def expert_mlp(rows: torch.Tensor, gw: torch.Tensor, uw: torch.Tensor,
               dw: torch.Tensor) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)); every op rounds to the activation dtype
    (utils/eval_core.py:11787-11790)."""
    gate = F.linear(rows, gw)
    up = F.linear(rows, uw)
    return F.linear(F.silu(gate) * up, dw)


def experts_world1(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor,
                   gate: Sequence[torch.Tensor], up: Sequence[torch.Tensor],
                   down: Sequence[torch.Tensor]) -> torch.Tensor:
    """Single-rank routed-expert pass: ascending expert id, scale by the route
    weight in the activation dtype, index_add_ into a zero tensor
    (utils/eval_core.py:14690-14721)."""
    t, h = x.shape
    num_experts = len(gate)
    final = torch.zeros((t, h), dtype=x.dtype)
    mask = F.one_hot(idx.to(torch.long), num_classes=num_experts).permute(2, 1, 0)
    for e in range(num_experts):
        idx_k, top_x = torch.where(mask[e])
        if top_x.numel() == 0:
            continue
        cur = x[top_x]
        y = expert_mlp(cur, gate[e], up[e], down[e])
        y = y * w[top_x, idx_k, None]
        final.index_add_(0, top_x, y.to(x.dtype))
    return final


def shared_expert(x: torch.Tensor, sh_gate: Optional[torch.Tensor],
                  sh_up: Optional[torch.Tensor], sh_down: Optional[torch.Tensor],
                  sh_scalar_gate: Optional[torch.Tensor]) -> torch.Tensor:
    """sigmoid(shared_expert_gate(x)) * shared_expert(x), or the plain shared
    MLP when there is no scalar gate (utils/eval_core.py:9455-9463)."""
    if sh_gate is None:
        return torch.zeros_like(x)
    shared = expert_mlp(x, sh_gate, sh_up, sh_down)
    if sh_scalar_gate is not None:
        shared = torch.sigmoid(F.linear(x, sh_scalar_gate)) * shared
    return shared


def combine_expert_outputs(parts: torch.Tensor, expert_ids: torch.Tensor) -> torch.Tensor:
    """Sum the K returned rows of each token in ascending expert id, every add
    rounding to the activation dtype (utils/eval_core.py:523-538)."""
    tokens, slots, hidden = parts.shape
    assert expert_ids.shape == (tokens, slots)
    order = torch.argsort(expert_ids, dim=1, stable=True)
    result = parts.new_zeros((tokens, hidden))
    rows = torch.arange(tokens)
    for s in range(slots):
        result.add_(parts[rows, order[:, s]])
    return result


# --------------------------------------------------------------------------
# Permutation  (utils/eval_core.py:13240-13253; 14873-14882)
# --------------------------------------------------------------------------

def expert_sorted_permutation(item_expert: torch.Tensor, num_experts: int
                              ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Stable sort of the flat (token, slot) items by expert id.

    Returns (slot_of_item[n], item_of_slot[n], expert_offsets[E+1]).  The
    reference sorts with `argsort` and takes segment boundaries from the sorted
    ids; which of several equal keys comes first is not defined there, so the
    stable order (smaller flat index first) is the canonical one."""
    flat = item_expert.reshape(-1).to(torch.long)
    item_of_slot = torch.argsort(flat, stable=True)
    slot_of_item = torch.empty_like(item_of_slot)
    slot_of_item[item_of_slot] = torch.arange(flat.numel())
    counts = torch.bincount(flat, minlength=num_experts)
    offsets = torch.zeros(num_experts + 1, dtype=torch.long)
    offsets[1:] = torch.cumsum(counts, 0)
    return slot_of_item, item_of_slot, offsets


# --------------------------------------------------------------------------
# Whole block, world = 1  (utils/eval_core.py:16418-16563)
# --------------------------------------------------------------------------

def cast_weights(w, dtype: torch.dtype) -> Dict[str, object]:
    """Cast a `sparse_b200.synth.BlockWeights`-like object to the model dtype."""
    c = lambda t: None if t is None else t.to(dtype)
    return {
        "router": c(w.router), "router_bias": c(w.router_bias),
        "gate": [c(t) for t in w.gate], "up": [c(t) for t in w.up],
        "down": [c(t) for t in w.down],
        "sh_gate": c(w.sh_gate), "sh_up": c(w.sh_up), "sh_down": c(w.sh_down),
        "sh_scalar_gate": c(w.sh_scalar_gate),
    }


def moe_block_forward(x: torch.Tensor, cw: Dict[str, object], top_k: int,
                      norm_topk_prob: bool = False,
                      router: str = "fixed_order",
                      logits_override: Optional[torch.Tensor] = None
                      ) -> Dict[str, torch.Tensor]:
    """One layer pass at world=1.  `x` is [T,H] in the model dtype, `cw` the
    output of `cast_weights` in the same dtype."""
    if logits_override is not None:
        logits = logits_override
    elif router == "library":
        logits = router_logits_library(x, cw["router"], cw["router_bias"])
    else:
        logits = router_logits_fixed_order(x, cw["router"], cw["router_bias"])
    topv, topi = softmax_topk(logits, top_k, norm_topk_prob, x.dtype)
    expert_out = experts_world1(x, topi, topv, cw["gate"], cw["up"], cw["down"])
    shared_out = shared_expert(x, cw["sh_gate"], cw["sh_up"], cw["sh_down"],
                               cw["sh_scalar_gate"])
    out = expert_out + shared_out
    return {"out": out, "logits": logits, "topi": topi, "topv": topv,
            "expert_out": expert_out, "shared_out": shared_out}


# --------------------------------------------------------------------------
# Expert-parallel pass, all ranks simulated in one process
# (utils/eval_core.py:14865-14900, 13156-13372, 15048-15060)
# --------------------------------------------------------------------------

def round_robin_owner(num_experts: int, ep: int) -> torch.Tensor:
    """rr_expert_to_rank[e] = e % ep (utils/eval_core.py:4573-4576)."""
    return torch.arange(num_experts, dtype=torch.long) % ep


def ep_dispatch_plan(topi: torch.Tensor, owner: torch.Tensor, ep: int
                     ) -> Dict[str, torch.Tensor]:
    """Source-side plan for one rank: destination of each flat item, stable
    sort by destination, per-destination send counts
    (utils/eval_core.py:14873-14882)."""
    flat_i = topi.reshape(-1).to(torch.long)
    dest = owner[flat_i]
    sort_idx = torch.argsort(dest, stable=True)
    send_counts = torch.bincount(dest, minlength=ep)
    return {"flat_i": flat_i, "dest": dest, "sort_idx": sort_idx,
            "send_counts": send_counts}


def ep_block_forward(xs: List[torch.Tensor], cw: Dict[str, object], top_k: int,
                     owner: torch.Tensor, norm_topk_prob: bool = False,
                     router: str = "fixed_order") -> List[Dict[str, torch.Tensor]]:
    """Layer pass with tokens sharded over `len(xs)` ranks and experts owned per
    `owner[e]`, or per source rank `owner[s][e]` when experts are replicated
    (the reference's dest_rank_table, utils/eval_core.py:672-717).  Mirrors dispatch -> local sorted-segment executor -> return ->
    unsort -> combine; the all-to-alls are list shuffles."""
    ep = len(xs)
    h = xs[0].shape[1]
    routed, plans = [], []
    for x in xs:
        if router == "library":
            logits = router_logits_library(x, cw["router"], cw["router_bias"])
        else:
            logits = router_logits_fixed_order(x, cw["router"], cw["router_bias"])
        topv, topi = softmax_topk(logits, top_k, norm_topk_prob, x.dtype)
        routed.append((logits, topv, topi))
        own = torch.as_tensor(owner)
        plans.append(ep_dispatch_plan(topi, own[len(plans)] if own.dim() == 2 else own, ep))
    # dispatch: chunk [src -> dst]
    send = []
    for r, x in enumerate(xs):
        p = plans[r]
        k = routed[r][2].shape[1]
        expanded = x.unsqueeze(1).expand(-1, k, -1).reshape(-1, h)
        sh = expanded[p["sort_idx"]]
        si = p["flat_i"][p["sort_idx"]]
        sw = routed[r][1].reshape(-1)[p["sort_idx"]]
        bounds = torch.zeros(ep + 1, dtype=torch.long)
        bounds[1:] = torch.cumsum(p["send_counts"], 0)
        send.append([(sh[bounds[d]:bounds[d + 1]], si[bounds[d]:bounds[d + 1]],
                      sw[bounds[d]:bounds[d + 1]]) for d in range(ep)])
    # local execution on each destination
    returned = [[None] * ep for _ in range(ep)]   # [dst][src] rows
    recv_meta = []
    for d in range(ep):
        rh = torch.cat([send[s][d][0] for s in range(ep)], 0)
        ri = torch.cat([send[s][d][1] for s in range(ep)], 0)
        rw = torch.cat([send[s][d][2] for s in range(ep)], 0)
        order = torch.argsort(ri, stable=True)
        out_sorted = torch.zeros_like(rh)
        hs, es, ws = rh[order], ri[order], rw[order]
        for e in torch.unique(es).tolist():
            m = es == e
            y = expert_mlp(hs[m], cw["gate"][e], cw["up"][e], cw["down"][e])
            out_sorted[m] = y * ws[m].unsqueeze(1)
        local_out = torch.zeros_like(rh)
        local_out[order] = out_sorted
        recv_meta.append({"recv_i": ri, "order": order})
        pos = 0
        for s in range(ep):
            n = send[s][d][0].shape[0]
            returned[d][s] = local_out[pos:pos + n]
            pos += n
    results = []
    for r, x in enumerate(xs):
        logits, topv, topi = routed[r]
        t, k = topi.shape
        gathered = torch.cat([returned[d][r] for d in range(ep)], 0)
        unsorted = torch.empty_like(gathered)
        unsorted[plans[r]["sort_idx"]] = gathered
        expert_out = combine_expert_outputs(unsorted.view(t, k, h), topi)
        shared_out = shared_expert(x, cw["sh_gate"], cw["sh_up"], cw["sh_down"],
                                   cw["sh_scalar_gate"])
        results.append({"out": expert_out + shared_out, "logits": logits,
                        "topi": topi, "topv": topv,
                        "send_counts": plans[r]["send_counts"],
                        "recv_i": recv_meta[r]["recv_i"]})
    return results
