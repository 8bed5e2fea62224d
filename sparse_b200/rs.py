"""RoutingScout: next-layer expert predictors and the prefetch planner.

Predictor modules and the checkpoint loader accept the reference's on-disk
format unchanged (files `rs_l{target}_inL{source}.pth`; payload keys written by
scripts/train_next_layer_rs.py:603-630; module layouts and state-dict key names
of utils/eval_core.py:3402-3461; loader rules of 3490-3658).  The predictors are
tiny fp32 MLPs and run as ordinary PyTorch modules (CUDA-graph captured by the
bounded stager); they are not part of the bf16 hot path.

The planner is pure host logic over a score map and the LRU cache
(utils/eval_core.py:10040-10107 scoring, 10135-10142 victims, 10144-10262 plan).
"""
from __future__ import annotations

import os
import re
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Set, Tuple

import torch
import torch.nn as nn


# ---- predictor modules (parameter names are part of the checkpoint format) --------

class RoutingScoutMLP(nn.Module):
    """Linear -> BatchNorm -> ReLU -> Dropout -> Linear -> softmax; keys `mlp.{0,1,4}`."""

    def __init__(self, input_dim: int, num_experts: int, hidden_dim: int = 1024):
        super().__init__()
        layers = [nn.Linear(input_dim, hidden_dim), nn.BatchNorm1d(hidden_dim), nn.ReLU(), nn.Dropout(0.1),
                  nn.Linear(hidden_dim, num_experts), nn.Softmax(dim=-1)]
        self.mlp = nn.Sequential(*layers)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.mlp(x.reshape(-1, x.shape[-1]))


class _ResidualBlock(nn.Module):
    """x + Linear(GELU(Linear(LayerNorm(x)))); keys `net.{0,1,4}`."""

    def __init__(self, hidden_dim: int, dropout: float):
        super().__init__()
        self.net = nn.Sequential(nn.LayerNorm(hidden_dim), nn.Linear(hidden_dim, 2 * hidden_dim), nn.GELU(),
                                 nn.Dropout(dropout), nn.Linear(2 * hidden_dim, hidden_dim), nn.Dropout(dropout))

    def forward(self, x):
        return x + self.net(x)


class RoutingScoutResidualMLP(nn.Module):
    """LayerNorm -> Linear -> GELU -> N residual blocks -> LayerNorm -> Linear -> softmax;
    keys `input.{0,1}`, `blocks.{i}.net.*`, `out_norm`, `head`."""

    def __init__(self, input_dim: int, num_experts: int, hidden_dim: int = 1024,
                 num_hidden_layers: int = 3, dropout: float = 0.05):
        super().__init__()
        self.input = nn.Sequential(nn.LayerNorm(input_dim), nn.Linear(input_dim, hidden_dim), nn.GELU(),
                                   nn.Dropout(dropout))
        self.blocks = nn.Sequential(*[_ResidualBlock(hidden_dim, dropout)
                                      for _ in range(max(0, int(num_hidden_layers)))])
        self.out_norm = nn.LayerNorm(hidden_dim)
        self.head = nn.Linear(hidden_dim, num_experts)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self.blocks(self.input(x.reshape(-1, x.shape[-1])))
        return torch.softmax(self.head(self.out_norm(h)), dim=-1)


def _state_dict_of(payload) -> Dict[str, torch.Tensor]:
    if isinstance(payload, dict):
        for key in ("state_dict", "model_state_dict"):
            if isinstance(payload.get(key), dict):
                return payload[key]
        if all(torch.is_tensor(v) for v in payload.values()):
            return payload
    raise RuntimeError("Cannot extract state_dict from payload type=%s" % type(payload))


def module_from_payload(payload, fallback_input_dim: int, fallback_num_experts: int) -> Tuple[nn.Module, str]:
    """Checkpoint payload -> (module, task).  Unknown dict payloads and bare
    state dicts fall back to the plain MLP with hidden 1024."""
    meta = payload if isinstance(payload, dict) else {}
    if meta.get("task", "") == "cache_value_rs":
        raise NotImplementedError("cache-value RS checkpoints are not supported (router_prob task only)")
    in_dim = int(meta.get("input_dim", fallback_input_dim))
    n_exp = int(meta.get("num_experts", fallback_num_experts))
    hid = int(meta.get("hidden_dim", 1024))
    kind = meta.get("model_type", "")
    if kind == "next_layer_residual_logits_rs":
        mod = RoutingScoutResidualMLP(in_dim, n_exp, hid, int(meta.get("num_hidden_layers", 3)), 0.05)
    elif kind == "independent_light_logits_rs":
        mod = RoutingScoutMLP(in_dim, n_exp, hid)
    else:
        mod = RoutingScoutMLP(fallback_input_dim, fallback_num_experts, 1024)
    mod.load_state_dict(_state_dict_of(payload), strict=True)
    if kind:
        mod.rs_feature_mode = str(meta.get("feature_mode", "hidden"))
    return mod, "router_prob"


_CKPT = re.compile(r"rs_l(\d+)_inL(-?\d+)\.pth")


def next_layer_targets(rs_dir: str) -> List[int]:
    out = set()
    for name in os.listdir(rs_dir):
        m = _CKPT.fullmatch(name)
        if m and int(m.group(1)) == int(m.group(2)) + 1:
            out.add(int(m.group(1)))
    return sorted(out)


def load_rs_bank(rs_dir: str, num_layers: int, hidden_dim: int, num_experts: int,
                 device: torch.device, require_complete: bool):
    """-> (ModuleList of num_layers predictors in fp32 eval mode, task, layout,
    source layer per module, list of missing files).

    Layout "next_layer": predictor for target layer t reads layer t-1's hidden
    state (file rs_l{t}_inL{t-1}.pth); otherwise "group" (rs_l{t}_inL0.pth).
    A missing file gets an untrained stand-in MLP unless `require_complete`;
    layers before the first available target are always optional."""
    targets = next_layer_targets(rs_dir)
    layout = "next_layer" if targets else "group"
    mods: List[nn.Module] = []
    sources: List[int] = []
    missing: List[str] = []
    for layer in range(int(num_layers)):
        src = layer - 1 if layout == "next_layer" else 0
        path = os.path.join(rs_dir, "rs_l%d_inL%d.pth" % (layer, src))
        if not os.path.exists(path):
            optional = layout == "next_layer" and bool(targets) and layer < targets[0]
            if not optional:
                missing.append("[L%d] tried: %s" % (layer, os.path.basename(path)))
                if require_complete:
                    continue
            mods.append(RoutingScoutMLP(hidden_dim, num_experts, 1024).to(device, dtype=torch.float32).eval())
            sources.append(src)
            continue
        payload = torch.load(path, map_location="cpu", weights_only=False)
        mod, _task = module_from_payload(payload, hidden_dim, num_experts)
        mods.append(mod.to(device, dtype=torch.float32).eval())
        sources.append(int(payload.get("source_layer", src)) if isinstance(payload, dict) else src)
    if require_complete and missing:
        raise RuntimeError("RS checkpoint set incomplete:\n" + "\n".join(missing[:32]))
    if len(mods) != int(num_layers):
        raise RuntimeError("RS bank size mismatch: got %d modules, expect %d" % (len(mods), num_layers))
    return nn.ModuleList(mods).eval(), "router_prob", layout, sources, missing


# ---- planner ---------------------------------------------------------------------

def prob_score_map(topi: torch.Tensor, topv: torch.Tensor, is_local: Callable[[int], bool],
                   counters: Optional[Callable[[str, int], None]] = None) -> Dict[int, float]:
    """Per predicted expert that this rank would execute:
    sum of its predicted probabilities * (1 + 0.15*(occurrences-1)) + 0.05*max."""
    ids = topi.reshape(-1).tolist()
    probs = topv.float().reshape(-1).tolist()
    total: Dict[int, float] = {}
    seen: Dict[int, int] = {}
    peak: Dict[int, float] = {}
    for e, p in zip(ids, probs):
        e = int(e)
        total[e] = total.get(e, 0.0) + float(p)
        seen[e] = seen.get(e, 0) + 1
        peak[e] = max(peak.get(e, 0.0), float(p))
    local = {e: s for e, s in total.items() if is_local(e)}
    if counters is not None:
        counters("rs_pred_candidate_count", len(total))
        counters("rs_pred_local_candidate_count", len(local))
        counters("rs_pred_nonlocal_candidate_count", len(total) - len(local))
    return {e: s * (1.0 + 0.15 * max(seen[e] - 1, 0)) + 0.05 * peak[e] for e, s in local.items()}


def victims_by_low_value(cache, score_map: Dict[int, float], protect_ids: Set[int],
                         keep_bias: Callable[[int], float]) -> List[int]:
    """Evictable residents, least worth keeping first; LRU order breaks ties."""
    ranked = []
    for pos, e in enumerate(cache.evictable_prefetch_ids(protect_ids)):
        ranked.append((float(score_map.get(int(e), 0.0)) + keep_bias(int(e)), pos, int(e)))
    ranked.sort(key=lambda t: (t[0], t[1]))
    return [e for _, _, e in ranked]


def build_prefetch_plan(score_map: Dict[int, float], cache, *, protect_ids: Set[int], budget: int,
                        min_score: float, replace_advantage: float, replace_margin: float,
                        allow_active_replace: bool, is_local: Callable[[int], bool],
                        keep_bias: Callable[[int], float],
                        counters: Optional[Callable[[str, int], None]] = None
                        ) -> List[Tuple[int, Optional[int]]]:
    """[(expert to fetch, victim to replace or None)], best candidates first.
    Free slots are filled first; then a candidate replaces the least valuable
    evictable resident only if it beats it by `replace_margin` (ratio) or by
    `replace_advantage` (difference); the first candidate that does not stops
    the plan."""
    note = counters or (lambda name, value: None)
    if budget <= 0 or not score_map:
        return []
    n_in = len(score_map)
    cached = low = 0
    cands: List[Tuple[float, int]] = []
    for e, s in score_map.items():
        e, s = int(e), float(s)
        if not is_local(e):
            continue
        if cache.has(e):
            cached += 1
        elif s < min_score:
            low += 1
        else:
            cands.append((s, e))
    note("rs_candidate_filter_in_count", n_in)
    note("rs_candidate_filter_out_cached_count", cached)
    note("rs_candidate_filter_out_low_score_count", low)
    note("prefetch_rejected_low_score", low)
    note("rs_candidate_survived_count", len(cands))
    note("rs_candidate_filter_out_count", max(0, n_in - len(cands)))
    if not cands:
        return []
    cands.sort(key=lambda t: t[0], reverse=True)
    victims = victims_by_low_value(cache, score_map, protect_ids, keep_bias)
    plan: List[Tuple[int, Optional[int]]] = []
    take = min(cache.prefetch_free_slots(), budget, len(cands))
    for s, e in cands[:take]:
        plan.append((e, None))
    pos = take
    left = budget - len(plan)
    if left <= 0:
        return plan
    if not allow_active_replace:
        note("prefetch_rejected_active_replace", min(left, max(0, len(cands) - pos)))
        return plan
    v = 0
    while pos < len(cands) and v < len(victims) and left > 0:
        s, e = cands[pos]
        victim = victims[v]
        worth = float(score_map.get(victim, 0.0)) + keep_bias(victim)
        if s >= worth * replace_margin or (s - worth) >= replace_advantage:
            plan.append((e, victim))
            left -= 1
            pos += 1
            v += 1
        else:
            note("prefetch_rejected_margin", max(1, len(cands) - pos))
            break
    if left > 0 and pos < len(cands) and v >= len(victims):
        note("prefetch_rejected_cache_full", min(left, len(cands) - pos))
    return plan
