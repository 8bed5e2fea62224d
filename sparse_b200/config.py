"""Runtime switches of the MoE block, read ONCE at construction.

The reference reads several hundred `SPARSE_*` environment variables, many of
them on the hot path of every call (utils/eval_core.py:279-292, 10267-10296,
13176, 14656, 16463).  Here the in-scope switches are parsed into one frozen
dataclass when a block is built.  Names, defaults and the per-rank CSV forms
(`NAME_BY_RANK=a,b,c,d`) follow the reference; `method_settings` is the
launcher's method table (scripts/run/run_case.sh:85-138, 220-281).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, Mapping, Optional, Tuple

_TRUE = ("1", "true", "yes", "on")


def env_flag(env: Mapping[str, str], name: str, default: str = "0") -> bool:
    return str(env.get(name, default)).strip().lower() in _TRUE


def env_int(env: Mapping[str, str], name: str, default: int) -> int:
    try:
        return int(str(env.get(name, default)).strip())
    except ValueError:
        return int(default)


def env_float(env: Mapping[str, str], name: str, default: float) -> float:
    try:
        return float(str(env.get(name, default)).strip())
    except ValueError:
        return float(default)


def rank_value(env: Mapping[str, str], name: str, rank: int) -> Optional[str]:
    """Entry `rank` of a comma-separated per-rank list, or None (utils/eval_core.py:10267-10293)."""
    raw = str(env.get(name, "") or "").strip()
    if not raw:
        return None
    parts = [p.strip() for p in raw.split(",")]
    if 0 <= rank < len(parts) and parts[rank] != "":
        return parts[rank]
    return None


def rank_int(env, name: str, rank: int, default: int) -> int:
    v = rank_value(env, name, rank)
    try:
        return int(v) if v is not None else int(default)
    except ValueError:
        return int(default)


def rank_float(env, name: str, rank: int, default: float) -> float:
    v = rank_value(env, name, rank)
    try:
        return float(v) if v is not None else float(default)
    except ValueError:
        return float(default)


def cache_capacity_for_rank(env, configured: int, rank: int) -> int:
    """`SPARSE_EXPERT_CACHE_BY_RANK` / `_BY_COMM_RANK` override the CLI value
    per rank; either a plain list `8,8,8,8` or `rank:value` pairs (utils/eval_core.py:295-362)."""
    for name in ("SPARSE_EXPERT_CACHE_BY_COMM_RANK", "SPARSE_EXPERT_CACHE_BY_RANK"):
        raw = str(env.get(name, "") or "").strip()
        if not raw:
            continue
        if ":" in raw:
            table: Dict[int, int] = {}
            for item in raw.replace(";", ",").split(","):
                item = item.strip()
                if not item:
                    continue
                k, _, v = item.partition(":")
                try:
                    table[int(k)] = int(v)
                except ValueError:
                    raise ValueError("%s: bad entry %r" % (name, item))
            if rank in table:
                return max(0, table[rank])
        else:
            v = rank_value(env, name, rank)
            if v is not None:
                return max(0, int(v))
    return max(0, int(configured))


@dataclass(frozen=True)
class BlockConfig:
    # placement stages
    scp_apply_prefill: bool = True
    scp_apply_decode: bool = False
    scp_transient_prefill_cache: bool = True
    # prefetch planner
    rs_prefetch_policy: str = "default"
    pred_topk: int = 4
    top_m: int = 1
    min_cand_score: float = 0.02
    replace_advantage: float = 0.02
    replace_margin: float = 1.05
    allow_active_replace: bool = True
    cache_safe_min_score: float = 0.03
    cache_safe_replace_advantage: float = 0.05
    cache_safe_replace_margin: float = 1.10
    recent_protect_steps: int = 0
    rs_prefetch_prefill: bool = False
    # EPIPE
    epipe_enable: bool = False
    epipe_decode_only: bool = True
    epipe_prefill_enable: bool = False
    epipe_mode: str = "upfront_scan"
    epipe_decode_rs_mode: str = "off"
    epipe_handle_late_prefetch: bool = False
    epipe_handle_demand_miss: bool = False
    epipe_force_demand_stage: bool = False
    epipe_max_staged: int = 1
    epipe_no_evict: bool = True
    epipe_transient_staging: bool = True
    epipe_rolling_gate: bool = False
    epipe_gate_window: int = 16
    epipe_gate_min_triggers: int = 1
    epipe_gate_skip_steps: int = 8
    epipe_demand_commit: bool = False
    # executor
    plain_exec_mode: str = "unique_mask"
    prefill_expert_math: str = "native"
    # timing toggles (event based, never a sync on the timed path)
    expert_timing: bool = False
    demand_h2d_timing: bool = False
    prefetch_h2d_timing: bool = False

    def effective_planner_thresholds(self) -> Tuple[float, float, float]:
        """(min score, replace advantage, replace margin) after the policy's floors
        (utils/eval_core.py:10162-10183)."""
        lo, adv, mar = self.min_cand_score, self.replace_advantage, self.replace_margin
        if self.rs_prefetch_policy in ("cache_safe", "cache-safe", "benefit_gate", "benefit-gate"):
            lo = max(lo, self.cache_safe_min_score)
            adv = max(adv, self.cache_safe_replace_advantage)
            mar = max(mar, self.cache_safe_replace_margin)
        return lo, adv, mar


def block_config_from_env(env: Optional[Mapping[str, str]] = None, rank: int = 0,
                          prefetch_top_m: int = 1) -> BlockConfig:
    env = os.environ if env is None else env
    math = str(env.get("SPARSE_PREFILL_EXPERT_MATH", "native") or "native").strip().lower()
    if math not in ("native", ""):
        raise NotImplementedError(
            "SPARSE_PREFILL_EXPERT_MATH=%s: only the native bf16 expert math exists on this path "
            "(the fixed-tile FP16 Triton variant of the reference is not built)" % math)
    exec_mode = str(env.get("SPARSE_PLAIN_EP_EXEC_MODE", "unique_mask") or "unique_mask").strip().lower()
    if exec_mode not in ("unique_mask", "sorted_segment"):
        raise ValueError("SPARSE_PLAIN_EP_EXEC_MODE must be unique_mask or sorted_segment, got %r" % exec_mode)
    epipe = env_flag(env, "SPARSE_EPIPE_ENABLE")
    rs_mode = str(env.get("SPARSE_EPIPE_DECODE_RS_MODE", env.get("SPARSE_EPIPE_DECODE_WITH_RS_MODE", "off"))
                  or "off").strip().lower()
    max_staged = env_int(env, "SPARSE_EPIPE_MAX_STAGED_EXPERTS", 1)
    if epipe and max_staged != 1:
        raise NotImplementedError("SPARSE_EPIPE_MAX_STAGED_EXPERTS must be 1 (utils/eval_core.py:5024-5027)")
    return BlockConfig(
        scp_apply_prefill=env_flag(env, "SPARSE_SCP_APPLY_PREFILL", "1"),
        scp_apply_decode=env_flag(env, "SPARSE_SCP_APPLY_DECODE", "0"),
        scp_transient_prefill_cache=env_flag(env, "SPARSE_SCP_TRANSIENT_PREFILL_CACHE", "1"),
        rs_prefetch_policy=str(env.get("SPARSE_RS_PREFETCH_POLICY", "default") or "default").strip().lower(),
        pred_topk=rank_int(env, "SPARSE_RS_PREFETCH_PRED_TOPK_BY_RANK", rank,
                           env_int(env, "SPARSE_RS_PREFETCH_PRED_TOPK", 4)),
        top_m=rank_int(env, "SPARSE_RS_PREFETCH_TOP_M_BY_RANK", rank, prefetch_top_m),
        min_cand_score=env_float(env, "SPARSE_PREFETCH_MIN_CAND_SCORE", 0.02),
        replace_advantage=env_float(env, "SPARSE_PREFETCH_REPLACE_ADVANTAGE", 0.02),
        replace_margin=env_float(env, "SPARSE_PREFETCH_REPLACE_MARGIN", 1.05),
        allow_active_replace=env_flag(env, "SPARSE_PREFETCH_ALLOW_ACTIVE_REPLACE", "1"),
        cache_safe_min_score=rank_float(env, "SPARSE_RS_CACHE_SAFE_MIN_SCORE_BY_RANK", rank,
                                        env_float(env, "SPARSE_RS_CACHE_SAFE_MIN_SCORE", 0.03)),
        cache_safe_replace_advantage=rank_float(env, "SPARSE_RS_CACHE_SAFE_REPLACE_ADVANTAGE_BY_RANK", rank,
                                                env_float(env, "SPARSE_RS_CACHE_SAFE_REPLACE_ADVANTAGE", 0.05)),
        cache_safe_replace_margin=rank_float(env, "SPARSE_RS_CACHE_SAFE_REPLACE_MARGIN_BY_RANK", rank,
                                             env_float(env, "SPARSE_RS_CACHE_SAFE_REPLACE_MARGIN", 1.10)),
        recent_protect_steps=rank_int(env, "SPARSE_RS_PREFETCH_RECENT_PROTECT_STEPS_BY_RANK", rank,
                                      env_int(env, "SPARSE_RS_PREFETCH_RECENT_PROTECT_STEPS", 0)),
        rs_prefetch_prefill=env_flag(env, "SPARSE_RS_PREFETCH_PREFILL", "0"),
        epipe_enable=epipe,
        epipe_decode_only=env_flag(env, "SPARSE_EPIPE_DECODE_ONLY", "1"),
        epipe_prefill_enable=env_flag(env, "SPARSE_EPIPE_PREFILL_ENABLE", "0"),
        epipe_mode=str(env.get("SPARSE_EPIPE_MODE", "upfront_scan") or "upfront_scan").strip().lower(),
        epipe_decode_rs_mode=rs_mode,
        epipe_handle_late_prefetch=env_flag(env, "SPARSE_EPIPE_RS_HANDLE_LATE_PREFETCH", "0"),
        epipe_handle_demand_miss=env_flag(env, "SPARSE_EPIPE_RS_HANDLE_DEMAND_MISS", "0"),
        epipe_force_demand_stage=env_flag(env, "SPARSE_EPIPE_RS_FORCE_DEMAND_STAGE", "0"),
        epipe_max_staged=max_staged,
        epipe_no_evict=env_flag(env, "SPARSE_EPIPE_NO_EVICT", "1"),
        epipe_transient_staging=env_flag(env, "SPARSE_EPIPE_TRANSIENT_STAGING", "1"),
        epipe_rolling_gate=env_flag(env, "SPARSE_EPIPE_RS_ROLLING_GATE", "0"),
        epipe_gate_window=env_int(env, "SPARSE_EPIPE_RS_GATE_WINDOW", 16),
        epipe_gate_min_triggers=env_int(env, "SPARSE_EPIPE_RS_GATE_MIN_TRIGGERS", 1),
        epipe_gate_skip_steps=env_int(env, "SPARSE_EPIPE_RS_GATE_SKIP_STEPS", 8),
        epipe_demand_commit=env_flag(env, "SPARSE_EPIPE_RS_DEMAND_COMMIT", "0"),
        plain_exec_mode=exec_mode,
        prefill_expert_math="native",
        expert_timing=env_flag(env, "SPARSE_EXPERT_TIMING"),
        demand_h2d_timing=env_flag(env, "SPARSE_DEMAND_H2D_TIMING"),
        prefetch_h2d_timing=env_flag(env, "SPARSE_PREFETCH_H2D_TIMING"),
    )


METHODS = ("rr", "scp", "rs", "epipe", "scp-rs", "rs-epipe", "sparse", "executor-no-epipe",
           "executor-with-epipe")


def method_settings(method: str, ep_size: int = 4, prefetch_top_m: int = 2, pred_topk: int = 4
                    ) -> Tuple[Dict[str, str], Dict[str, str]]:
    """(CLI flags, environment) the launcher derives from a method name
    (scripts/run/run_case.sh:85-138 and the env block at 220-281)."""
    if method not in METHODS:
        raise ValueError("unknown method: %s" % method)
    scp = method in ("scp", "scp-rs", "sparse", "executor-no-epipe", "executor-with-epipe")
    rs = method in ("rs", "scp-rs", "rs-epipe", "sparse", "executor-no-epipe", "executor-with-epipe")
    epipe = method in ("epipe", "rs-epipe", "sparse", "executor-with-epipe")
    rs_mode = "residual_scan" if method in ("rs-epipe", "sparse", "executor-with-epipe") else "off"
    sorted_exec = method in ("epipe", "rs-epipe", "sparse", "executor-no-epipe", "executor-with-epipe")
    per_rank = lambda v: ",".join([str(v)] * ep_size)
    flags = {
        "--placement-mode": "scp_ep" if scp else "round_robin",
        "--planner-mode": "rs_prefetch" if rs else "none",
        "--routing-mode": "router", "--expert-source": "router", "--expert-offload": "cpu",
        "--cache-policy": "lru", "--prefetch-top-m": str(prefetch_top_m),
    }
    env = {
        "SPARSE_SCP_APPLY_PREFILL": "1" if scp else "0",
        "SPARSE_SCP_APPLY_DECODE": "0",
        "SPARSE_SCP_TRANSIENT_PREFILL_CACHE": "1",
        "SPARSE_RS_PREFETCH_POLICY": "cache_safe",
        "SPARSE_RS_PREFETCH_PRED_TOPK": str(pred_topk),
        "SPARSE_RS_PREFETCH_TOP_M_BY_RANK": per_rank(prefetch_top_m),
        "SPARSE_RS_PREFETCH_PRED_TOPK_BY_RANK": per_rank(pred_topk),
        "SPARSE_RS_CACHE_SAFE_MIN_SCORE_BY_RANK": per_rank("0.04"),
        "SPARSE_RS_CACHE_SAFE_REPLACE_ADVANTAGE_BY_RANK": per_rank("0.08"),
        "SPARSE_RS_CACHE_SAFE_REPLACE_MARGIN_BY_RANK": per_rank("1.20"),
        "SPARSE_RS_PREFETCH_RECENT_PROTECT_STEPS_BY_RANK": per_rank(1),
        "SPARSE_PREFETCH_MIN_CAND_SCORE": "0.04",
        "SPARSE_PREFETCH_REPLACE_ADVANTAGE": "0.08",
        "SPARSE_PREFETCH_REPLACE_MARGIN": "1.20",
        "SPARSE_PREFETCH_ALLOW_ACTIVE_REPLACE": "1" if rs else "0",
        "SPARSE_EPIPE_ENABLE": "1" if epipe else "0",
        "SPARSE_EPIPE_DECODE_ONLY": "1",
        "SPARSE_EPIPE_PREFILL_ENABLE": "0",
        "SPARSE_EPIPE_MODE": "upfront_scan",
        "SPARSE_EPIPE_DECODE_RS_MODE": rs_mode,
        "SPARSE_EPIPE_RS_HANDLE_LATE_PREFETCH": "1" if epipe else "0",
        "SPARSE_EPIPE_RS_HANDLE_DEMAND_MISS": "1" if epipe else "0",
        "SPARSE_EPIPE_RS_FORCE_DEMAND_STAGE": "1" if epipe else "0",
        "SPARSE_EPIPE_NO_EVICT": "1",
        "SPARSE_EPIPE_TRANSIENT_STAGING": "1",
        "SPARSE_EPIPE_MAX_STAGED_EXPERTS": "1",
        "SPARSE_PLAIN_EP_EXEC_MODE": "sorted_segment" if sorted_exec else "unique_mask",
        "SPARSE_EP_FUSED_WEIGHT_DISPATCH": "0",
        "SPARSE_RESET_RUNTIME_STATE_EACH_REPEAT": "1",
        "SPARSE_CLEAR_EXPERT_CACHE_EACH_REPEAT": "1",
    }
    return flags, env
