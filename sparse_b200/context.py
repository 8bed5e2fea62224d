"""Process-wide serving state and counters.

`SparseContext` is the small subset of the reference's class-level registry
that the MoE hot path and its callers use (utils/eval_core.py:2349-2363,
2391-2401, 2445-2484, 2768-2770, 3063-3097): current phase, runtime call id,
layer registry, the RS predictor bank, and the per-request reset.
`Metrics` keeps the counters the launcher's summary needs
(utils/eval_core.py:1689-2009; keys in scripts/perf.py:2422-2460).
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional


class SparseContext:
    num_layers: int = 0
    num_experts: int = 0
    rs_group: int = 3
    current_phase: str = ""          # "prefill" | "decode" | ""
    runtime_call_id: int = -1
    current_moe_layer_idx: int = -1
    layer_blocks: Dict[int, Any] = {}
    rs_bank: Any = None
    rs_bank_task: str = "router_prob"
    rs_bank_layout: str = "group"
    rs_bank_source_layers: List[int] = []

    @classmethod
    def initialize(cls, num_layers: int, rs_group: int = 3, num_experts: int = 0) -> None:
        cls.num_layers, cls.num_experts, cls.rs_group = int(num_layers), int(num_experts), int(rs_group)
        cls.layer_blocks = {}
        cls.rs_bank = None
        cls.rs_bank_task, cls.rs_bank_layout, cls.rs_bank_source_layers = "router_prob", "group", []
        cls.current_phase, cls.runtime_call_id, cls.current_moe_layer_idx = "", -1, -1

    @classmethod
    def register_layer_block(cls, layer_idx: int, block: Any) -> None:
        cls.layer_blocks[int(layer_idx)] = block

    @classmethod
    def begin_runtime_call(cls, call_id: int) -> None:
        cls.runtime_call_id = int(call_id)

    @classmethod
    def stage(cls, seq_len: int) -> str:
        """prefill/decode: the declared phase, else one token per sequence means
        decode (utils/eval_core.py:6149-6158)."""
        if cls.current_phase in ("prefill", "decode"):
            return cls.current_phase
        return "decode" if int(seq_len) == 1 else "prefill"

    @classmethod
    def reset_runtime_state_for_new_request(cls, clear_caches: bool = False) -> None:
        cls.current_phase, cls.runtime_call_id, cls.current_moe_layer_idx = "", -1, -1
        for blk in cls.layer_blocks.values():
            fn = getattr(blk, "reset_runtime_state_for_new_request", None)
            if callable(fn):
                fn(clear_cache=clear_caches)


@dataclass
class Metrics:
    expert_weight_h2d_bytes: int = 0
    expert_weight_h2d_demand_bytes: int = 0
    expert_weight_h2d_prefetch_bytes: int = 0
    expert_weight_peer_bytes: int = 0              # weights copied from an owner GPU's slab over NVLink
    expert_weight_peer_demand_bytes: int = 0
    expert_weight_peer_prefetch_bytes: int = 0
    local_cached_item_count: int = 0               # items of non-owned experts executed out of a local cache slot
    owner_fallback_item_count: int = 0             # items sent to the owner because the weights were not (yet) here
    load_exposed_ms: float = 0.0                   # compute-stream time spent waiting for weight copies
    cache_hit_count: int = 0
    cache_miss_count: int = 0
    prefetch_issued_count: int = 0
    prefetch_admitted_count: int = 0
    prefetch_completed_count: int = 0
    prefetch_wasted_count: int = 0
    prefetch_complete_before_use_count: int = 0
    prefetch_late_count: int = 0
    demand_h2d_exposed_ms: float = 0.0
    demand_h2d_exposed_prefill_ms: float = 0.0
    demand_h2d_exposed_decode_ms: float = 0.0
    comm_bytes_activation: int = 0
    comm_bytes_activation_remote: int = 0
    epipe_attempt_count: int = 0
    epipe_trigger_count: int = 0
    epipe_staged_expert_count: int = 0
    epipe_ready_group_count: int = 0
    epipe_fallback_count: int = 0
    wall_prefill_ms: float = 0.0                   # greedy_decode_profiled's wall clocks (utils/eval_core.py:18511, 18590)
    wall_decode_ms: float = 0.0
    wall_ttft_ms: float = 0.0
    warmup_time_ms: float = 0.0
    peak_allocated_mb: float = 0.0
    peak_reserved_mb: float = 0.0
    moe_router_ms: float = 0.0
    moe_expert_ms: float = 0.0
    moe_shared_ms: float = 0.0
    rs_counters: Dict[str, int] = field(default_factory=dict)
    pending_events: List[Any] = field(default_factory=list)   # (kind, phase, start_event, end_event)
    decode_step_stats: Any = None                  # a RunningStats when per-step latencies are wanted

    def reset_for_repeat(self) -> None:
        fresh = Metrics()
        for f in fields(self):
            setattr(self, f.name, getattr(fresh, f.name))

    def count_rs(self, name: str, value: int = 1) -> None:
        self.rs_counters[name] = self.rs_counters.get(name, 0) + int(value)

    def finalize_events(self) -> None:
        """Turn finished (start, end) event pairs into milliseconds.  Called after a
        forward, never on the timed path (utils/eval_core.py:18231-18421)."""
        keep = []
        for kind, phase, start, end in self.pending_events:
            if not end.query():
                keep.append((kind, phase, start, end))
                continue
            ms = float(start.elapsed_time(end))
            if kind == "load_exposed":
                self.load_exposed_ms += ms
            if kind == "demand_h2d":
                self.demand_h2d_exposed_ms += ms
                if phase == "prefill":
                    self.demand_h2d_exposed_prefill_ms += ms
                else:
                    self.demand_h2d_exposed_decode_ms += ms
        self.pending_events = keep

    def summary(self) -> Dict[str, Any]:
        out = {f.name: getattr(self, f.name) for f in fields(self)
               if f.name not in ("rs_counters", "pending_events", "decode_step_stats")}
        if self.decode_step_stats is not None:
            out.update(self.decode_step_stats.summary("decode_step_"))
        out.update({"rs_" + k if not k.startswith(("rs_", "prefetch_")) else k: v for k, v in self.rs_counters.items()})
        return out
