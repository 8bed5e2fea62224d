"""`DistributedSparseMoeBlock`: the reference's plugin class, B200 edition.

Same constructor keywords and the same forward contract as the reference's
block (utils/eval_core.py:4408-4440 constructor, 16418-16563 forward), so
`layer.mlp = DistributedSparseMoeBlock(layer_idx=i, mlp_block=layer.mlp, ...)`
(utils/eval_core.py:17959-17990) keeps working.  The inner block is duck-typed
exactly as there (4342-4362): `.gate`, `.experts` (ModuleList of
gate_proj/up_proj/down_proj or fused gate_up_proj/down_proj), `.shared_expert`
+ `.shared_expert_gate` (Qwen) or `.shared_experts` (DeepSeek).

What happens inside is different: weights are packed once into device slabs,
the layer pass is a handful of CUDA kernels behind the C ABI, expert
parallelism moves rows over NVLink peer memory, and offloaded experts live in
preallocated cache slots filled by side-stream copies.  Compute dtype is bf16.
"""
from __future__ import annotations

import os
from typing import Any, Dict, List, Optional, Sequence

import torch
import torch.nn as nn

from .cache import ExpertWeightCache
from .config import BlockConfig, block_config_from_env, cache_capacity_for_rank
from .context import Metrics, SparseContext
from .layer import LayerRunner, LayerWeights
from .placement import Placement
from .rs import build_prefetch_plan, load_rs_bank, prob_score_map
from .store import CachedLayerRunner, ExpertStore, HostExperts


def looks_like_sparse_moe_block(mlp: nn.Module) -> bool:
    if not all(hasattr(mlp, a) for a in ("gate", "experts")):
        return False
    return (all(hasattr(mlp, a) for a in ("shared_expert", "shared_expert_gate"))
            or hasattr(mlp, "shared_experts"))


def _expert_matrices(experts, e: int):
    """(gate [I,H], up [I,H], down [H,I]) of expert e from either weight layout:
    a ModuleList of gate_proj/up_proj/down_proj modules, or fused 3-D parameters
    gate_up_proj [E,2I,H] (the I gate rows first) and down_proj [E,H,I], which is
    how the reference applies them (F.linear(x, gate_up_proj[e]) then chunk(2),
    utils/eval_core.py:11714-11724)."""
    if all(hasattr(experts, a) for a in ("gate_up_proj", "down_proj")):
        gu = experts.gate_up_proj[e]
        dn = experts.down_proj[e]
        if gu.dim() != 2 or dn.dim() != 2 or gu.shape[0] % 2 != 0 or \
                gu.shape[1] != dn.shape[0] or dn.shape[1] * 2 != gu.shape[0]:
            raise ValueError("fused expert weights must be gate_up_proj [E,2I,H] and down_proj [E,H,I]; got %s and %s"
                             % (tuple(experts.gate_up_proj.shape), tuple(experts.down_proj.shape)))
        i = gu.shape[0] // 2
        return gu[:i], gu[i:], dn
    m = list(experts)[e]
    return m.gate_proj.weight, m.up_proj.weight, m.down_proj.weight


class DistributedSparseMoeBlock(nn.Module):
    def __init__(self, layer_idx: int, mlp_block: nn.Module, scp_map: Dict[str, int], env, num_layers: int,
                 num_experts: int, top_k: int, dtype: torch.dtype, expert_offload: str, expert_cache: int,
                 routing_mode: str, rs_dir: str, rs_require_complete: bool, rs_prob_to_logit_eps: float,
                 log_routing_stats: bool, rs_group: int = 3, rs_debug: bool = False,
                 metrics: Optional[Metrics] = None, debug_a2a_checks: bool = False,
                 collect_per_layer: bool = False, log_per_layer: bool = False, planner_mode: str = "none",
                 prefetch_top_m: int = 1, oracle_mode: str = "none", oracle_ignore_cache_capacity: bool = True,
                 placement_mode: str = "scp", expert_source: str = "router", cache_policy: str = "lru",
                 runtime_mode: str = "baseline", topology=None, scp_ep_placement: Optional[dict] = None,
                 max_tokens: int = 4096, process_group=None):
        super().__init__()
        if not looks_like_sparse_moe_block(mlp_block):
            raise ValueError("mlp_block does not look like a sparse MoE block (needs gate, experts, shared expert)")
        if dtype != torch.bfloat16:
            raise NotImplementedError("the B200 MoE path computes in bfloat16; got %s" % dtype)
        if expert_offload not in ("cpu", "gpu"):
            raise ValueError("expert_offload must be cpu or gpu")
        if planner_mode not in ("none", "rs_prefetch"):
            raise ValueError("planner_mode must be none or rs_prefetch")
        if cache_policy != "lru":
            raise NotImplementedError("only cache_policy=lru is built (the launchers use nothing else)")
        if routing_mode != "router" or expert_source != "router" or oracle_mode != "none":
            raise NotImplementedError("only routing_mode=router, expert_source=router, oracle_mode=none are built")
        if runtime_mode not in ("baseline", "canonical_ep_dp_serving_baseline"):
            raise ValueError("This codebase keeps only one runtime path: baseline")
        self.layer_idx, self.num_layers, self.num_experts, self.top_k = int(layer_idx), int(num_layers), int(num_experts), int(top_k)
        self.env, self.device = env, env.device
        self.rank, self.world = int(env.rank), int(env.world)
        self.comm_rank = int(getattr(topology, "ep_rank", self.rank)) if topology is not None else self.rank
        self.comm_world = int(getattr(topology, "ep_size", self.world)) if topology is not None else self.world
        self.metrics = metrics
        self.planner_mode, self.expert_offload, self.placement_mode = planner_mode, expert_offload, placement_mode
        self.rs_group = int(rs_group)
        self.cfg: BlockConfig = block_config_from_env(os.environ, rank=self.comm_rank, prefetch_top_m=prefetch_top_m)
        self.moe_family = "qwen_shared" if hasattr(mlp_block, "shared_expert") else "deepseek_shared"
        self.norm_topk_prob = bool(getattr(mlp_block, "norm_topk_prob", False))
        self.scp_apply_decode = self.cfg.scp_apply_decode

        gate_w = mlp_block.gate.weight
        self.hidden_size = int(gate_w.shape[1])
        g0, _, _ = _expert_matrices(mlp_block.experts, 0)
        inter = int(g0.shape[0])
        shared = getattr(mlp_block, "shared_expert", None) or getattr(mlp_block, "shared_experts", None)
        shared_inter = int(shared.gate_proj.weight.shape[0]) if shared is not None else 0

        # placement: which experts may this rank execute, in either stage
        obj = scp_ep_placement if placement_mode == "scp_ep" else (scp_map if placement_mode == "scp" else None)
        self.placement = Placement(placement_mode, num_layers, num_experts, max(1, self.comm_world), obj=obj,
                                   apply_prefill=self.cfg.scp_apply_prefill, apply_decode=self.cfg.scp_apply_decode)
        if self.comm_world > 1:
            local = sorted(self.placement.receive_experts(self.layer_idx, self.comm_rank))
        else:
            local = list(range(num_experts))
        self.local_expert_ids: List[int] = local
        self._local_eid_set = set(local)

        capacity = cache_capacity_for_rank(os.environ, int(expert_cache), self.comm_rank)
        offloaded = expert_offload == "cpu" and capacity < len(local)
        # one staging slot for EPIPE's transient copy, plus a pool for the bounded stager if asked for
        staging = 1 + max(0, int(os.environ.get("SPARSE_B200_RS_STAGING_SLOTS", "0") or 0))
        n_slots = (capacity + staging) if offloaded else len(local)
        lw = LayerWeights(self.hidden_size, inter, num_experts, max(1, n_slots), shared_inter, self.device)
        lw.set_router(gate_w.detach(), getattr(mlp_block.gate, "bias", None))
        if shared is not None:
            sg = getattr(mlp_block, "shared_expert_gate", None)
            lw.set_shared(shared.gate_proj.weight.detach(), shared.up_proj.weight.detach(),
                          shared.down_proj.weight.detach(), sg.weight.detach() if sg is not None else None)
        self.weights = lw
        self.store: Optional[ExpertStore] = None
        self._runner: Optional[LayerRunner] = None
        self._cached: Optional[CachedLayerRunner] = None
        self._ep = None
        fp32_logits = self.moe_family == "deepseek_shared"
        if offloaded:
            host = HostExperts(self.hidden_size, inter)
            for e in local:
                g, u, d = _expert_matrices(mlp_block.experts, e)
                host.add(e, g.detach(), u.detach(), d.detach())
            self.store = ExpertStore(lw, host, capacity, staging_slots=staging, cfg=self.cfg, metrics=metrics,
                                     layer_idx=self.layer_idx)
            self.store.push_slot_map()
            self._cached = CachedLayerRunner(self.store, top_k, renorm=self.norm_topk_prob, fp32_logits=fp32_logits)
            self._cache = self.store.cache
            if self.comm_world > 1:
                from .ep import CachedExpertParallelLayer
                self._ep = CachedExpertParallelLayer(self._cached, top_k, max_tokens, self.comm_rank,
                                                     self.comm_world, process_group,
                                                     owner=self.placement.dest_table(self.layer_idx, "prefill"),
                                                     owner_decode=self.placement.dest_table(self.layer_idx, "decode"),
                                                     renorm=self.norm_topk_prob, fp32_logits=fp32_logits)
        else:
            slot_of = [-1] * num_experts
            for slot, e in enumerate(local):
                g, u, d = _expert_matrices(mlp_block.experts, e)
                lw.load_expert(slot, g.detach(), u.detach(), d.detach())
                slot_of[e] = slot
            lw.set_slot_map(slot_of)
            self._cache = ExpertWeightCache(0)
            if self.comm_world > 1:
                from .ep import ExpertParallelLayer
                self._ep = ExpertParallelLayer(lw, top_k, max_tokens, self.comm_rank, self.comm_world,
                                               process_group,
                                               owner=self.placement.dest_table(self.layer_idx, "prefill"),
                                               owner_decode=self.placement.dest_table(self.layer_idx, "decode"),
                                               renorm=self.norm_topk_prob, fp32_logits=fp32_logits)
            else:
                self._runner = LayerRunner(lw, top_k, max_tokens, renorm=self.norm_topk_prob,
                                           fp32_logits=fp32_logits)
        # RS predictor bank is shared by all layers (loaded once)
        if planner_mode == "rs_prefetch" and rs_dir and SparseContext.rs_bank is None:
            bank, task, layout, sources, _ = load_rs_bank(rs_dir, num_layers, self.hidden_size, num_experts,
                                                          self.device, rs_require_complete)
            SparseContext.rs_bank, SparseContext.rs_bank_task = bank, task
            SparseContext.rs_bank_layout, SparseContext.rs_bank_source_layers = layout, sources
        self._current_forward_batch_size, self._current_forward_seq_len = 1, 1

    # -- prefetch scheduling (decode only unless SPARSE_RS_PREFETCH_PREFILL=1) -------------
    def _effective_rs_prefetch_top_m(self) -> int:
        return int(self.cfg.top_m)

    def _rs_prefetch_predict_topk(self) -> int:
        return int(self.cfg.pred_topk)

    def _compute_and_schedule_next_layer_rs(self, x: torch.Tensor, seq_len: int) -> None:
        """Predict the next layer's experts from this layer's input and start
        copies for the ones worth having (utils/eval_core.py:10916-11010)."""
        if self.planner_mode != "rs_prefetch" or SparseContext.rs_bank is None:
            return
        if seq_len != 1 and not self.cfg.rs_prefetch_prefill:
            return
        target_layer = self.layer_idx + 1
        target = SparseContext.layer_blocks.get(target_layer)
        if target is None or getattr(target, "store", None) is None or target._effective_rs_prefetch_top_m() <= 0:
            return
        store: ExpertStore = target.store
        store.end_prefetch_group()
        with torch.inference_mode():
            probs = SparseContext.rs_bank[target_layer](x.float())
            k = min(self.num_experts, target._rs_prefetch_predict_topk())
            topv, topi = torch.topk(probs, k=k, dim=-1)
        note = (lambda n, v=1: self.metrics.count_rs(n, v)) if self.metrics is not None else None
        local = target._local_eid_set
        smap = prob_score_map(topi.cpu(), topv.cpu(), lambda e: e in local, note)
        lo, adv, mar = target.cfg.effective_planner_thresholds()
        plan = build_prefetch_plan(smap, store.cache, protect_ids=store.protect_ids(),
                                   budget=target._effective_rs_prefetch_top_m(), min_score=lo,
                                   replace_advantage=adv, replace_margin=mar,
                                   allow_active_replace=target.cfg.allow_active_replace,
                                   is_local=lambda e: e in local, keep_bias=store.keep_bias, counters=note)
        store.admit_prefetch_plan(plan)

    # -- forward ------------------------------------------------------------------
    def _return_tensor_only_mlp(self) -> bool:
        return self.moe_family == "deepseek_shared"

    def forward(self, hidden_states: torch.Tensor):
        b, s, h = hidden_states.shape
        x = hidden_states.reshape(-1, h).contiguous()
        self._current_forward_batch_size, self._current_forward_seq_len = int(b), int(s)
        SparseContext.current_moe_layer_idx = self.layer_idx
        stage = SparseContext.stage(s)
        self._compute_and_schedule_next_layer_rs(x, s)
        if self._ep is not None:
            out = self._ep.forward(x, stage=stage).clone()
            logits = self._ep.logits[:x.shape[0]]
        elif self._cached is not None:
            out, idx, wts, logits = self._cached.forward(x, stage)
        else:
            out, idx, wts, logits = self._runner.forward(x)
            out = out.clone()
        if self.metrics is not None:
            self.metrics.finalize_events()
        out = out.view(b, s, h)
        return out if self._return_tensor_only_mlp() else (out, logits)

    # -- methods callers use between requests ------------------------------------------
    def clear_all_expert_caches(self) -> None:
        if self.store is not None:
            self.store.clear()
            self.store.push_slot_map()

    def demote_prefill_scp_transients_for_decode(self) -> int:
        return self._cache.demote_prefill_scp_transients() if self.store is not None else 0

    def reset_runtime_state_for_new_request(self, clear_cache: bool = False) -> None:
        if self.store is not None:
            self.store.end_prefetch_group()
            self.store.cache.reset_request_metadata(unpin=True)
            self.store.last_used_decode_step.clear()
            if clear_cache:
                self.clear_all_expert_caches()

    def check_status(self) -> None:
        for r in (self._runner, self._ep):
            if r is not None:
                r.check_status()
        if self._cached is not None and int(self._cached.status.item()) != 0:
            code = int(self._cached.status.item())
            self._cached.status.zero_()
            raise RuntimeError("sparse_b200 device status %d" % code)
