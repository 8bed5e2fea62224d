"""`utils.eval_core` of the reference under its own symbol names.

What `scripts/perf.py` imports (scripts/perf.py:24-40 of the reference):
CoreBuildConfig, DistEnv, Metrics, RunningStats, SparseContext,
all_reduce_max_, all_reduce_sum_, barrier, build_model_and_tokenizer,
destroy_dist, greedy_decode_profiled, init_dist,
print_routing_stats_if_enabled, set_sdpa_mode, wall_timer_s; plus the block
itself and its cache for callers such as scripts/benchmark_lightweight.py.

`build_model_and_tokenizer` builds randomly initialised models of the benchmark
shapes ("synthetic:qwen", "synthetic:deepseek", "synthetic:tiny" as
`model_path`): no checkpoints or tokenizers are available offline, and loading
them is the framework's job, not the MoE path's.
"""
from __future__ import annotations

import os
import time
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Any, Optional, Tuple

import torch
import torch.distributed as dist

from sparse_b200.cache import ExpertWeightCache  # noqa: F401
from sparse_b200.context import Metrics, SparseContext  # noqa: F401
from sparse_b200.model import (DEEPSEEK_MODEL, QWEN_MODEL, TINY_MODEL, RunningStats,  # noqa: F401
                               ShapedMoeModel, greedy_decode_profiled)
from sparse_b200.moe_block import DistributedSparseMoeBlock  # noqa: F401


@dataclass(frozen=True)
class CoreBuildConfig:
    """Same fields and defaults as utils/eval_core.py:17687-17725."""
    model_path: str
    scp_path: str
    rs_dir: str
    dtype: str = "float16"
    expert_offload: str = "cpu"
    expert_cache: int = 0
    cache_policy: str = "lru"
    enable_skvs: bool = False
    skvs_sink: int = 4
    skvs_window: int = 32
    skvs_ratio: float = 0.6
    skvs_min_kv_len: int = 0
    skvs_min_sparse_drop_ratio: float = 0.0
    skvs_guidance_every_k: int = 1
    skvs_guidance_start_kv_len: int = 0
    skvs_allow_prefill_sparse: bool = False
    prompt_len: int = 0
    max_new_tokens: int = 0
    routing_mode: str = "router"
    expert_source: str = "router"
    placement_mode: str = "scp"
    scp_ep_path: str = ""
    runtime_mode: str = "baseline"
    rs_require_complete: bool = True
    rs_prob_to_logit_eps: float = 1e-9
    log_routing_stats: bool = False
    lm_head_device: str = "cuda"
    rs_group: int = 3
    rs_debug: bool = False
    debug_a2a_checks: bool = False
    collect_per_layer: bool = False
    log_per_layer: bool = False
    planner_mode: str = "none"
    prefetch_top_m: int = 1
    oracle_mode: str = "none"
    oracle_trace_dir: str = ""
    oracle_ignore_cache_capacity: bool = True
    ep_size: int = 0
    batch: int = 0                      # addition: sequences per rank the model is sized for (0 = 1)


@dataclass
class DistEnv:
    rank: int
    world: int
    local_rank: int
    device: torch.device


@dataclass(frozen=True)
class DistTopology:
    runtime_mode: str
    ep_size: int
    dp_size: int
    ep_rank: int
    dp_rank: int
    ep_group: Any
    ep_global_ranks: Tuple[int, ...]

    @property
    def is_ep_leader(self) -> bool:
        return self.ep_rank == 0


@dataclass
class ModelBundle:
    model: Any
    tokenizer: Any
    hf_config: Any
    routing_mode: str = "router"
    num_experts: int = 0
    top_k: int = 0


def init_dist(backend: str = "nccl") -> DistEnv:
    """One rank per GPU from the torchrun environment (utils/eval_core.py:224-270)."""
    if "LOCAL_RANK" not in os.environ:
        raise RuntimeError("LOCAL_RANK not found. Please launch with torchrun.")
    local_rank = int(os.environ["LOCAL_RANK"])
    if backend == "nccl":
        if torch.cuda.device_count() <= 0:
            raise RuntimeError("No CUDA device visible.")
        device = torch.device("cuda", local_rank)
        torch.cuda.set_device(device)
        dist.init_process_group(backend="nccl", device_id=device)
    else:
        device = torch.device("cpu")
        dist.init_process_group(backend=backend)
    return DistEnv(rank=dist.get_rank(), world=dist.get_world_size(), local_rank=local_rank, device=device)


def build_dist_topology(env: DistEnv, runtime_mode: str, ep_size: int) -> DistTopology:
    """EP groups of `ep_size` consecutive ranks, DP replicas of them (utils/eval_core.py:188-222)."""
    if runtime_mode not in ("baseline", "canonical_ep_dp_serving_baseline"):
        raise ValueError("This codebase now keeps only one runtime path: baseline. "
                         f"Unsupported runtime_mode={runtime_mode}")
    ep_size = int(ep_size)
    if ep_size <= 0 or env.world % ep_size != 0:
        raise ValueError(f"baseline requires world % ep_size == 0, got world={env.world}, ep_size={ep_size}")
    dp_size, dp_rank, ep_rank = env.world // ep_size, env.rank // ep_size, env.rank % ep_size
    mine, mine_ranks = None, None
    for dp in range(dp_size):
        ranks = tuple(range(dp * ep_size, (dp + 1) * ep_size))
        g = dist.new_group(ranks=list(ranks))
        if dp == dp_rank:
            mine, mine_ranks = g, ranks
    return DistTopology("baseline", ep_size, dp_size, ep_rank, dp_rank, mine, mine_ranks)


def barrier(env: DistEnv) -> None:
    if env.device.type == "cuda":
        dist.barrier(device_ids=[env.local_rank])
    else:
        dist.barrier()


def destroy_dist() -> None:
    try:
        dist.destroy_process_group()
    except Exception:
        pass


def all_reduce_sum_(x: torch.Tensor) -> torch.Tensor:
    dist.all_reduce(x, op=dist.ReduceOp.SUM)
    return x


def all_reduce_max_(x: torch.Tensor) -> torch.Tensor:
    dist.all_reduce(x, op=dist.ReduceOp.MAX)
    return x


def set_sdpa_mode(flash: bool, mem_efficient: bool, math_sdp: bool) -> None:
    try:
        torch.backends.cuda.enable_flash_sdp(bool(flash))
        torch.backends.cuda.enable_mem_efficient_sdp(bool(mem_efficient))
        torch.backends.cuda.enable_math_sdp(bool(math_sdp))
    except Exception:
        pass


@contextmanager
def wall_timer_s():
    t0 = time.perf_counter()
    yield lambda: (time.perf_counter() - t0)


_SYNTHETIC = {"qwen": QWEN_MODEL, "deepseek": DEEPSEEK_MODEL, "tiny": TINY_MODEL}


class _IdsTokenizer:
    """Stand-in tokenizer of a synthetic model: prompts are token ids already."""
    pad_token_id = 0
    eos_token_id = None

    def __init__(self, vocab: int):
        self.vocab_size = vocab


def build_model_and_tokenizer(cfg: CoreBuildConfig, env: DistEnv, metrics: Optional[Metrics] = None) -> ModelBundle:
    """`synthetic:<shape>` model paths build a randomly initialised model of that
    shape on `env.device`, sized for `cfg.prompt_len + cfg.max_new_tokens`
    positions; experts are sharded over the EP group by round-robin ownership."""
    if cfg.enable_skvs:
        raise NotImplementedError("SKVS attention is not part of the B200 MoE-layer path")
    if cfg.oracle_mode != "none" or cfg.routing_mode != "router" or cfg.expert_source != "router":
        raise NotImplementedError("only routing_mode=router, expert_source=router, oracle_mode=none are built")
    if cfg.dtype != "bfloat16":
        raise NotImplementedError("the B200 MoE path computes in bfloat16; pass --dtype bfloat16")
    if not cfg.model_path.startswith("synthetic:") or cfg.model_path.split(":", 1)[1] not in _SYNTHETIC:
        raise NotImplementedError(
            "model_path=%r: checkpoints are loaded by the serving framework; this package builds "
            "synthetic:qwen, synthetic:deepseek and synthetic:tiny" % cfg.model_path)
    if cfg.placement_mode not in ("round_robin",):
        raise NotImplementedError("the synthetic model harness shards experts round-robin; placement files apply "
                                  "to DistributedSparseMoeBlock")
    shape = _SYNTHETIC[cfg.model_path.split(":", 1)[1]]
    ep = int(cfg.ep_size) if cfg.ep_size else env.world
    if ep != env.world:
        raise NotImplementedError("data-parallel replicas of an EP group (world > ep_size) are independent "
                                  "processes here: launch one job per replica")
    group = dist.group.WORLD if env.world > 1 else None
    SparseContext.initialize(shape.layers, num_experts=shape.moe.num_experts)
    model = ShapedMoeModel(shape, env.device, max(1, cfg.batch), cfg.prompt_len + cfg.max_new_tokens + 1, seed=0,
                           ep_rank=env.rank, ep_size=ep, process_group=group)
    return ModelBundle(model=model, tokenizer=_IdsTokenizer(shape.vocab), hf_config=shape,
                       routing_mode=cfg.routing_mode, num_experts=shape.moe.num_experts, top_k=shape.moe.top_k)


def print_routing_stats_if_enabled(env: DistEnv, bundle: ModelBundle, tag: str = "") -> None:
    """Coverage of the last step's routing per layer, on rank 0 (utils/eval_core.py:3377-3400)."""
    if env.rank != 0 or bundle is None or not hasattr(bundle.model, "layers"):
        return
    print(f"[RoutingStats]{'[' + tag + ']' if tag else ''} mode={bundle.routing_mode} "
          f"E={bundle.num_experts} K={bundle.top_k}", flush=True)
    for l, ly in enumerate(bundle.model.layers):
        if ly.block is None:
            continue
        idx, _ = ly.block.topk(bundle.model.batch)
        uniq = int(torch.unique(idx).numel())
        print(f"L{l}: cov={uniq / max(1, bundle.num_experts):.3f} uniq={uniq}", flush=True)
