#!/usr/bin/env python
"""The reference's `scripts/perf.py` launcher for the B200 build.

Accepts the reference's command line (scripts/perf.py:3655-3734 of the
reference) and writes the summary files its analysis scripts read
(`<run_tag>_summary.json`, a timestamped copy, `run_*_raw_repeats.json`,
`runs.jsonl`; scripts/perf.py:3402-3427) with the throughput keys
`scripts/analysis/summarize_results.py` consumes (`e2e_output_tok_s`,
`decode_throughput_tok_s` and their `_std`).  Launch one rank per GPU:

    torchrun --nproc-per-node 8 -m sparse_b200.compat.scripts.perf \
        --model-path synthetic:qwen --dataset synthetic --dtype bfloat16 \
        --batch 8 --prompt-len 2048 --max-new 128 --expert-offload gpu

No prompt dataset, tokenizer or checkpoint exists offline: `--dataset synthetic`
draws `--batch` prompts of `--prompt-len` uniform random token ids per repeat
(seeded), `--model-path synthetic:<qwen|deepseek|tiny>` builds a randomly
initialised model of that shape.  Each rank decodes its own `--batch`
sequences (data-parallel attention, expert-parallel MoE); token counts are
summed over all ranks, not taken from EP rank 0 as the reference does for its
replicated inputs.  Flags of subsystems outside the MoE path (SKVS, oracle
record/replay) parse and are refused when switched on.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time
from typing import Any, Dict, List

HERE = os.path.dirname(os.path.abspath(__file__))
COMPAT = os.path.dirname(HERE)
ROOT = os.path.dirname(os.path.dirname(COMPAT))
for p in (ROOT, COMPAT):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="B200 MoE serving benchmark with the reference's flag surface")
    ap.add_argument("--model-path", type=str, required=True)
    ap.add_argument("--scp-path", type=str, default="")
    ap.add_argument("--rs-dir", type=str, default="")
    ap.add_argument("--prompt", type=str, default="The quick brown fox jumps over the lazy dog. " * 16)
    ap.add_argument("--dataset", type=str, required=True)
    ap.add_argument("--use-dataset-prompts", action="store_true", default=True)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--max-new", type=int, default=64)
    ap.add_argument("--dtype", type=str, default="float16", choices=["float16", "bfloat16"])
    ap.add_argument("--routing-mode", type=str, default="router", choices=["rs", "router"])
    ap.add_argument("--rs-require-complete", dest="rs_require_complete", action="store_true")
    ap.add_argument("--no-rs-require-complete", dest="rs_require_complete", action="store_false")
    ap.set_defaults(rs_require_complete=True)
    ap.add_argument("--log-routing-stats", action="store_true")
    ap.add_argument("--enable-skvs", action="store_true")
    ap.add_argument("--skvs-sink", type=int, default=4)
    ap.add_argument("--skvs-window", type=int, default=16)
    ap.add_argument("--skvs-ratio", type=float, default=0.6)
    ap.add_argument("--skvs-min-kv-len", type=int, default=0)
    ap.add_argument("--skvs-min-sparse-drop-ratio", type=float, default=0.0)
    ap.add_argument("--skvs-guidance-every-k", type=int, default=24)
    ap.add_argument("--skvs-guidance-start-kv-len", type=int, default=0)
    ap.add_argument("--skvs-allow-prefill-sparse", action="store_true")
    ap.add_argument("--expert-offload", type=str, default="cpu", choices=["cpu", "gpu"])
    ap.add_argument("--expert-cache", type=int, default=10)
    ap.add_argument("--cache-policy", type=str, default="lru", choices=["lru", "lfu", "tiered"])
    ap.add_argument("--debug-a2a-checks", action="store_true")
    ap.add_argument("--log-per-layer", action="store_true")
    ap.add_argument("--collect-per-layer", action="store_true")
    ap.add_argument("--measure-ttft", action="store_true")
    ap.add_argument("--save-output-tokens", action="store_true")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeat", type=int, default=1)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--out-dir", type=str, default=os.path.join(ROOT, "results", "eval_perf"))
    ap.add_argument("--run-tag", type=str, default="")
    ap.add_argument("--sdpa-flash", action="store_true")
    ap.add_argument("--sdpa-mem-efficient", action="store_true")
    ap.add_argument("--sdpa-math", action="store_true")
    ap.add_argument("--planner-mode", type=str, default="none", choices=["none", "rs_prefetch"])
    ap.add_argument("--expert-source", type=str, default="router", choices=["router", "rs"])
    ap.add_argument("--prefetch-top-m", type=int, default=4)
    ap.add_argument("--rs-group", type=int, default=3)
    ap.add_argument("--rs-debug", action="store_true")
    ap.add_argument("--oracle-mode", type=str, default="none", choices=["none", "record", "replay"])
    ap.add_argument("--oracle-trace-dir", type=str, default="")
    ap.add_argument("--oracle-ignore-cache-capacity", action="store_true")
    ap.add_argument("--lm-head-device", type=str, default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--max-scan-samples", type=int, default=2000)
    ap.add_argument("--dataset-skip-valid", type=int, default=int(os.environ.get("DATASET_SKIP_VALID", "0") or 0))
    ap.add_argument("--placement-mode", type=str, default=os.environ.get("SPARSE_PLACEMENT", "round_robin"),
                    choices=["scp", "scp_ep", "round_robin", "weighted_random_balanced"])
    ap.add_argument("--scp-ep-placement", type=str, default=os.environ.get("SPARSE_SCP_EP_PLACEMENT", ""))
    ap.add_argument("--runtime-mode", type=str, default="baseline", choices=["baseline"])
    ap.add_argument("--ep-size", type=int, default=0)
    return ap


def check_args(args, world: int) -> None:
    """The constraints the reference enforces at start (scripts/perf.py:3756-3763) and this build's own."""
    ep = args.ep_size if args.ep_size else world
    if ep <= 0 or world % ep != 0:
        raise SystemExit(f"world % ep_size must be 0 (world={world}, ep_size={ep})")
    if args.batch < world // ep:
        raise SystemExit(f"batch ({args.batch}) must be >= dp_size ({world // ep})")
    if args.enable_skvs:
        raise SystemExit("--enable-skvs: SKVS attention is not part of the B200 MoE-layer path")
    if args.oracle_mode != "none":
        raise SystemExit("--oracle-mode record/replay is not part of the B200 MoE-layer path")
    if args.routing_mode != "router" or args.expert_source != "router":
        raise SystemExit("only --routing-mode router and --expert-source router are built")
    if args.cache_policy != "lru":
        raise SystemExit("only --cache-policy lru is built (the reference's launchers use nothing else)")
    if args.dtype != "bfloat16":
        raise SystemExit("the B200 MoE path computes in bfloat16: pass --dtype bfloat16")
    if args.dataset != "synthetic":
        raise SystemExit("--dataset: no prompt dataset is available offline; pass --dataset synthetic")
    if args.lm_head_device != "cuda":
        raise SystemExit("--lm-head-device cpu is not built")


def _std(values: List[float]):
    return statistics.stdev(values) if len(values) > 1 else None


def reduce_and_build_perf_record(args, env, metrics, prompt_tokens: int, gen_tokens: int, wall_total_s: float,
                                 ec) -> Dict[str, Any]:
    """One repeat's record with the reference's key names (scripts/perf.py:2422-2460):
    token counts summed over ranks, wall clocks as the maximum over ranks."""
    dev = env.device
    tok = torch.tensor([prompt_tokens, gen_tokens], dtype=torch.float64, device=dev)
    wall = torch.tensor([wall_total_s * 1e3, metrics.wall_prefill_ms, metrics.wall_decode_ms, metrics.wall_ttft_ms],
                        dtype=torch.float64, device=dev)
    counters = ["expert_weight_h2d_bytes", "expert_weight_h2d_demand_bytes", "expert_weight_h2d_prefetch_bytes",
                "expert_weight_peer_bytes", "cache_hit_count", "cache_miss_count", "prefetch_issued_count",
                "prefetch_admitted_count", "prefetch_completed_count", "prefetch_wasted_count",
                "prefetch_complete_before_use_count", "prefetch_late_count", "comm_bytes_activation",
                "comm_bytes_activation_remote", "epipe_attempt_count", "epipe_trigger_count",
                "epipe_staged_expert_count", "epipe_fallback_count"]
    cnt = torch.tensor([float(getattr(metrics, c)) for c in counters], dtype=torch.float64, device=dev)
    if env.world > 1:
        ec.all_reduce_sum_(tok)
        ec.all_reduce_max_(wall)
        ec.all_reduce_sum_(cnt)
    p, g = float(tok[0].item()), float(tok[1].item())
    total_ms, prefill_ms, decode_ms, ttft_ms = [float(v) for v in wall.tolist()]
    streams = args.batch * env.world
    rec: Dict[str, Any] = {
        "prompt_len": args.prompt_len, "prompt_tokens": int(p), "gen_tokens": int(g),
        "prompt_tokens_all_ranks": int(p), "gen_tokens_all_ranks": int(g),
        "wall_total_ms": total_ms, "wall_prefill_ms": prefill_ms, "wall_decode_ms": decode_ms,
        "wall_ttft_ms": ttft_ms,
        "decode_initial_tokens_excluded": streams,
        "decode_tokens_counted": max(0, int(g) - streams),
        "e2e_total_tok_s": (p + g) / max(total_ms * 1e-3, 1e-12),
        "e2e_output_tok_s": g / max(total_ms * 1e-3, 1e-12),
        "throughput_tok_s": (p + g) / max(total_ms * 1e-3, 1e-12),
        "decode_throughput_tok_s": max(0.0, g - streams) / max(decode_ms * 1e-3, 1e-12),
        "decode_throughput_tok_s_semantics": "Decode throughput excludes the first generated token per active "
                                             "request stream and divides by wall_decode_s.",
        "token_count_semantics": "summed over all ranks: every rank decodes its own sequences",
        "comm_mb_activation": float(cnt[counters.index("comm_bytes_activation")].item()) / 1024 ** 2,
        "comm_mb_activation_remote": float(cnt[counters.index("comm_bytes_activation_remote")].item()) / 1024 ** 2,
        "peak_allocated_mb": metrics.peak_allocated_mb, "peak_reserved_mb": metrics.peak_reserved_mb,
    }
    for c, v in zip(counters, cnt.tolist()):
        rec[c] = int(v)
    rec["h2d_total_mb"] = rec["expert_weight_h2d_bytes"] / 1024 ** 2
    if metrics.decode_step_stats is not None:
        rec.update(metrics.decode_step_stats.summary("decode_step_"))
    return rec


def aggregate_repeats(records: List[Dict[str, Any]], args, env) -> Dict[str, Any]:
    """Mean over repeats plus `_std` of the throughput keys (scripts/perf.py:3300-3400)."""
    summary: Dict[str, Any] = {
        "model_path": args.model_path, "dataset": args.dataset, "batch": args.batch, "max_new": args.max_new,
        "dtype": args.dtype, "world_size": env.world, "ep_size": args.ep_size or env.world,
        "placement_mode": args.placement_mode, "planner_mode": args.planner_mode,
        "expert_offload": args.expert_offload, "expert_cache": args.expert_cache, "warmup": args.warmup,
        "repeat": args.repeat, "run_tag": args.run_tag, "seed": args.seed,
    }
    numeric = [k for k, v in records[0].items() if isinstance(v, (int, float)) and not isinstance(v, bool)]
    for k in numeric:
        vals = [float(r[k]) for r in records]
        summary[k] = sum(vals) / len(vals)
    for k in records[0]:
        if k not in summary:
            summary[k] = records[0][k]
    for k in ("e2e_output_tok_s", "decode_throughput_tok_s", "e2e_total_tok_s"):
        summary[k + "_std"] = _std([float(r[k]) for r in records])
    summary["raw_repeats"] = records
    return summary


def save_aggregated_perf(summary: Dict[str, Any], args) -> List[str]:
    os.makedirs(args.out_dir, exist_ok=True)
    ts = time.strftime("%Y%m%d-%H%M%S")
    tag = args.run_tag or "default"
    light = dict(summary)
    light.pop("raw_repeats", None)
    paths = [os.path.join(args.out_dir, f"{tag}_summary.json"),
             os.path.join(args.out_dir, f"run_{ts}_{tag}_summary.json")]
    for pth in paths:
        with open(pth, "w", encoding="utf-8") as f:
            json.dump(light, f, indent=2, ensure_ascii=False)
    raw = os.path.join(args.out_dir, f"run_{ts}_{tag}_raw_repeats.json")
    with open(raw, "w", encoding="utf-8") as f:
        json.dump(summary.get("raw_repeats", []), f, indent=2, ensure_ascii=False)
    with open(os.path.join(args.out_dir, "runs.jsonl"), "a", encoding="utf-8") as f:
        f.write(json.dumps(light, ensure_ascii=False) + "\n")
    return paths + [raw]


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    check_args(args, world)
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    import sparse_b200.compat as compat
    compat.activate()
    import utils.eval_core as ec
    torch.manual_seed(args.seed)
    env = ec.init_dist("nccl")
    ec.set_sdpa_mode(args.sdpa_flash or not (args.sdpa_mem_efficient or args.sdpa_math),
                     args.sdpa_mem_efficient or not (args.sdpa_flash or args.sdpa_math),
                     args.sdpa_math or not (args.sdpa_flash or args.sdpa_mem_efficient))
    metrics = ec.Metrics()
    metrics.decode_step_stats = ec.RunningStats()
    cfg = ec.CoreBuildConfig(
        model_path=args.model_path, scp_path=args.scp_path, rs_dir=args.rs_dir, dtype=args.dtype,
        expert_offload=args.expert_offload, expert_cache=args.expert_cache, cache_policy=args.cache_policy,
        prompt_len=args.prompt_len, max_new_tokens=args.max_new, routing_mode=args.routing_mode,
        expert_source=args.expert_source, placement_mode=args.placement_mode, scp_ep_path=args.scp_ep_placement,
        runtime_mode=args.runtime_mode, rs_require_complete=args.rs_require_complete,
        log_routing_stats=args.log_routing_stats, planner_mode=args.planner_mode,
        prefetch_top_m=args.prefetch_top_m, ep_size=args.ep_size, batch=args.batch)
    bundle = ec.build_model_and_tokenizer(cfg, env, metrics)
    model = bundle.model
    vocab = bundle.tokenizer.vocab_size
    records: List[Dict[str, Any]] = []
    for it in range(args.warmup + args.repeat):
        timed = it >= args.warmup
        g = torch.Generator().manual_seed(args.seed * 100003 + 1009 * it + env.rank)
        new = args.max_new if timed else min(8, args.max_new)           # the launchers warm up with 8 tokens
        ids = torch.randint(0, vocab, (args.batch, args.prompt_len), generator=g).to(env.device)
        metrics.reset_for_repeat()
        metrics.decode_step_stats = ec.RunningStats()
        ec.SparseContext.reset_runtime_state_for_new_request(clear_caches=True)
        if env.world > 1:
            ec.barrier(env)
        with ec.wall_timer_s() as wt:
            out = ec.greedy_decode_profiled(model, ids, torch.ones_like(ids), new, env, metrics, args.measure_ttft)
            torch.cuda.synchronize(env.device)
        wall_s = wt()
        if timed:
            records.append(reduce_and_build_perf_record(args, env, metrics, int(ids.numel()),
                                                        int(out.shape[0] * (out.shape[1] - ids.shape[1])), wall_s, ec))
    if args.log_routing_stats:
        ec.print_routing_stats_if_enabled(env, bundle)
    if env.rank == 0:
        summary = aggregate_repeats(records, args, env)
        paths = save_aggregated_perf(summary, args)
        print("\n===== PERF RUN SUMMARY (rank0, aggregated over repeats) =====")
        for k in ("e2e_output_tok_s", "decode_throughput_tok_s", "wall_total_ms", "wall_prefill_ms", "wall_decode_ms"):
            print(f"{k}: {summary[k]:.3f}")
        print("summary:", paths[0])
    if env.world > 1:
        ec.barrier(env)
    ec.destroy_dist()
    return 0


if __name__ == "__main__":
    sys.exit(main())
