"""CPU: the reference's module paths and launcher flags resolve to this build
(scripts/perf.py:24-42 and 3655-3734 of the reference), and the staging
ownership rules the reference's tests pin (tests/test_rs_staging.py of the
reference) hold through the shim names."""
import json
import threading

import pytest


@pytest.fixture()
def compat_modules():
    import sparse_b200.compat as compat
    compat.activate()
    import utils.eval_core as ec
    import utils.rs_overlap as ro
    import utils.rs_staging as rs
    import utils.runtime.config as rc
    return ec, rs, ro, rc


def test_every_symbol_the_launcher_imports_exists(compat_modules):
    ec, rs, ro, rc = compat_modules
    for name in ("CoreBuildConfig", "DistEnv", "Metrics", "RunningStats", "SparseContext", "all_reduce_max_",
                 "all_reduce_sum_", "barrier", "build_model_and_tokenizer", "destroy_dist", "greedy_decode_profiled",
                 "init_dist", "print_routing_stats_if_enabled", "set_sdpa_mode", "wall_timer_s",
                 "DistributedSparseMoeBlock", "ExpertWeightCache", "build_dist_topology", "DistTopology"):
        assert hasattr(ec, name), name
    for name in ("Transfer", "TargetJob", "DemandCacheView", "select_candidates"):
        assert hasattr(rs, name), name
    assert hasattr(ro, "BoundedRS") and hasattr(ro, "GraphPrediction")
    assert rc.ers_config_from_env().enabled is False
    cfg = ec.CoreBuildConfig(model_path="synthetic:tiny", scp_path="", rs_dir="")
    assert cfg.dtype == "float16" and cfg.expert_offload == "cpu" and cfg.rs_prob_to_logit_eps == 1e-9
    with ec.wall_timer_s() as wt:
        pass
    assert wt() >= 0.0
    stats = ec.RunningStats()
    for v in (1.0, 2.0, 3.0, 10.0):
        stats.add_ms(v)
    s = stats.summary("decode_step_")
    assert s["decode_step_avg_ms"] == 4.0 and s["decode_step_p50_ms"] == 2.5 and s["decode_step_max_ms"] == 10.0


def test_unbuilt_subsystems_are_refused_not_ignored(compat_modules, monkeypatch):
    ec, rs, ro, rc = compat_modules
    import torch
    env = ec.DistEnv(rank=0, world=1, local_rank=0, device=torch.device("cpu"))
    with pytest.raises(NotImplementedError):
        ec.build_model_and_tokenizer(ec.CoreBuildConfig("synthetic:tiny", "", "", dtype="bfloat16", enable_skvs=True), env)
    with pytest.raises(NotImplementedError):
        ec.build_model_and_tokenizer(ec.CoreBuildConfig("/models/qwen", "", "", dtype="bfloat16"), env)
    with pytest.raises(NotImplementedError):
        ec.build_model_and_tokenizer(ec.CoreBuildConfig("synthetic:tiny", "", "", dtype="float16"), env)
    monkeypatch.setenv("SPARSE_ERS_ENABLE", "1")
    with pytest.raises(NotImplementedError):
        rc.ers_config_from_env()


def test_staging_rules_through_the_reference_names(compat_modules):
    """publish declines after close and never submits twice; close hands over what
    was issued; the demand view marks use on get but not on peek; candidate
    scores are sum * (1 + 0.15 (n - 1)) + 0.05 max."""
    ec, rs, ro, rc = compat_modules
    job = rs.TargetJob(ticket=7, slots=[0, 1])
    made = []

    def submit(e):
        def f():
            made.append(e)
            return rs.Transfer(expert=e, payload=("w", e), event=None, slot=len(made) - 1, nbytes=10)
        return f

    assert job.publish(3, submit(3)) is True
    issued = job.close()
    assert list(issued) == [3] and job.publish(4, submit(4)) is False and made == [3]

    class Resident:
        def __init__(self):
            self.d = {1: "r1"}

        def has(self, e):
            return e in self.d

        def get(self, e):
            return self.d.get(e)

        def peek(self, e):
            return self.d.get(e)

        def resident_ids(self):
            return list(self.d)

    view = rs.DemandCacheView(Resident())
    view.staged.update(issued)
    assert view.has(1) and view.has(3) and not view.has(9)
    assert view.peek(3) == ("w", 3) and not issued[3].used
    assert view.get(3) == ("w", 3) and issued[3].used and view.used_in_order == [issued[3]]
    assert view.get(1) == "r1" and view.resident_ids() == [1]
    picked = rs.select_candidates([5, 5, 6, 7, 8], [0.2, 0.2, 0.3, 0.01, 0.5], allowed={5, 6, 7}, resident={6},
                                  minimum=0.05, budget=4)
    assert picked == [5]                     # 8 not allowed, 6 resident, 7 below the minimum
    # publish is serialised with close: a racing closer either sees the transfer or prevents it
    job2 = rs.TargetJob(ticket=8, slots=[0])
    seen = {}
    t = threading.Thread(target=lambda: seen.update(job2.close()))
    ok = job2.publish(2, lambda: rs.Transfer(2, "p", None, 0, 1))
    t.start(); t.join()
    assert ok and list(seen) == [2]


def test_launcher_parses_the_reference_flag_surface(tmp_path):
    from sparse_b200.compat.scripts import perf
    args = perf.build_parser().parse_args([
        "--model-path", "synthetic:qwen", "--dataset", "synthetic", "--dtype", "bfloat16", "--batch", "8",
        "--prompt-len", "2048", "--max-new", "128", "--expert-offload", "cpu", "--expert-cache", "8",
        "--planner-mode", "rs_prefetch", "--prefetch-top-m", "2", "--placement-mode", "scp_ep",
        "--scp-ep-placement", "p.json", "--rs-dir", "rs", "--routing-mode", "router", "--expert-source", "router",
        "--cache-policy", "lru", "--runtime-mode", "baseline", "--ep-size", "8", "--warmup", "1", "--repeat", "3",
        "--measure-ttft", "--save-output-tokens", "--log-routing-stats", "--skvs-window", "16", "--rs-group", "3",
        "--oracle-mode", "none", "--lm-head-device", "cuda", "--max-scan-samples", "10", "--sdpa-math",
        "--out-dir", str(tmp_path), "--run-tag", "rs"])
    assert args.ep_size == 8 and args.prefetch_top_m == 2 and args.rs_require_complete is True
    perf.check_args(args, world=8)
    with pytest.raises(SystemExit):
        perf.check_args(args, world=12)                 # world % ep_size
    for bad in (["--enable-skvs"], ["--oracle-mode", "record"], ["--dtype", "float16"], ["--cache-policy", "lfu"],
                ["--dataset", "c4.jsonl"]):
        a = perf.build_parser().parse_args(["--model-path", "synthetic:qwen", "--dataset", "synthetic", "--dtype",
                                            "bfloat16"] + bad)
        with pytest.raises(SystemExit):
            perf.check_args(a, world=1)
    # the summary files and keys the reference's analysis script reads
    rec = {"e2e_output_tok_s": 10.0, "decode_throughput_tok_s": 20.0, "e2e_total_tok_s": 30.0, "wall_total_ms": 5.0,
           "wall_prefill_ms": 1.0, "wall_decode_ms": 4.0}

    class Env:
        world = 8

    summary = perf.aggregate_repeats([dict(rec), dict(rec, e2e_output_tok_s=14.0)], args, Env())
    assert summary["e2e_output_tok_s"] == 12.0 and summary["e2e_output_tok_s_std"] is not None
    paths = perf.save_aggregated_perf(summary, args)
    saved = json.loads(open(paths[0]).read())
    assert paths[0].endswith("rs_summary.json") and "raw_repeats" not in saved
    assert {"e2e_output_tok_s", "decode_throughput_tok_s", "e2e_output_tok_s_std", "decode_throughput_tok_s_std"} <= set(saved)
    assert (tmp_path / "runs.jsonl").exists()
