"""Golden cases for the prefetch planner, produced by the REFERENCE's own
methods (`_build_target_layer_prob_score_map`, `_build_prefetch_plan_from_score_map`,
`_pick_victims_by_low_value` of DistributedSparseMoeBlock) bound to a small
stand-in object, in the manner of the reference's AST-extraction unit tests.

    python tests/golden/make_planner_golden.py --reference <checkout of louislichen/SPARSE>
"""
import argparse
import json
import os
import random
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    a = ap.parse_args()
    sys.path.insert(0, a.reference)
    for k in list(os.environ):
        if k.startswith("SPARSE_"):
            del os.environ[k]
    import torch
    import utils.eval_core as ec
    B = ec.DistributedSparseMoeBlock
    cases = []
    rnd = random.Random(5)
    for ci in range(300):
        E = 16
        local = set(rnd.sample(range(E), rnd.randrange(6, E + 1)))
        cap = rnd.choice([2, 3, 4, 6])
        cache = ec.ExpertWeightCache(cap)
        setup = []
        for _ in range(rnd.randrange(0, cap + 2)):
            e = rnd.choice(sorted(local))
            pinned = rnd.random() < 0.25
            cache.put(e, "w", pinned=pinned)
            setup.append([e, pinned])
        freq = {e: rnd.randrange(0, 20) for e in rnd.sample(range(E), 5)}
        prefetched = set(rnd.sample(range(E), rnd.randrange(0, 3)))
        policy = rnd.choice(["default", "cache_safe"])
        os.environ["SPARSE_RS_PREFETCH_POLICY"] = policy
        me = types.SimpleNamespace()
        me.layer_idx, me.comm_rank, me.planner_mode = 3, 0, "rs_prefetch"
        me._cache = cache
        me._expert_access_freq = freq
        me._prefetched_ids_this_group = prefetched
        me._prefetch_min_candidate_score = rnd.choice([0.02, 0.04])
        me._prefetch_replace_advantage = rnd.choice([0.02, 0.08])
        me._prefetch_replace_margin = rnd.choice([1.05, 1.2])
        me._prefetch_allow_active_replace = rnd.random() < 0.8
        counters = {}
        me._record_rs_counter = lambda name, value=1: counters.__setitem__(name, counters.get(name, 0) + int(value))
        me._record_rs_resolver_match = lambda **kw: None
        me._stage_prefetch_eid_set = lambda stage=None: set(local)
        me._current_stage = lambda: "decode"
        me.resolve_prefetch_target_rank = lambda **kw: types.SimpleNamespace(
            target_rank=0 if int(kw["expert_id"]) in local else 1)
        me._rs_prefetch_policy = lambda: policy
        me._rank_env_float = lambda name, default: float(default)
        me._rs_env_float = lambda name, default: float(default)
        me._prefetch_free_slots = lambda: cache.prefetch_free_slots()
        me._prefetch_evictable_ids = lambda protect=None: cache.evictable_prefetch_ids(protect)
        me._resident_keep_bias = types.MethodType(B._resident_keep_bias, me)
        me._pick_victims_by_low_value = types.MethodType(B._pick_victims_by_low_value, me)
        T, K = rnd.randrange(1, 5), 4
        topi = torch.tensor([[rnd.randrange(E) for _ in range(K)] for _ in range(T)])
        topv = torch.tensor([[round(rnd.random() * 0.5, 4) for _ in range(K)] for _ in range(T)])
        score_map = B._build_target_layer_prob_score_map(me, topi, topv)
        protect = set(rnd.sample(range(E), rnd.randrange(0, 3)))
        budget = rnd.randrange(0, 4)
        plan = B._build_prefetch_plan_from_score_map(me, dict(score_map), protect_ids=set(protect), budget=budget)
        cases.append({
            "local": sorted(local), "capacity": cap, "setup": setup, "freq": {str(k): v for k, v in freq.items()},
            "prefetched": sorted(prefetched), "policy": policy,
            "min_score": me._prefetch_min_candidate_score, "adv": me._prefetch_replace_advantage,
            "margin": me._prefetch_replace_margin, "active": me._prefetch_allow_active_replace,
            "topi": topi.tolist(), "topv": topv.tolist(), "protect": sorted(protect), "budget": budget,
            "score_map": {str(k): v for k, v in score_map.items()},
            "plan": [[int(e), None if v is None else int(v)] for e, v in plan],
            "counters": counters,
        })
    with open(os.path.join(HERE, "planner_golden.json"), "w") as fh:
        json.dump(cases, fh, separators=(",", ":"))
    print("planner cases", len(cases), "non-empty plans", sum(1 for c in cases if c["plan"]),
          "with victims", sum(1 for c in cases if any(v is not None for _, v in c["plan"])))


if __name__ == "__main__":
    main()
