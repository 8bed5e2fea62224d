"""Golden traces for the host-side logic, produced by running the REFERENCE:

    python tests/golden/make_host_golden.py --reference <checkout of louislichen/SPARSE>

Writes tests/golden/host_golden.json with
  * random operation sequences on the reference's `ExpertWeightCache` and what
    every call returned plus the resident order after it;
  * random inputs to the reference's `select_candidates` and its outputs;
  * the reference's placement functions evaluated on synthetic placement files
    of every schema (plain, replicated with/without cost matrix and tables,
    weighted-random-balanced).
"""
import argparse
import json
import os
import random
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def cache_traces(ec, n_traces=60, n_ops=80):
    out = []
    for t in range(n_traces):
        rnd = random.Random(1000 + t)
        cap = rnd.choice([0, 1, 2, 3, 4, 6])
        c = ec.ExpertWeightCache(cap)
        ops = []
        for _ in range(n_ops):
            kind = rnd.choice(["get", "get", "put", "put", "put", "admit", "admit", "peek", "has", "unpin_all",
                               "discard", "demote", "evictable", "clear_transient", "unpin", "promote"])
            e = rnd.randrange(8)
            prot = sorted(rnd.sample(range(8), rnd.randrange(0, 3)))
            if kind == "get":
                res = c.get(e)
                args = [e]
            elif kind == "peek":
                res = c.peek(e); args = [e]
            elif kind == "has":
                res = c.has(e); args = [e]
            elif kind == "put":
                pinned, tr = rnd.random() < 0.2, rnd.random() < 0.3
                payload = "p%d_%d" % (e, len(ops))
                res = c.put(e, payload, pinned=pinned, protect_ids=set(prot), prefill_scp_transient=tr)
                args = [e, payload, pinned, prot, tr]
                res = [res, c.last_evicted_was_prefill_scp_transient()]
            elif kind == "admit":
                pv = rnd.choice([None, rnd.randrange(8)])
                payload = "a%d_%d" % (e, len(ops))
                res = c.admit_prefetch(e, payload, protect_ids=set(prot), preferred_victim=pv)
                args = [e, payload, prot, pv]
            elif kind == "unpin_all":
                c.unpin_all(); res = None; args = []
            elif kind == "unpin":
                c.unpin(e); res = None; args = [e]
            elif kind == "promote":
                c.promote_hot(e); res = None; args = [e]
            elif kind == "discard":
                res = c.discard(e); args = [e]
            elif kind == "demote":
                res = c.demote_prefill_scp_transients(); args = []
            elif kind == "evictable":
                res = c.evictable_prefetch_ids(set(prot)); args = [prot]
            elif kind == "clear_transient":
                res = c.clear_prefill_scp_transient(e); args = [e]
            state = [[int(k), v.payload, bool(v.pinned), bool(v.prefill_scp_transient)] for k, v in c._lru.items()]
            ops.append({"op": kind, "args": args, "ret": res, "state": state, "free": c.prefetch_free_slots()})
        out.append({"capacity": cap, "ops": ops})
    return out


def candidate_cases(rs, n=200):
    out = []
    rnd = random.Random(7)
    for _ in range(n):
        m = rnd.randrange(0, 12)
        ids = [rnd.randrange(16) for _ in range(m)]
        ws = [round(rnd.random(), 3) for _ in range(m)]
        allowed = sorted(rnd.sample(range(16), rnd.randrange(4, 16)))
        resident = sorted(rnd.sample(range(16), rnd.randrange(0, 6)))
        minimum = rnd.choice([0.0, 0.02, 0.04, 0.2, 0.5])
        budget = rnd.randrange(0, 5)
        diag = {}
        res = rs.select_candidates(ids, ws, allowed=set(allowed), resident=set(resident), minimum=minimum,
                                   budget=budget, diagnostics=diag)
        out.append({"ids": ids, "weights": ws, "allowed": allowed, "resident": resident, "minimum": minimum,
                    "budget": budget, "ret": res, "diag": diag})
    out.append({"ids": [0, 8, 8, 9, 12], "weights": [.9, .1, .1, 1., .15], "allowed": [8, 9, 12], "resident": [9],
                "minimum": .04, "budget": 1,
                "ret": rs.select_candidates([0, 8, 8, 9, 12], [.9, .1, .1, 1., .15], allowed={8, 9, 12},
                                            resident={9}, minimum=.04, budget=1), "diag": None})
    return out


def placement_cases(ec):
    rnd = random.Random(11)
    L, E = 3, 12
    cases = []
    for ep in (2, 4):
        plain = {"placement": {str(l): {str(e): rnd.randrange(ep) for e in range(E)} for l in range(L)}}
        reps = {str(l): {str(e): sorted(rnd.sample(range(ep), rnd.randrange(1, ep + 1))) for e in range(E)}
                for l in range(L)}
        rep_v1 = {"format": "replicated_scp_ep_v1", "replicas": reps,
                  "rank_to_node": {str(r): r // 2 for r in range(ep)}}
        cm = [[0.0 if s == d else round(rnd.uniform(0.5, 9), 2) for d in range(ep)] for s in range(ep)]
        rep_v2 = {"format": "replicated_scp_ep_v2", "replicas": reps, "replica_choice_cost_matrix": cm}
        nodes = ep // 2
        table = {str(l): {str(n): [rnd.choice(reps[str(l)][str(e)]) for e in range(E)] for n in range(nodes)}
                 for l in range(L)}
        table_dec = {str(l): {str(n): {str(e): rnd.choice(reps[str(l)][str(e)]) for e in range(E)}
                              for n in range(nodes)} for l in range(L)}
        rep_v3 = {"format": "replicated_scp_ep_v3", "replicas": reps, "dest_rank_table": table,
                  "dest_rank_table_decode": table_dec, "source_nodes": list(range(nodes))}
        for name, obj, r2n in (("plain", plain, None), ("rep_v1", rep_v1, [r // 2 for r in range(ep)]),
                               ("rep_v2", rep_v2, None), ("rep_v3", rep_v3, [r // 2 for r in range(ep)])):
            exp = {}
            for l in range(L):
                for stage in ("", "prefill", "decode"):
                    for s in range(ep):
                        a = ec._scp_ep_layer_assignment(obj, layer_idx=l, num_experts=E, world=ep, source_rank=s,
                                                        stage=stage, rank_to_node=r2n)
                        exp["%d|%s|%d" % (l, stage, s)] = a
                    for r in range(ep):
                        rx = ec._scp_ep_layer_receive_experts(obj, layer_idx=l, num_experts=E, world=ep, rank=r,
                                                              stage=stage, rank_to_node=r2n)
                        exp["rx|%d|%s|%d" % (l, stage, r)] = None if rx is None else sorted(rx)
            cases.append({"name": name, "ep": ep, "L": L, "E": E, "obj": obj, "rank_to_node": r2n, "expect": exp})
    wrb = {}
    for ep in (2, 4, 8):
        for l in (0, 5):
            wrb["%d|%d" % (ep, l)] = ec._weighted_random_balanced_assignment(60, ep, l)
    return cases, wrb


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    a = ap.parse_args()
    sys.path.insert(0, a.reference)
    for k in list(os.environ):
        if k.startswith("SPARSE_"):
            del os.environ[k]
    import utils.eval_core as ec
    import utils.rs_staging as rs
    pc, wrb = placement_cases(ec)
    data = {"cache": cache_traces(ec), "candidates": candidate_cases(rs), "placement": pc, "wrb": wrb}
    with open(os.path.join(HERE, "host_golden.json"), "w") as fh:
        json.dump(data, fh, separators=(",", ":"))
    print("cache traces", len(data["cache"]), "candidate cases", len(data["candidates"]),
          "placement cases", len(pc))


if __name__ == "__main__":
    main()
