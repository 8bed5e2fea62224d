"""CPU: host-side logic against traces recorded from the reference
(tests/golden/host_golden.json, written by tests/golden/make_host_golden.py)
and the scenarios the reference's own unit tests pin
(tests/test_rs_staging.py:74-150, 308-312 of the reference)."""
import itertools
import json
import os
import threading

import pytest

from conftest import GOLDEN_DIR
from sparse_b200.cache import ExpertWeightCache
from sparse_b200.placement import Placement, balanced_replicated_placement, weighted_random_balanced
from sparse_b200.staging import DemandView, StagingJob, Transfer, select_candidates


@pytest.fixture(scope="module")
def golden():
    with open(os.path.join(GOLDEN_DIR, "host_golden.json")) as fh:
        return json.load(fh)


def _apply(c, op, a):
    if op == "get":
        return c.get(a[0])
    if op == "peek":
        return c.peek(a[0])
    if op == "has":
        return c.has(a[0])
    if op == "put":
        r = c.put(a[0], a[1], pinned=a[2], protect_ids=set(a[3]), prefill_scp_transient=a[4])
        return [r, c.last_evicted_was_prefill_scp_transient()]
    if op == "admit":
        return c.admit_prefetch(a[0], a[1], protect_ids=set(a[2]), preferred_victim=a[3])
    if op == "unpin_all":
        return c.unpin_all()
    if op == "unpin":
        return c.unpin(a[0])
    if op == "promote":
        return c.promote_hot(a[0])
    if op == "discard":
        return c.discard(a[0])
    if op == "demote":
        return c.demote_prefill_scp_transients()
    if op == "evictable":
        return c.evictable_prefetch_ids(set(a[0]))
    if op == "clear_transient":
        return c.clear_prefill_scp_transient(a[0])
    raise AssertionError(op)


def test_cache_replays_reference_traces(golden):
    n_ops = 0
    for trace in golden["cache"]:
        c = ExpertWeightCache(trace["capacity"])
        for step in trace["ops"]:
            got = _apply(c, step["op"], step["args"])
            assert got == step["ret"], (trace["capacity"], step)
            state = [[k, e.payload, e.pinned, e.transient] for k, e in c._order.items()]
            assert state == step["state"], step
            assert c.prefetch_free_slots() == step["free"]
            n_ops += 1
    assert n_ops >= 4000


def test_wrong_forecasts_never_perturb_lru_order():
    """All 2^6 access sequences over two experts: a DemandView in front of the
    cache, with staged-but-unused transfers, leaves the same order as a plain LRU."""
    for seq in itertools.product([0, 1], repeat=6):
        plain, real = ExpertWeightCache(2), ExpertWeightCache(2)
        view = DemandView(real)
        view.staged[7] = Transfer(7, "spec", None, None, 1)      # a forecast nobody uses
        for e in seq:
            for c in (plain, view):
                if c.get(e) is None:
                    (plain if c is plain else real).put(e, "w%d" % e)
        assert real.resident_ids() == plain.resident_ids()
        assert view.used_in_order == []


def test_select_candidates_matches_reference(golden):
    for case in golden["candidates"]:
        diag = {} if case["diag"] is not None else None
        got = select_candidates(case["ids"], case["weights"], allowed=set(case["allowed"]),
                                resident=set(case["resident"]), minimum=case["minimum"],
                                budget=case["budget"], diagnostics=diag)
        assert got == case["ret"], case
        if diag is not None:
            assert diag == case["diag"]
    assert select_candidates([0, 8, 8, 9, 12], [.9, .1, .1, 1., .15], allowed={8, 9, 12}, resident={9},
                             minimum=.04, budget=1) == [8]


def test_staging_job_publish_and_close_exclude_each_other():
    job = StagingJob(ticket=1, slots=2)
    entered, release = threading.Event(), threading.Event()

    def slow_submit():
        entered.set()
        assert release.wait(5)
        return Transfer(3, "payload", "event", "slot", 10)

    worker = threading.Thread(target=lambda: job.publish(3, slow_submit))
    worker.start()
    assert entered.wait(5)
    closed = {}
    closer = threading.Thread(target=lambda: closed.update(job.close()))
    closer.start()
    closer.join(0.2)
    assert closer.is_alive(), "close() must wait for the submission in progress"
    release.set()
    worker.join(5)
    closer.join(5)
    assert list(closed) == [3]
    assert job.publish(4, lambda: Transfer(4, None, None, None, 0)) is False


def test_demand_view_marks_use_once_and_peek_is_silent():
    real = ExpertWeightCache(2)
    real.put(1, "resident")
    view = DemandView(real)
    tr = Transfer(5, "staged", "ev", "slot", 4)
    view.staged[5] = tr
    assert view.has(5) and view.has(1) and not view.has(6)
    assert view.peek(5) == "staged" and tr.used is False and view.used_in_order == []
    assert view.get(5) == "staged" and view.get(5) == "staged"
    assert view.used_in_order == [tr]
    assert view.get(1) == "resident" and view.capacity == 2


def test_placement_matches_reference(golden):
    for case in golden["placement"]:
        p = Placement("scp_ep", case["L"], case["E"], case["ep"], obj=case["obj"],
                      rank_to_node=case["rank_to_node"], apply_prefill=True, apply_decode=True)
        for key, want in case["expect"].items():
            parts = key.split("|")
            if parts[0] == "rx":
                _, l, stage, r = parts
                if want is None:
                    continue
                # the reference's receive view is per stage; with no stage it uses the default table
                got = set()
                for row in p.dest_table(int(l), stage):
                    got.update(e for e, d in enumerate(row) if d == int(r))
                if p.replicated and p._stage_table(stage) is None:
                    assert sorted(got) == want, (case["name"], key)
                continue
            l, stage, s = parts
            assert p.assignment(int(l), int(s), stage) == want, (case["name"], key)
    for key, want in golden["wrb"].items():
        ep, l = key.split("|")
        assert weighted_random_balanced(60, int(ep), int(l)) == want


def test_placement_modes_and_errors():
    rr = Placement("round_robin", 2, 10, 4)
    assert rr.dest_table(0)[3] == [e % 4 for e in range(10)]
    flat = Placement("scp", 2, 4, 2, obj={"0": 1, "5": 0})
    assert flat.assignment(0, 0, "prefill") == [1, 1, 0, 1]
    assert flat.assignment(1, 0, "prefill") == [0, 0, 0, 1]
    assert flat.assignment(0, 0, "decode") == [0, 1, 0, 1]          # decode keeps round-robin by default
    with pytest.raises(KeyError):
        Placement("scp_ep", 2, 4, 2, obj={"placement": {"0": {"0": 0}}}).assignment(0, 0, "prefill")
    with pytest.raises(ValueError):
        Placement("scp_ep", 1, 2, 2, obj={"placement": {"0": {"0": 0, "1": 5}}}).assignment(0, 0, "prefill")
    with pytest.raises(ValueError):
        Placement("nonsense", 1, 2, 2)
    with pytest.raises(ValueError):
        Placement("scp_ep", 1, 2, 2)


def test_balanced_replicated_placement_spreads_a_hot_expert():
    load = [[100, 5, 5, 5, 5, 5, 5, 5]]
    obj = balanced_replicated_placement(load, 4)
    p = Placement("scp_ep", 1, 8, 4, obj=obj, apply_decode=True)
    assert len(p.replicas(0)[0]) >= 3
    per_rank = [0.0] * 4
    for s in range(4):
        for e, d in enumerate(p.assignment(0, s, "prefill")):
            per_rank[d] += load[0][e] / 4
    assert max(per_rank) < 0.45 * sum(per_rank)


def test_rs_trainer_learns_a_routing_function_and_writes_loadable_checkpoints(tmp_path):
    """`rs_train` on data whose next-layer routing is a fixed function of the
    input: recall far above chance, and the checkpoint it writes is read back by
    the serving-side loader with identical outputs."""
    import torch
    from sparse_b200 import rs, rs_train
    torch.manual_seed(0)
    n, h, e, k = 3000, 32, 12, 2
    x = torch.randn(n, h)
    w = torch.randn(e, h)
    ids = torch.topk(x @ w.t(), k, dim=-1).indices
    pairs = {(0, 1): (x, ids), (1, 2): (x, ids.flip(1))}
    rows = rs_train.train_bank(pairs, str(tmp_path), e, hidden_dim=64, num_hidden_layers=1, epochs=25,
                               device=torch.device("cpu"), eval_ks=(2, 4))
    assert [r["target_layer"] for r in rows] == [1, 2]
    chance = 4 / e
    assert all(r["recall@4"] > 0.75 > chance for r in rows), rows
    bank, task, layout, sources, missing = rs.load_rs_bank(str(tmp_path), 3, h, e, torch.device("cpu"), False)
    assert task == "router_prob" and layout == "next_layer" and sources[1:] == [0, 1] and not missing
    mod, _ = rs_train.train_pair(x[:200], ids[:200], e, 64, 1, epochs=1, device=torch.device("cpu"))
    payload = torch.load(rows[0]["ckpt"], map_location="cpu", weights_only=False)
    assert payload["label_type"] == "next_layer_true_router_topk_multihot" and payload["lead_layers"] == 1
    probs = bank[1](x[:50])
    assert probs.shape == (50, e) and torch.allclose(probs.sum(-1), torch.ones(50), atol=1e-5)
    assert rs_train.recall_at_k(probs, ids[:50], 4) > 0.7
