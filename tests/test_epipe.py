"""CPU: EPIPE ordering decisions (the rules of utils/eval_core.py:11867-12167 and
12169-12512 of the reference: at least one ready group must cover the copy;
the residual is the first late expert, else the first demand miss; exactly
one expert is staged)."""
from sparse_b200.epipe import RollingGate, classify, plan_residual_scan, plan_upfront_scan


def test_classify_and_upfront_scan():
    resident = {1, 4, 7}
    needed = [1, 2, 4, 9]
    plan = plan_upfront_scan(needed, lambda e: e in resident)
    assert plan.first == [1, 4] and plan.residual == 2 and plan.residual_kind == "demand" and plan.rest == [9]
    assert plan_upfront_scan([2, 9], lambda e: e in resident) is None        # nothing to hide the copy behind
    assert plan_upfront_scan([1, 4], lambda e: e in resident) is None        # nothing missing
    assert plan_upfront_scan([], lambda e: True) is None


def test_residual_scan_prefers_late_prefetch():
    resident, pending = {1, 3, 5}, {3}
    is_res, is_pend = (lambda e: e in resident), (lambda e: e in pending)
    assert classify([1, 2, 3, 5, 8], is_res, is_pend) == ([1, 5], [3], [2, 8])
    plan = plan_residual_scan([1, 2, 3, 5, 8], is_res, is_pend)
    assert (plan.first, plan.residual, plan.residual_kind, plan.rest) == ([1, 5], 3, "late", [2, 8])
    plan = plan_residual_scan([1, 2, 5, 8], is_res, is_pend)
    assert (plan.first, plan.residual, plan.residual_kind, plan.rest) == ([1, 5], 2, "demand", [8])
    assert plan_residual_scan([2, 3], is_res, is_pend) is None               # no ready group
    assert plan_residual_scan([1, 5], is_res, is_pend) is None               # nothing to overlap
    assert plan_residual_scan([1, 2], is_res, is_pend, handle_demand=False) is None
    assert plan_residual_scan([1, 3], is_res, is_pend, handle_late=False) is None


def test_rolling_gate_skips_after_a_dry_window():
    g = RollingGate(window=4, min_triggers=1, skip_steps=3)
    for _ in range(4):
        assert g.should_attempt()
        g.record(False)
    assert [g.should_attempt() for _ in range(4)] == [False, False, False, True]
    g2 = RollingGate(window=4, min_triggers=1, skip_steps=3)
    for i in range(8):
        assert g2.should_attempt()
        g2.record(i % 4 == 0)


def test_scans_make_the_reference_decisions():
    """400 cases recorded by calling the reference's own
    `_try_execute_local_recv_groups_epipe` and `..._epipe_rs_residual_scan`
    (utils/eval_core.py:11867-12512) on a stand-in object
    (tests/golden/make_epipe_golden.py): whether EPIPE triggers, which expert is
    overlapped with the ready ones, what runs before and after it."""
    import json
    import os
    from sparse_b200.epipe import plan_residual_scan, plan_upfront_scan
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "epipe_golden.json")
    with open(path) as fh:
        cases = json.load(fh)
    assert len(cases) == 400
    triggered = 0
    for c in cases:
        needed = [s[0] for s in c["segments"]]
        resident, pending = set(c["resident"]), set(c["pending"])
        if c["scan"] == "upfront":
            plan = plan_upfront_scan(needed, lambda e: e in resident)
        else:
            plan = plan_residual_scan(needed, lambda e: e in resident, lambda e: e in pending)
        assert (plan is None) == c["fell_back"], c
        if plan is None:
            continue
        triggered += 1
        order = c["order"]
        n_first = len(plan.first)
        # the reference computes the ready segments first (one by one; here one grouped launch) ...
        assert sorted(order[:n_first]) == sorted(plan.first), c
        # ... then the overlapped expert, then the others in segment order
        assert order[n_first] == plan.residual, c
        assert order[n_first + 1:] == plan.rest, c
        if c["staged"]:
            assert plan.residual_kind == "demand" and c["staged"] == [plan.residual], c
        else:
            assert plan.residual_kind == "late", c
    assert triggered > 200
