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
