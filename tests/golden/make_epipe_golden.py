"""Golden cases for the EPIPE readiness scheduler, produced by the REFERENCE's
own methods `_try_execute_local_recv_groups_epipe` (upfront scan,
utils/eval_core.py:11867-12167) and
`_try_execute_local_recv_groups_epipe_rs_residual_scan` (12169-12512) bound to
a stand-in object, in the manner of the reference's AST-extraction unit tests:
the cache is the reference's `ExpertWeightCache`, CUDA streams and events are
fakes, and the segment compute is a recorder.  Stored per case: the expert
segments, which experts were resident / had a prefetch copy in flight, and
what the reference did: fell back (returned None), or the order in which it
computed the segments and which expert it staged.

    python tests/golden/make_epipe_golden.py --reference <checkout of louislichen/SPARSE>
"""
import argparse
import contextlib
import json
import os
import random
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))


class FakeEvent:
    def __init__(self, done=True, **kw):
        self.done = done

    def record(self, *a, **k):
        pass

    def query(self):
        return self.done

    def synchronize(self):
        pass


class FakeStream:
    def wait_event(self, ev):
        pass

    def wait_stream(self, s):
        pass


class Stub:
    """Attributes the scans read are set explicitly; every other `_record_*` /
    bookkeeping method is a no-op that counts its calls."""

    def __init__(self):
        self.calls = {}

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)

        def noop(*a, **k):
            self.calls[name] = self.calls.get(name, 0) + 1
            return None
        return noop


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    a = ap.parse_args()
    sys.path.insert(0, a.reference)
    for k in list(os.environ):
        if k.startswith("SPARSE_"):
            del os.environ[k]
    import torch
    import utils.eval_core as ec
    B = ec.DistributedSparseMoeBlock
    torch.cuda.is_available = lambda: True
    torch.cuda.stream = lambda s: contextlib.nullcontext()
    torch.cuda.Event = FakeEvent
    torch.cuda.current_stream = lambda dev=None: FakeStream()
    rnd = random.Random(11)
    cases = []
    for ci in range(400):
        scan = "upfront" if ci % 2 == 0 else "residual"
        E = 12
        n_seg = rnd.randrange(1, 7)
        eids = sorted(rnd.sample(range(E), n_seg))
        pos, segments = 0, []
        for e in eids:
            n = rnd.randrange(1, 5)
            segments.append((e, pos, pos + n, True))
            pos += n
        cap = rnd.choice([2, 4, 8])
        cache = ec.ExpertWeightCache(cap)
        resident = [e for e in eids if rnd.random() < 0.6][:cap]
        for e in resident:
            cache.put(e, ("w", e))
        pending = [e for e in resident if scan == "residual" and rnd.random() < 0.3]
        me = Stub()
        me._epipe_validate_output = False
        me.expert_offload, me.cache_policy, me.planner_mode = "cpu", "lru", ("rs_prefetch" if scan == "residual" else "none")
        me.device = types.SimpleNamespace(type="cuda")
        me.layer_idx, me.metrics = 0, None
        me._cache = cache
        me._epipe_enable, me._epipe_prefill_enable = True, False
        me._epipe_shadow = me._epipe_prefill_shadow = me._epipe_prefill_multistage_shadow = False
        me._epipe_min_free_mb = me._epipe_prefill_min_free_mb = 256.0
        me._epipe_decode_only, me._epipe_no_evict, me._epipe_transient_staging = True, True, True
        me._epipe_max_staged_experts = 1
        me._epipe_min_ready_experts = me._epipe_min_missing_experts = me._epipe_min_ready_items = 1
        me._epipe_min_missing_h2d_bytes = 1
        me._epipe_sort_ready_by_work = False
        me._epipe_prefill_commit, me._epipe_prefill_mark_transient = False, False
        me._global_expert_cache_enabled = False
        me.epipe_stream = FakeStream()
        me._epipe_rs_rolling_gate = False
        me._epipe_rs_handle_late_prefetch = me._epipe_rs_handle_demand_miss = True
        me._epipe_rs_force_demand_stage = True
        me._epipe_rs_min_buffer_groups, me._epipe_rs_min_buffer_items = 1, 1
        me._epipe_rs_demand_commit = False
        me._epipe_rs_gate_skip_remaining = me._epipe_rs_gate_calls = me._epipe_rs_gate_triggers = 0
        me._epipe_rs_gate_window, me._epipe_rs_gate_min_triggers, me._epipe_rs_gate_skip_steps = 16, 1, 8
        me._prefetch_events = {e: FakeEvent(done=False) for e in pending}
        me._prefetched_ids_this_group = set(pending)
        me._prefetch_used_ids_this_group = set()
        order, staged = [], []
        me._current_stage = lambda: "decode"
        me._cache_contains_no_touch = lambda eid: cache.has(int(eid))
        me._epipe_timing_sampled = lambda *a, **k: False
        me._epipe_estimate_expert_nbytes = lambda eid: 1000
        me._epipe_memory_headroom_ok = lambda nbytes, min_free_mb=0.0: True
        me._epipe_rs_demand_stage_gate_can_open = lambda *a, **k: True
        me._epipe_rs_demand_stage_gate_open = lambda *a, **k: True
        me._light_policy = None
        me._epipe_get_prefetch_pending_event = lambda eid: me._prefetch_events.get(int(eid), None)
        me._record_demand_h2d_window_begin = lambda *a, **k: None

        def load(eid):
            staged.append(int(eid))
            return ("w", int(eid)), 1000
        me._epipe_load_payload_to_device = load

        def compute(**kw):
            order.append(int(kw["eid"]))
            return torch.zeros_like(kw["cur"]), 0.0
        me._epipe_compute_segment = compute
        me._plain_ep_compute_segment = compute
        total = pos
        hidden = torch.zeros((total, 4))
        fn = (B._try_execute_local_recv_groups_epipe if scan == "upfront"
              else B._try_execute_local_recv_groups_epipe_rs_residual_scan)
        err = None
        try:
            res = fn(me, hidden_sorted=hidden, recv_i_sorted=torch.zeros(total, dtype=torch.long),
                     w_sorted=torch.ones(total), segments=list(segments), allow_nonlocal=False,
                     cp_cuda_timing=False, cp_sampled=False, cp_compute_events=[])
        except Exception as ex:          # noqa: BLE001
            res, err = None, type(ex).__name__ + ": " + str(ex)[:80]
        cases.append({"scan": scan, "segments": [[s[0], s[1], s[2]] for s in segments], "resident": resident,
                      "pending": pending, "capacity": cap, "fell_back": res is None, "order": order,
                      "staged": staged, "error": err})
    with open(os.path.join(HERE, "epipe_golden.json"), "w") as fh:
        json.dump(cases, fh, separators=(",", ":"))
    print("cases", len(cases), "triggered", sum(1 for c in cases if not c["fell_back"]),
          "errors", sum(1 for c in cases if c["error"]))
    for c in cases[:6]:
        print(c)


if __name__ == "__main__":
    main()
