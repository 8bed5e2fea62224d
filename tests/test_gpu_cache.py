"""GPU: offloaded experts, LRU slots, prefetch planner, EPIPE ordering and the
bounded stager.  Whatever the residency machinery does, a layer's output must be
bit-identical to the all-resident layer."""
import os

import pytest
import torch
import torch.nn as nn

from conftest import block_weights
from sparse_b200 import synth

pytestmark = pytest.mark.gpu


class _MLP(nn.Module):
    def __init__(self, g, u, d):
        super().__init__()
        i, h = g.shape
        self.gate_proj, self.up_proj, self.down_proj = nn.Linear(h, i, bias=False), nn.Linear(h, i, bias=False), nn.Linear(i, h, bias=False)
        self.act_fn = nn.SiLU()
        with torch.no_grad():
            self.gate_proj.weight.copy_(g); self.up_proj.weight.copy_(u); self.down_proj.weight.copy_(d)


class _Inner(nn.Module):
    def __init__(self, w):
        super().__init__()
        s = w.shape
        self.gate = nn.Linear(s.hidden, s.num_experts, bias=w.router_bias is not None)
        with torch.no_grad():
            self.gate.weight.copy_(w.router)
            if w.router_bias is not None:
                self.gate.bias.copy_(w.router_bias)
        self.experts = nn.ModuleList([_MLP(w.gate[e], w.up[e], w.down[e]) for e in range(s.num_experts)])
        self.shared_expert = _MLP(w.sh_gate, w.sh_up, w.sh_down)
        self.shared_expert_gate = nn.Linear(s.hidden, 1, bias=False)
        with torch.no_grad():
            self.shared_expert_gate.weight.copy_(w.sh_scalar_gate)
        self.norm_topk_prob = False


class _Env:
    def __init__(self):
        self.rank, self.world, self.local_rank, self.device = 0, 1, 0, torch.device("cuda:0")


def _make_block(w, layer_idx=0, num_layers=1, offload="gpu", cache=0, planner="none", env=None, metrics=None):
    from sparse_b200.moe_block import DistributedSparseMoeBlock
    old = dict(os.environ)
    os.environ.update(env or {})
    try:
        return DistributedSparseMoeBlock(
            layer_idx=layer_idx, mlp_block=_Inner(w).to(torch.bfloat16), scp_map={}, env=_Env(),
            num_layers=num_layers, num_experts=w.shape.num_experts, top_k=w.shape.top_k, dtype=torch.bfloat16,
            expert_offload=offload, expert_cache=cache, routing_mode="router", rs_dir="", rs_require_complete=False,
            rs_prob_to_logit_eps=1e-6, log_routing_stats=False, metrics=metrics, planner_mode=planner,
            prefetch_top_m=2, placement_mode="round_robin", max_tokens=256)
    finally:
        os.environ.clear()
        os.environ.update(old)


def _tokens(step, n, hidden):
    return synth.make_hidden(n, hidden, seed=1000 + step).to(torch.bfloat16).view(n, 1, hidden).cuda()


@pytest.mark.parametrize("method", ["rr", "epipe"])
def test_offloaded_layer_equals_resident_layer(method):
    from sparse_b200.config import method_settings
    from sparse_b200.context import Metrics, SparseContext
    w = block_weights("TINY", 1.2)
    SparseContext.initialize(1, num_experts=w.shape.num_experts)
    ref = _make_block(w, offload="gpu")
    _, env = method_settings(method, ep_size=1)
    metrics = Metrics()
    blk = _make_block(w, offload="cpu", cache=3, env=env, metrics=metrics)
    assert blk.store is not None and blk.store.cache.capacity == 3
    SparseContext.current_phase = "decode"
    triggered = 0
    for step in range(12):
        SparseContext.begin_runtime_call(step)
        x = _tokens(step, 2, w.shape.hidden)
        want, want_logits = ref(x)
        got, logits = blk(x)
        torch.cuda.synchronize()
        blk.check_status()
        assert torch.equal(logits, want_logits)
        assert torch.equal(got, want), "step %d" % step
        if blk._cached.last_plan is not None:
            triggered += 1
            assert len(blk._cached.last_plan.first) >= 1
    assert metrics.cache_miss_count > 0 and metrics.expert_weight_h2d_demand_bytes > 0
    assert len(blk.store.cache.resident_ids()) <= 3
    if method == "epipe":
        assert triggered > 0 and metrics.epipe_staged_expert_count == triggered
        assert metrics.epipe_attempt_count == 12
    else:
        assert triggered == 0
    # prefill-sized call through the same block
    SparseContext.current_phase = "prefill"
    x = synth.make_hidden(150, w.shape.hidden, seed=9).to(torch.bfloat16).view(1, 150, -1).cuda()
    want, _ = ref(x)
    blk2 = _make_block(w, offload="cpu", cache=w.shape.num_experts - 1, env=env)
    got, _ = blk2(x)
    assert torch.equal(got, want)


def _install_rs_bank(w, num_layers, overlap=0.7):
    """Synthetic predictor: for target layer t it emits a fixed distribution that
    favours a seeded subset of experts (stands in for a trained RS checkpoint)."""
    from sparse_b200 import rs
    from sparse_b200.context import SparseContext
    torch.manual_seed(3)
    bank = nn.ModuleList([rs.RoutingScoutResidualMLP(w.shape.hidden, w.shape.num_experts, 32, 1).cuda().float().eval()
                          for _ in range(num_layers)])
    SparseContext.rs_bank = bank
    SparseContext.rs_bank_source_layers = list(range(-1, num_layers - 1))
    return bank


def test_rs_prefetch_and_sparse_modes_keep_outputs_identical():
    from sparse_b200.config import method_settings
    from sparse_b200.context import Metrics, SparseContext
    w = block_weights("TINY", 1.2)
    layers = 3
    for method in ("rs", "rs-epipe"):
        SparseContext.initialize(layers, num_experts=w.shape.num_experts)
        _, env = method_settings(method, ep_size=1)
        env["SPARSE_RS_CACHE_SAFE_MIN_SCORE_BY_RANK"] = "0.0"
        env["SPARSE_PREFETCH_MIN_CAND_SCORE"] = "0.0"
        metrics = Metrics()
        refs = [_make_block(w, layer_idx=l, num_layers=layers) for l in range(layers)]
        blks = [_make_block(w, layer_idx=l, num_layers=layers, offload="cpu", cache=3, planner="rs_prefetch",
                            env=env, metrics=metrics) for l in range(layers)]
        for l, b in enumerate(blks):
            SparseContext.register_layer_block(l, b)
        _install_rs_bank(w, layers)
        SparseContext.current_phase = "decode"
        for step in range(10):
            SparseContext.begin_runtime_call(step)
            x = _tokens(step, 1, w.shape.hidden)
            for l in range(layers):
                want, _ = refs[l](x)
                got, _ = blks[l](x)
                assert torch.equal(got, want), (method, step, l)
                x = (x + got).contiguous()
        torch.cuda.synchronize()
        assert metrics.prefetch_issued_count > 0 and metrics.prefetch_admitted_count > 0
        assert metrics.expert_weight_h2d_prefetch_bytes > 0
        assert metrics.rs_counters.get("rs_pred_candidate_count", 0) > 0


def test_bounded_stager_commits_used_transfers_by_slot_exchange():
    from sparse_b200.bounded import BoundedStager
    from sparse_b200.config import method_settings
    from sparse_b200.context import Metrics, SparseContext
    w = block_weights("TINY", 1.2)
    layers = 3
    SparseContext.initialize(layers, num_experts=w.shape.num_experts)
    _, env = method_settings("rs", ep_size=1)
    env.update({"SPARSE_B200_RS_STAGING_SLOTS": "4", "SPARSE_RS_CACHE_SAFE_MIN_SCORE_BY_RANK": "0.0",
                "SPARSE_PREFETCH_MIN_CAND_SCORE": "0.0"})
    metrics = Metrics()
    refs = [_make_block(w, layer_idx=l, num_layers=layers) for l in range(layers)]
    blks = {l: _make_block(w, layer_idx=l, num_layers=layers, offload="cpu", cache=3, env=env, metrics=metrics)
            for l in range(layers)}
    for l, b in blks.items():
        SparseContext.register_layer_block(l, b)
        b.planner_mode = "none"               # the stager drives prediction, not the in-line planner
    _install_rs_bank(w, layers)
    stager = BoundedStager(blks, slots=4)
    stager.install(batch=1)
    SparseContext.current_phase = "decode"
    try:
        for step in range(10):
            SparseContext.begin_runtime_call(step)
            x = _tokens(step, 1, w.shape.hidden)
            for l in range(layers):
                stager.predict(l, x.view(1, -1))
                if l > 0:
                    import time
                    time.sleep(0.002)          # give the worker a chance to publish before demand closes the job
                stager.activate(l)
                want, _ = refs[l](x)
                got, _ = blks[l](x)
                stager.release(l)
                assert torch.equal(got, want), (step, l)
                x = (x + got).contiguous()
        stats = stager.finish()
    finally:
        stager.close()
    assert stats["predictions"] > 0 and stats["issued"] > 0
    assert stats["used"] + stats["wasted"] == stats["issued"]
    assert stats["retained"] == stats["used"]
    for l in range(layers):
        st = blks[l].store
        slots = [st.cache.peek(e) for e in st.cache.resident_ids()]
        assert len(set(slots)) == len(slots), "two residents share a slab slot"
        assert st.view is None


class _FusedExperts(nn.Module):
    """Experts as two 3-D parameters, the layout the reference's fused-weight
    path reads (utils/eval_core.py:11714-11731): gate_up_proj [E, 2I, H] with the
    I gate rows first, down_proj [E, H, I]."""

    def __init__(self, w):
        super().__init__()
        gu = torch.stack([torch.cat([w.gate[e], w.up[e]], dim=0) for e in range(w.shape.num_experts)])
        dn = torch.stack([w.down[e] for e in range(w.shape.num_experts)])
        self.gate_up_proj = nn.Parameter(gu, requires_grad=False)
        self.down_proj = nn.Parameter(dn, requires_grad=False)
        self.act_fn = nn.SiLU()


@pytest.mark.parametrize("offload", ["gpu", "cpu"])
def test_fused_gate_up_layout_equals_module_list_layout(offload):
    """The same weights handed over as fused 3-D parameters give the bits of the
    per-expert module list, resident and offloaded."""
    from sparse_b200.context import SparseContext
    w = block_weights("TINY", 1.2)
    SparseContext.initialize(1, num_experts=w.shape.num_experts)
    ref = _make_block(w, offload="gpu")
    from sparse_b200.moe_block import DistributedSparseMoeBlock
    inner = _Inner(w)
    inner.experts = _FusedExperts(w)
    blk = DistributedSparseMoeBlock(
        layer_idx=0, mlp_block=inner.to(torch.bfloat16), scp_map={}, env=_Env(), num_layers=1,
        num_experts=w.shape.num_experts, top_k=w.shape.top_k, dtype=torch.bfloat16, expert_offload=offload,
        expert_cache=3 if offload == "cpu" else 0, routing_mode="router", rs_dir="", rs_require_complete=False,
        rs_prob_to_logit_eps=1e-6, log_routing_stats=False, planner_mode="none", prefetch_top_m=2,
        placement_mode="round_robin", max_tokens=256)
    assert (blk.store is not None) == (offload == "cpu")
    for step, n in enumerate((1, 7, 130)):
        SparseContext.begin_runtime_call(step)
        x = synth.make_hidden(n, w.shape.hidden, seed=2000 + step).to(torch.bfloat16).view(1, n, -1).cuda()
        want, want_logits = ref(x)
        got, logits = blk(x)
        torch.cuda.synchronize()
        blk.check_status()
        assert torch.equal(logits, want_logits)
        assert torch.equal(got, want)
