"""CPU: prefetch planner and RS checkpoint loader.

The planner is replayed on cases recorded from the reference's own planner
methods (tests/golden/planner_golden.json); the loader is fed checkpoints
synthesised in the reference's payload format
(scripts/train_next_layer_rs.py:603-630 of the reference)."""
import json
import os

import pytest
import torch

from conftest import GOLDEN_DIR
from sparse_b200 import rs
from sparse_b200.cache import ExpertWeightCache
from sparse_b200.config import BlockConfig, block_config_from_env, cache_capacity_for_rank, method_settings


def test_planner_matches_reference_cases():
    with open(os.path.join(GOLDEN_DIR, "planner_golden.json")) as fh:
        cases = json.load(fh)
    for c in cases:
        local = set(c["local"])
        cache = ExpertWeightCache(c["capacity"])
        for e, pinned in c["setup"]:
            cache.put(e, "w", pinned=pinned)
        freq = {int(k): v for k, v in c["freq"].items()}
        prefetched = set(c["prefetched"])
        counters = {}
        note = lambda name, value=1: counters.__setitem__(name, counters.get(name, 0) + int(value))

        def keep_bias(e):
            return 0.02 * float(min(freq.get(e, 0), 16)) + (0.10 if e in prefetched else 0.0)

        smap = rs.prob_score_map(torch.tensor(c["topi"]), torch.tensor(c["topv"]), lambda e: e in local, note)
        want_map = {int(k): v for k, v in c["score_map"].items()}
        assert list(smap) == list(want_map)
        for k in smap:
            assert smap[k] == pytest.approx(want_map[k], rel=1e-12, abs=1e-15)
        cfg = BlockConfig(rs_prefetch_policy=c["policy"], min_cand_score=c["min_score"],
                          replace_advantage=c["adv"], replace_margin=c["margin"])
        lo, adv, mar = cfg.effective_planner_thresholds()
        plan = rs.build_prefetch_plan(smap, cache, protect_ids=set(c["protect"]), budget=c["budget"],
                                      min_score=lo, replace_advantage=adv, replace_margin=mar,
                                      allow_active_replace=c["active"], is_local=lambda e: e in local,
                                      keep_bias=keep_bias, counters=note)
        assert [[e, v] for e, v in plan] == c["plan"], c
        assert counters == c["counters"], c


def _residual_payload(hidden, experts, hid, blocks, target):
    torch.manual_seed(target)
    mod = rs.RoutingScoutResidualMLP(hidden, experts, hid, blocks, 0.05)
    return {"model_type": "next_layer_residual_logits_rs", "task": "router_prob",
            "state_dict": mod.state_dict(), "input_dim": hidden, "hidden_dim": hid,
            "num_hidden_layers": blocks, "num_experts": experts, "source_layer": target - 1,
            "target_layer": target, "lead_layers": 1, "top_k": 4, "label_type": "router_prob",
            "feature_mode": "hidden"}, mod


def test_rs_bank_loader_next_layer_layout(tmp_path):
    hidden, experts, layers = 32, 8, 4
    mods = {}
    for t in (2, 3):
        payload, mods[t] = _residual_payload(hidden, experts, 16, 2, t)
        torch.save(payload, tmp_path / ("rs_l%d_inL%d.pth" % (t, t - 1)))
    bank, task, layout, sources, missing = rs.load_rs_bank(str(tmp_path), layers, hidden, experts,
                                                            torch.device("cpu"), require_complete=True)
    assert (task, layout, len(bank)) == ("router_prob", "next_layer", layers)
    assert sources == [-1, 0, 1, 2] and missing == []       # layers before the first target are optional
    x = torch.randn(5, hidden)
    for t in (2, 3):
        assert isinstance(bank[t], rs.RoutingScoutResidualMLP)
        want = mods[t].eval()(x)
        assert torch.equal(bank[t](x), want)
        assert torch.allclose(want.sum(-1), torch.ones(5), atol=1e-5)
    assert isinstance(bank[0], rs.RoutingScoutMLP)
    os.remove(tmp_path / "rs_l3_inL2.pth")
    with pytest.raises(RuntimeError, match="incomplete"):
        rs.load_rs_bank(str(tmp_path), layers, hidden, experts, torch.device("cpu"), require_complete=True)
    bank2, _, _, _, missing2 = rs.load_rs_bank(str(tmp_path), layers, hidden, experts, torch.device("cpu"),
                                               require_complete=False)
    assert len(bank2) == layers and len(missing2) == 1
    keys = set(mods[2].state_dict())
    assert {"input.0.weight", "input.1.weight", "blocks.0.net.0.weight", "blocks.0.net.1.weight",
            "blocks.1.net.4.bias", "out_norm.weight", "head.weight"} <= keys


def test_block_config_from_method_table():
    for method, (placement, planner, epipe, rs_mode, exec_mode) in {
        "rr": ("round_robin", "none", False, "off", "unique_mask"),
        "scp": ("scp_ep", "none", False, "off", "unique_mask"),
        "rs": ("round_robin", "rs_prefetch", False, "off", "unique_mask"),
        "epipe": ("round_robin", "none", True, "off", "sorted_segment"),
        "scp-rs": ("scp_ep", "rs_prefetch", False, "off", "unique_mask"),
        "rs-epipe": ("round_robin", "rs_prefetch", True, "residual_scan", "sorted_segment"),
        "sparse": ("scp_ep", "rs_prefetch", True, "residual_scan", "sorted_segment"),
        "executor-no-epipe": ("scp_ep", "rs_prefetch", False, "off", "sorted_segment"),
        "executor-with-epipe": ("scp_ep", "rs_prefetch", True, "residual_scan", "sorted_segment"),
    }.items():
        flags, env = method_settings(method, ep_size=4)
        assert flags["--placement-mode"] == placement and flags["--planner-mode"] == planner
        cfg = block_config_from_env(env, rank=1, prefetch_top_m=4)
        assert cfg.epipe_enable is epipe and cfg.epipe_decode_rs_mode == rs_mode
        assert cfg.plain_exec_mode == exec_mode
        assert cfg.scp_apply_prefill is (placement == "scp_ep") and cfg.scp_apply_decode is False
        assert cfg.top_m == 2 and cfg.pred_topk == 4
        assert cfg.effective_planner_thresholds() == (0.04, 0.08, 1.20)
        assert cfg.epipe_handle_demand_miss is epipe
    with pytest.raises(ValueError):
        method_settings("nope")
    with pytest.raises(NotImplementedError):
        block_config_from_env({"SPARSE_PREFILL_EXPERT_MATH": "fixed64"})
    assert cache_capacity_for_rank({"SPARSE_EXPERT_CACHE_BY_RANK": "8,6,4,2"}, 10, 2) == 4
    assert cache_capacity_for_rank({"SPARSE_EXPERT_CACHE_BY_RANK": "0:3,2:5"}, 10, 1) == 10
    assert cache_capacity_for_rank({}, 10, 1) == 10
