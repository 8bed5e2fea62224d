"""Generate expert-parallel golden vectors by running the REFERENCE's own EP path.

    python tests/golden/make_ep_golden.py --reference <checkout of louislichen/SPARSE>

Spawns `world` CPU processes with a gloo process group (the pattern of the
reference's tests/test_lightweight_policy.py:91-127), builds the reference's
unmodified `DistributedSparseMoeBlock` on every rank with a real
`DistTopology` (utils/eval_core.py:188-222) and round-robin ownership, and runs
one forward per rank on that rank's own tokens, so that the block takes
`_experts_ep_group` (utils/eval_core.py:14865-15060): dispatch all-to-all,
local sorted-segment executor, return all-to-all, unsort, combine.  Stored per
rank: the expert ids of the received rows in arrival order (`recv_i`, captured
at the call of `_execute_local_recv_groups`), the per-destination send counts,
the top-k indices, the router logits and the block's output rows.

Weights and inputs are re-drawn from the seeds of `sparse_b200.synth`; the
fixtures hold outputs only.  The reference cannot travel to the GPU box; these
files can.
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile
from datetime import timedelta

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

from sparse_b200 import synth  # noqa: E402

# name -> (shape, zipf_s, dtype, tokens per rank, input seed)
CASES = {
    "ep2_tiny_bf16": ("TINY", 1.2, "bfloat16", [70, 33], 5),
    "ep4_tiny_bf16": ("TINY", 1.2, "bfloat16", [5, 0, 130, 64], 5),
    "ep2_tiny_fp32": ("TINY", 0.0, "float32", [41, 23], 6),
    "ep4_qwen_bf16": ("QWEN_MOE", 1.2, "bfloat16", [64, 17, 40, 7], 8),
}


def _bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


def worker(rank: int, world: int, rendezvous: str, reference: str, name: str, out_dir: str) -> None:
    sys.path.insert(0, reference)
    import utils.eval_core as ec
    from make_golden import _InnerBlock
    dist.init_process_group("gloo", init_method=rendezvous, rank=rank, world_size=world,
                            timeout=timedelta(seconds=300))
    try:
        shape_name, zipf_s, dtype_name, tokens, seed = CASES[name]
        dtype = getattr(torch, dtype_name)
        shape = getattr(synth, shape_name)
        torch.set_num_threads(max(1, (os.cpu_count() or 2) // world))
        w = synth.make_weights(shape, weight_seed=0, zipf_s=zipf_s)
        env = ec.DistEnv(rank=rank, world=world, local_rank=rank, device=torch.device("cpu"))
        topo = ec.build_dist_topology(env, "baseline", world)
        ec.SparseContext.initialize(1, num_experts=shape.num_experts)
        inner = _InnerBlock(w, qwen_style=shape.shared_gate).to(dtype)
        blk = ec.DistributedSparseMoeBlock(
            layer_idx=0, mlp_block=inner, scp_map={}, env=env, num_layers=1, num_experts=shape.num_experts,
            top_k=shape.top_k, dtype=dtype, expert_offload="gpu", expert_cache=0, routing_mode="router",
            rs_dir="", rs_require_complete=False, rs_prob_to_logit_eps=1e-6, log_routing_stats=False,
            placement_mode="round_robin", topology=topo)
        blk.eval()
        seen = {}
        inner_exec = blk._execute_local_recv_groups

        def spy(recv_hidden, recv_i, recv_w, **kw):
            seen["recv_i"] = recv_i.clone()
            seen["recv_w"] = recv_w.clone()
            return inner_exec(recv_hidden, recv_i, recv_w, **kw)

        blk._execute_local_recv_groups = spy
        inner_route = blk._routing_router

        def spy_route(x2):
            res = inner_route(x2)
            seen["route"] = res
            return res

        blk._routing_router = spy_route
        x_all = synth.make_hidden(sum(tokens), shape.hidden, seed=seed).to(dtype)
        x = list(torch.split(x_all, tokens))[rank].contiguous()
        with torch.no_grad():
            res = blk(x.view(1, x.shape[0], shape.hidden))
        out = res[0] if isinstance(res, tuple) else res
        logits = res[1] if isinstance(res, tuple) else torch.zeros((x.shape[0], shape.num_experts), dtype=dtype)
        topv, topi = seen["route"][0], seen["route"][1]
        recv_i = seen.get("recv_i", torch.zeros((0,), dtype=torch.long))
        owner = torch.tensor([e % world for e in range(shape.num_experts)])
        send_counts = torch.bincount(owner[topi.reshape(-1).long()], minlength=world)
        np.savez_compressed(
            os.path.join(out_dir, "%s_rank%d.npz" % (name, rank)),
            shape=shape_name, dtype=dtype_name, zipf_s=zipf_s, input_seed=seed, world=world, rank=rank,
            tokens=np.asarray(tokens, dtype=np.int64),
            recv_i=recv_i.numpy().astype(np.int16), send_counts=send_counts.numpy().astype(np.int64),
            topi=topi.reshape(x.shape[0], shape.top_k).numpy().astype(np.int16),
            topv=_bits(topv.reshape(x.shape[0], shape.top_k).to(dtype)),
            logits=_bits(logits.reshape(x.shape[0], shape.num_experts).to(dtype)),
            out=_bits(out.reshape(x.shape[0], shape.hidden).to(dtype)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--only", default="")
    a = ap.parse_args()
    for name, case in CASES.items():
        if a.only and a.only != name:
            continue
        world = len(case[3])
        with tempfile.TemporaryDirectory() as tmp:
            rendezvous = "file://" + os.path.join(tmp, "rendezvous")
            mp.spawn(worker, args=(world, rendezvous, os.path.abspath(a.reference), name, HERE), nprocs=world,
                     join=True)
        print("wrote", name)


if __name__ == "__main__":
    main()
