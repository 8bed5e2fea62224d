"""One rank of the multi-GPU expert-parallel parity check (launched by
tests/test_gpu_ep.py through torch.distributed.run)."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from sparse_b200 import synth  # noqa: E402
from sparse_b200.block import B200MoeBlock  # noqa: E402
from sparse_b200.layer import LayerRunner, LayerWeights  # noqa: E402


class _RankEnv:
    def __init__(self, rank, world, dev):
        self.rank, self.world, self.local_rank, self.device = rank, world, dev.index, dev


def offloaded_case(rank, world, dev):
    """The reference-style block with expert_offload="cpu" under EP: owned experts
    in pinned host memory, 3 device slots per rank, rr and epipe settings.  Rows
    must equal the all-resident EP block bit for bit."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from test_gpu_cache import _Inner
    from sparse_b200.config import method_settings
    from sparse_b200.context import Metrics, SparseContext
    from sparse_b200.moe_block import DistributedSparseMoeBlock
    shape = synth.TINY
    w = synth.make_weights(shape, weight_seed=0, zipf_s=1.2)
    SparseContext.initialize(1, num_experts=shape.num_experts)

    def build(offload, cache, env_vars, metrics=None):
        old = dict(os.environ)
        os.environ.update(env_vars)
        try:
            return DistributedSparseMoeBlock(
                layer_idx=0, mlp_block=_Inner(w).to(torch.bfloat16), scp_map={}, env=_RankEnv(rank, world, dev),
                num_layers=1, num_experts=shape.num_experts, top_k=shape.top_k, dtype=torch.bfloat16,
                expert_offload=offload, expert_cache=cache, routing_mode="router", rs_dir="",
                rs_require_complete=False, rs_prob_to_logit_eps=1e-6, log_routing_stats=False, metrics=metrics,
                planner_mode="none", prefetch_top_m=2, placement_mode="round_robin", max_tokens=256,
                process_group=dist.group.WORLD)
        finally:
            os.environ.clear()
            os.environ.update(old)

    ref = build("gpu", 0, {})
    for method in ("rr", "epipe"):
        _, env_vars = method_settings(method, ep_size=world)
        metrics = Metrics()
        blk = build("cpu", 3, env_vars, metrics)
        assert blk.store is not None and blk._ep is not None and blk.store.cache.capacity == 3
        for step, tokens in enumerate((2, 2, 40, 2, 150, 1, 2)):
            SparseContext.current_phase = "decode" if tokens <= 2 else "prefill"
            SparseContext.begin_runtime_call(step)
            x = synth.make_hidden(tokens, shape.hidden, seed=300 + 7 * step + rank).to(torch.bfloat16)
            x = x.view(1, tokens, shape.hidden).to(dev) if tokens > 2 else x.view(tokens, 1, shape.hidden).to(dev)
            want, want_logits = ref(x)
            got, logits = blk(x)
            torch.cuda.synchronize()
            blk.check_status()
            ref.check_status()
            assert torch.equal(logits, want_logits)
            assert torch.equal(got, want), "offloaded EP rows differ (method %s step %d rank %d)" % (method, step, rank)
        assert metrics.cache_miss_count > 0 and len(blk.store.cache.resident_ids()) <= 3
        dist.barrier()


def local_cache_case(rank, world, dev):
    """Non-owned experts in local cache slots, filled from the owner GPU over
    NVLink: whatever runs locally and whatever goes to the owner, a decode-sized
    step gives the rows of the all-resident EP layer bit for bit, under every
    miss / late policy, with and without a prefetch plan."""
    from sparse_b200.context import Metrics
    from sparse_b200.peer_cache import LocalCacheEpLayer, build_rank_layer
    for shape_name, cache_slots in (("TINY", 2), ("QWEN_MOE", 6)):
        shape = getattr(synth, shape_name)
        w = synth.make_weights(shape, weight_seed=0, zipf_s=1.2)
        owner_of = [e % world for e in range(shape.num_experts)]
        ref = B200MoeBlock.from_block_weights(w, dev, ep_rank=rank, ep_size=world, max_tokens=16,
                                              process_group=dist.group.WORLD)
        lw, slab, owned, slot_at_owner = build_rank_layer(w, dev, rank, world, owner_of, cache_slots)
        slab.exchange(dist.group.WORLD)
        torch.cuda.synchronize()
        dist.barrier()                       # every owner's slab is loaded before anyone copies from it
        xs = [synth.make_hidden(4 if rank == 0 else 3, shape.hidden, seed=2100 + 10 * it + rank)
              .to(torch.bfloat16).to(dev) for it in range(6)]
        wants, chosen = [], []
        for x in xs:
            wants.append(ref.forward_device(x).clone())
            chosen.append(ref.topk(x.shape[0])[0].clone())
        torch.cuda.synchronize()
        ref.check_status()
        dist.barrier()
        total_local = 0
        for miss, late, prefetch in (("load", "wait", False), ("owner", "wait", False), ("load", "wait", True),
                                     ("owner", "owner", True)):
            metrics = Metrics()
            lay = LocalCacheEpLayer(lw, slab, owned, slot_at_owner, owner_of, shape.top_k, 16, rank, world,
                                    dist.group.WORLD, cache_slots, miss=miss, late=late, metrics=metrics)
            for it, x in enumerate(xs):
                lay.begin_step()
                if prefetch:
                    # a predictor that knows part of the truth: the experts of the step's first token
                    guess = {int(e): 1.0 for e in chosen[it][0].tolist()}
                    guess[(it * 3 + rank) % shape.num_experts] = 0.5
                    lay.prefetch(guess, budget=2)
                out = lay.forward(x).clone()
                torch.cuda.synchronize()
                lay.check_status()
                assert torch.equal(out, wants[it]), "local-cache EP rows differ (rank %d, %s/%s, step %d)" % (
                    rank, miss, late, it)
                assert len(lay.store.cache.resident_ids()) <= cache_slots
            if miss == "load":
                assert metrics.local_cached_item_count > 0 and metrics.expert_weight_peer_bytes > 0
            total_local += metrics.local_cached_item_count
            dist.barrier()
        assert total_local > 0
        del lay, ref
        torch.cuda.synchronize()
        dist.barrier()
        slab.close()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    for shape_name, tokens in (("TINY", 97 + 13 * rank), ("QWEN_MOE", 512)):
        shape = getattr(synth, shape_name)
        w = synth.make_weights(shape, weight_seed=0, zipf_s=1.2)
        blk = B200MoeBlock.from_block_weights(w, dev, ep_rank=rank, ep_size=world, max_tokens=tokens + 64,
                                              process_group=dist.group.WORLD)
        ref = LayerRunner(LayerWeights.from_block_weights(w, dev), shape.top_k, tokens)
        for it in range(3):          # several passes reuse the peer buffers
            x = synth.make_hidden(tokens, shape.hidden, seed=100 * it + rank).to(torch.bfloat16).to(dev)
            out = blk.forward_device(x).clone()
            want, want_idx, _, _ = ref.forward(x)
            torch.cuda.synchronize()
            blk.check_status()
            idx, _ = blk.topk(tokens)
            assert torch.equal(idx, want_idx), "indices differ on rank %d" % rank
            assert torch.equal(out, want), "EP rows differ from the single-GPU layer on rank %d" % rank
        # decode-sized steps (fused count exchange + plan, weight-streaming expert
        # kernels), eagerly and replayed from a captured CUDA graph
        t_small = 8 if rank % 2 == 0 else 5
        ref_small = LayerRunner(LayerWeights.from_block_weights(w, dev), shape.top_k, 16)
        xs = [synth.make_hidden(t_small, shape.hidden, seed=700 + 10 * it + rank).to(torch.bfloat16).to(dev)
              for it in range(3)]
        wants = [ref_small.forward(x)[0].clone() for x in xs]
        for it in range(3):
            out = blk.forward_device(xs[it]).clone()
            torch.cuda.synchronize()
            blk.check_status()
            assert torch.equal(out, wants[it]), "decode-sized EP rows differ on rank %d" % rank
        dist.barrier()
        x_static = xs[0].clone()
        out_static = torch.empty_like(x_static)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            blk.forward_device(x_static, out_static)
            with torch.cuda.graph(graph, stream=side):
                blk.forward_device(x_static, out_static)
        torch.cuda.current_stream(dev).wait_stream(side)
        for it in range(3):
            x_static.copy_(xs[it])
            graph.replay()
            torch.cuda.synchronize()
            blk.check_status()
            assert torch.equal(out_static, wants[it]), "graph-replayed EP rows differ on rank %d" % rank
        dist.barrier()
        # One step in which the ranks take different branches: rank 0 sends a
        # decode-sized batch, the others a prefill-sized one, so the decode-sized
        # rank receives expert groups far above 16 rows.  Eagerly and replayed.
        # A row may be computed by the streaming kernels on one rank and by the
        # tile kernel on another (fp32 summation order differs), so rows are
        # compared within the layer tolerance, not bit for bit.
        def close(a, b):
            a, b = a.double(), b.double()
            return float((a - b).norm() / b.norm()) < 5e-3 and float((a - b).abs().max()) < 2e-2

        t_mix = 8 if rank == 0 else 97
        ref_mix = LayerRunner(LayerWeights.from_block_weights(w, dev), shape.top_k, 128)
        xm = [synth.make_hidden(t_mix, shape.hidden, seed=1300 + 10 * it + rank).to(torch.bfloat16).to(dev)
              for it in range(2)]
        want_mix = [ref_mix.forward(x)[0].clone() for x in xm]
        for it in range(2):
            out = blk.forward_device(xm[it]).clone()
            torch.cuda.synchronize()
            blk.check_status()
            assert close(out, want_mix[it]), "mixed-branch EP rows differ on rank %d" % rank
        dist.barrier()
        blk.use_graphs = True
        for it in range(4):          # first use of each buffer records, later ones replay
            out = blk.forward_device(xm[it % 2]).clone()
            torch.cuda.synchronize()
            blk.check_status()
            assert close(out, want_mix[it % 2]), "graph-replayed mixed-branch rows differ on rank %d" % rank
        # the prefill-sized step through the block's own graph cache
        xg = [synth.make_hidden(tokens, shape.hidden, seed=1500 + 10 * it + rank).to(torch.bfloat16).to(dev)
              for it in range(2)]
        want_g = [ref.forward(x)[0].clone() for x in xg]
        for it in range(6):
            out = blk.forward_device(xg[it % 2]).clone()
            torch.cuda.synchronize()
            blk.check_status()
            assert torch.equal(out, want_g[it % 2]), "graph-replayed EP rows differ on rank %d (pass %d)" % (rank, it)
        blk.use_graphs = False
        dist.barrier()
        # the other step order (router beside the shared expert's gate/up pass instead
        # of in front of it) gives the same rows
        ep_layer = getattr(blk, "_ep", None) or getattr(blk, "ep_layer", None)
        if ep_layer is not None and hasattr(ep_layer, "router_first"):
            ep_layer.router_first = not ep_layer.router_first
            for it in range(2):
                out = blk.forward_device(xg[it]).clone()
                torch.cuda.synchronize()
                blk.check_status()
                assert torch.equal(out, want_g[it]), "rows differ with the other router order on rank %d" % rank
            ep_layer.router_first = not ep_layer.router_first
            dist.barrier()
    offloaded_case(rank, world, dev)
    local_cache_case(rank, world, dev)
    print("EP_WORKER_OK rank %d" % rank, flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
