"""CPU, 2 gloo ranks: the host-side logic of the expert-parallel path.

The device kernels cannot run here; what is checked is everything around them:
the receive-buffer layout formula (host mirror of `sb_ep_plan`) against the
oracle's EP simulation, with counts and rows really exchanged between two
processes, and the handle exchange used to map peer buffers."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _worker(rank, world, init_file, result_file):
    import sys
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from datetime import timedelta
    dist.init_process_group("gloo", init_method="file://" + init_file, rank=rank, world_size=world,
                            timeout=timedelta(seconds=60))
    try:
        from oracle import moe_oracle as mo
        from sparse_b200 import synth
        from sparse_b200.ep import plan_layout_reference, PeerBuffers, exchange_handles
        shape = synth.TINY
        w = synth.make_weights(shape, weight_seed=0, zipf_s=1.2)
        cw = mo.cast_weights(w, torch.bfloat16)
        x_all = synth.make_hidden(90, shape.hidden, seed=5).to(torch.bfloat16)
        xs = list(torch.tensor_split(x_all, world))
        x = xs[rank]
        e, k = shape.num_experts, shape.top_k
        owner = mo.round_robin_owner(e, world)
        logits = mo.router_logits_fixed_order(x, cw["router"], cw["router_bias"])
        topv, topi = mo.softmax_topk(logits, k, False, x.dtype)
        flat = topi.reshape(-1)
        slot_of_item, item_of_slot, local_off = mo.expert_sorted_permutation(topi, e)
        counts = (local_off[1:] - local_off[:-1]).contiguous()
        gathered = [torch.zeros_like(counts) for _ in range(world)]
        dist.all_gather(gathered, counts)
        counts_all = torch.stack(gathered)
        dst_base, recv_offsets, seg_begin = plan_layout_reference(counts_all, owner, rank)
        assert seg_begin.shape == (world, e)
        # where every local item goes
        item_row = dst_base[flat] + (slot_of_item - local_off[flat])
        item_rank = owner[flat]
        # move (expert id, source rank, source item) records with a real all-to-all
        recs = torch.stack([flat, torch.full_like(flat, rank), torch.arange(flat.numel()), item_row], 1)
        send = [recs[item_rank == d].contiguous() for d in range(world)]
        send_n = torch.tensor([s.shape[0] for s in send])
        recv_n = torch.zeros_like(send_n)
        dist.all_to_all_single(recv_n, send_n)
        got = torch.zeros((int(recv_n.sum()), 4), dtype=recs.dtype)
        dist.all_to_all_single(got, torch.cat(send), output_split_sizes=recv_n.tolist(),
                               input_split_sizes=send_n.tolist())
        total = int(recv_offsets[-1])
        assert got.shape[0] == total
        placed = torch.full((total, 3), -1, dtype=torch.long)
        placed[got[:, 3]] = got[:, :3]
        assert int((placed[:, 0] < 0).sum()) == 0, "every receive row is written exactly once"
        assert int(got[:, 3].unique().numel()) == total
        # rows arrive sorted by expert id, then source rank, then source item order
        key = placed[:, 0] * 10 ** 8 + placed[:, 1] * 10 ** 5 + placed[:, 2]
        assert bool((key[1:] > key[:-1]).all())
        for ex in range(e):
            seg = placed[recv_offsets[ex]:recv_offsets[ex + 1], 0]
            assert bool((seg == ex).all())
            if int(owner[ex]) != rank:
                assert seg.numel() == 0
        # same multiset of expert ids as the oracle's simulation of this rank
        sim = mo.ep_block_forward(xs, cw, k, owner)
        assert torch.equal(placed[:, 0], sim[rank]["recv_i"].sort(stable=True).values)

        # handle exchange with a stand-in exporter (no CUDA here)
        bufs = PeerBuffers(shape.hidden, e, 256, world, rank)
        bufs.export_handles = lambda: bytes([rank]) * 256
        seen = {}
        bufs.import_handles = lambda peer, blob: seen.__setitem__(peer, blob)
        exchange_handles(bufs, None)
        assert sorted(seen) == [p for p in range(world) if p != rank]
        assert all(v == bytes([p]) * 256 for p, v in seen.items())
        with open(result_file + str(rank), "w") as fh:
            fh.write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_ep_layout_and_exchange_two_gloo_ranks():
    world = 2
    with tempfile.TemporaryDirectory() as d:
        init_file = os.path.join(d, "rdzv")
        result = os.path.join(d, "res")
        mp.spawn(_worker, args=(world, init_file, result), nprocs=world, join=True)
        for r in range(world):
            assert open(result + str(r)).read() == "ok"


def test_plan_reference_small_known_answer():
    from sparse_b200.ep import plan_layout_reference
    counts = torch.tensor([[2, 0, 1, 3], [1, 4, 0, 2]])
    owner = torch.tensor([0, 1, 0, 1])
    d0, r0, s0 = plan_layout_reference(counts, owner, 0)
    d1, r1, s1 = plan_layout_reference(counts, owner, 1)
    assert s0[0].tolist() == [0, 3, 3, 4] and s0[1].tolist() == [0, 0, 4, 4]
    assert d0.tolist() == [0, 0, 3, 4]
    assert d1.tolist() == [2, 0, 4, 7]
    assert r0.tolist() == [0, 3, 3, 4, 4]
    assert r1.tolist() == [0, 0, 4, 4, 9]
