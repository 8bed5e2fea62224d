#!/usr/bin/env python
"""MoE-layer throughput on B200: tokens/s through one Qwen1.5-MoE-shaped block.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the MoE layer hot path (router top-k -> expert-sorted
permute -> grouped SwiGLU GEMMs for routed and shared experts -> combine) over
one batch of synthetic tokens.  Workload at every N: per GPU 4096 tokens of
hidden states ~N(0,1) in bf16, weights N(0,0.02) seed 0, router bias
log Zipf(1.2) over a seeded expert permutation (weak scaling; at N>1 the 60
experts are sharded over the N GPUs -- by default with a load-balanced
replicated placement derived from a calibration batch, `--placement rr` for
round-robin -- and rows travel over NVLink peer memory).

Prints ONE JSON line (rank 0).  `value` is device-timed with inputs resident in
HBM; `e2e` goes through the block-level host API (`HostPipeline`) with pinned
HOST buffers, every step's host->device and device->host copies inside the
timed region.  `roofline`
describes the dominant kernel (the grouped tcgen05 GEMM, tensor-bound at this
size); `stages` breaks a step into its kernels with achieved HBM GB/s for the
memory-bound ones.  `--impl reference` times the CPU restatement of the
reference block on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch

TOKENS_PER_GPU = 4096
ZIPF_S = 1.2
WORKLOAD = "qwen1.5-moe-a2.7b-shaped MoE block, bf16, %d tokens/GPU, zipf(1.2) router bias" % TOKENS_PER_GPU
CPU_SAMPLE_TOKENS = 512
N_INPUT_BATCHES = 4          # rotated so a step never re-reads the previous step's activations

# dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernel
# (pair_gemm_kernel), averaged over the four launches of one step (routed
# gate/up 737.1 MB, routed down 412.4 MB, shared gate/up 105.7 MB, shared down
# 74.9 MB = 1330.1 MB per step), from one `ncu --set full` capture of this
# workload on a B200 (2026-11-25).  The algorithmic bytes of the same four
# launches are 1355.8 MB: nothing is re-read from DRAM.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 332530368


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.01)

    def start(self):
        if self._nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()

    def stop(self):
        self._stop.set()
        if self._thr is not None:
            self._thr.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                    "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def _physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# ------------------------------------------------------------------ CPU arm ----

def cpu_reference_tokens_per_s(steps: int, warmup: int):
    """The reference block's CPU path (fp32, world=1) restated by the oracle,
    on all host cores, over a bounded sample of the workload."""
    from oracle import moe_oracle as mo
    from sparse_b200 import synth
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    shape = synth.QWEN_MOE
    w = synth.make_weights(shape, weight_seed=0, zipf_s=ZIPF_S)
    cw = mo.cast_weights(w, torch.float32)
    x = synth.make_hidden(TOKENS_PER_GPU, shape.hidden, seed=1)[:CPU_SAMPLE_TOKENS].contiguous()
    with torch.no_grad():
        for _ in range(max(1, warmup)):
            mo.moe_block_forward(x, cw, shape.top_k, router="library")
        t0 = time.perf_counter()
        for _ in range(max(1, steps)):
            mo.moe_block_forward(x, cw, shape.top_k, router="library")
        dt = time.perf_counter() - t0
    per_step = dt / max(1, steps)
    return CPU_SAMPLE_TOKENS / per_step, per_step * 1e3, torch.get_num_threads()


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, args.steps)
    warmup = max(3, args.warmup)
    tps, ms, cores = cpu_reference_tokens_per_s(steps, warmup)
    sample = ("each step = the first %d of the %d tokens of a batch, fp32, all host threads; "
              "%d steps after %d warm-up steps" % (CPU_SAMPLE_TOKENS, TOKENS_PER_GPU, steps, warmup))
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(max(1, args.gpus), "n/a (host cores)"),
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def workload_config(world, placement_note):
    """The `config` object of the JSON line (both arms print the same one)."""
    from sparse_b200 import synth
    shape = synth.QWEN_MOE
    return {"workload": WORKLOAD, "tokens_per_gpu": TOKENS_PER_GPU, "experts": shape.num_experts,
            "top_k": shape.top_k, "hidden": shape.hidden, "inter": shape.inter,
            "shared_inter": shape.shared_inter,
            "parallelism": "ep%d" % world if world > 1 else "ep1",
            "placement": placement_note,
            "l2": "weights 1.1 GB per layer exceed the 126 MB L2; %d input batches rotated" % N_INPUT_BATCHES}


# ------------------------------------------------------------------ GPU arm ----

def _time_steps(fn, steps, stream):
    """Like _time_region, with an event after every step: (total ms, per-step ms list)."""
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    evs[0].record(stream)
    for i in range(steps):
        fn(i)
        evs[i + 1].record(stream)
    evs[-1].synchronize()
    per = [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]
    return evs[0].elapsed_time(evs[-1]), per


def _step_stats(per):
    s = sorted(per)
    n = len(s)
    head = per[:min(10, n)]
    return {"min": s[0], "median": s[n // 2], "p90": s[min(n - 1, int(0.9 * n))], "max": s[-1],
            "first_10_mean": sum(head) / len(head)}


def torch_eager_tokens_per_s(w, shape, x, steps=5):
    """The reference block's own op sequence (library GEMMs: F.linear per expert,
    softmax, torch.topk, index_add_ in ascending expert order;
    utils/eval_core.py:9519-9595, 14690-14721, 9455-9463 of the reference) run
    eagerly on this GPU in bf16: the cuBLAS/ATen bar the hand-written kernels
    have to beat on the same box.  Not used for any parity claim."""
    import torch.nn.functional as F
    dev = x.device
    bf = torch.bfloat16
    router = w.router.to(bf).to(dev)
    rbias = None if w.router_bias is None else w.router_bias.to(bf).to(dev)
    gate = [g.to(bf).to(dev) for g in w.gate]
    up = [u.to(bf).to(dev) for u in w.up]
    down = [d.to(bf).to(dev) for d in w.down]
    sg, su, sd = w.sh_gate.to(bf).to(dev), w.sh_up.to(bf).to(dev), w.sh_down.to(bf).to(dev)
    ssg = w.sh_scalar_gate.to(bf).to(dev)

    def forward(xx):
        logits = F.linear(xx, router, rbias)
        probs = torch.softmax(logits, dim=-1, dtype=torch.float32)
        topv, topi = torch.topk(probs, shape.top_k, dim=-1)
        topv = topv.to(xx.dtype)
        out = torch.zeros_like(xx)
        mask = F.one_hot(topi, num_classes=shape.num_experts).permute(2, 1, 0)
        for e in range(shape.num_experts):
            idx_k, top_x = torch.where(mask[e])
            if top_x.numel() == 0:
                continue
            cur = xx[top_x]
            y = F.linear(F.silu(F.linear(cur, gate[e])) * F.linear(cur, up[e]), down[e])
            out.index_add_(0, top_x, y * topv[top_x, idx_k, None])
        sh = F.linear(F.silu(F.linear(xx, sg)) * F.linear(xx, su), sd)
        return out + torch.sigmoid(F.linear(xx, ssg)) * sh

    with torch.no_grad():
        for _ in range(2):
            forward(x)
        torch.cuda.synchronize()
        ms = _time_region(lambda i: forward(x), steps, torch.cuda.current_stream(dev)) / steps
    return x.shape[0] / (ms * 1e-3), ms


def routing_parity_rates(w, shape, x):
    """How the kernel's routing compares with the reference's own calls on this
    device (softmax in fp32 + torch.topk on CUDA, utils/eval_core.py:9591-9595):
    from the kernel's logits, and from the library GEMM's logits."""
    from sparse_b200 import ops
    import torch.nn.functional as F
    dev = x.device
    wg = w.router.to(torch.bfloat16).to(dev)
    bias = None if w.router_bias is None else w.router_bias.to(torch.bfloat16).to(dev)
    idx, _, logits, _ = ops.router_topk(x, wg, shape.top_k, bias=bias)
    ours = idx.long().sort(dim=1).values
    _, ti = torch.topk(torch.softmax(logits, dim=-1, dtype=torch.float32), shape.top_k, dim=-1)
    lib_logits = F.linear(x, wg, bias)
    _, tl = torch.topk(torch.softmax(lib_logits, dim=-1, dtype=torch.float32), shape.top_k, dim=-1)
    return {
        "rows": int(x.shape[0]),
        "set_match_torch_topk_cuda_same_logits": float((ti.sort(dim=1).values == ours).all(dim=1).float().mean()),
        "ordered_match_torch_topk_cuda_same_logits": float((ti == idx.long()).all(dim=1).float().mean()),
        "set_match_vs_library_gemm_logits": float((tl.sort(dim=1).values == ours).all(dim=1).float().mean()),
        "logits_equal_to_library_gemm": float((lib_logits == logits).float().mean()),
    }

def _time_region(fn, steps, stream):
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for i in range(steps):
        fn(i)
    end.record(stream)
    end.synchronize()
    return start.elapsed_time(end)      # ms


def stage_breakdown(lw, shape, xs, steps):
    """Per-kernel device time of one step through the per-stage entry points."""
    from sparse_b200 import ops
    dev = lw.device
    stream = torch.cuda.current_stream(dev)
    t, k, e, h, i, ish = xs[0].shape[0], shape.top_k, shape.num_experts, shape.hidden, shape.inter, shape.shared_inter
    x = xs[0]
    idx, wts, _, sg = ops.router_topk(x, lw.router_w, k, bias=lw.router_bias, w_shared_gate=lw.shared_gate_w)
    p = ops.permute(x, idx.reshape(-1), e, k, item_scale=wts.reshape(-1))
    y, _ = ops.grouped_swiglu(p.rows, lw.w13, lw.w2, tile_table=p.tile_table,
                              slot_of_expert=lw.slot_of_expert, row_scale=p.slot_scale)
    ys, _ = ops.grouped_swiglu(x, lw.shared_w13, lw.shared_w2, dense_rows=t, row_scale=sg)
    torch.cuda.synchronize()
    out = {}
    reps = max(5, min(steps, 50))

    def timed(name, fn):
        # Each stage is replayed from a CUDA graph of 4 calls so that the host side of
        # the wrappers (allocations, ctypes) cannot stretch the device time of the
        # short kernels.
        for j in range(3):
            fn(j)
        torch.cuda.synchronize()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(stream)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for j in range(4):
                    fn(j)
        stream.wait_stream(side)
        torch.cuda.synchronize()
        graph.replay()
        out[name] = _time_region(lambda i: graph.replay(), reps, stream) / (reps * 4)

    timed("router_topk", lambda j: ops.router_topk(xs[j % len(xs)], lw.router_w, k, bias=lw.router_bias,
                                                   w_shared_gate=lw.shared_gate_w))
    timed("permute", lambda j: ops.permute(xs[j % len(xs)], idx.reshape(-1), e, k, item_scale=wts.reshape(-1)))
    timed("routed_swiglu", lambda j: ops.grouped_swiglu(p.rows, lw.w13, lw.w2, tile_table=p.tile_table,
                                                        slot_of_expert=lw.slot_of_expert, row_scale=p.slot_scale))
    timed("shared_swiglu", lambda j: ops.grouped_swiglu(xs[j % len(xs)], lw.shared_w13, lw.shared_w2,
                                                        dense_rows=t, row_scale=sg))
    timed("combine", lambda j: ops.combine(y, p.slot_of_item, idx, ys, t))
    n = t * k
    distinct = int((p.expert_offsets[1:] != p.expert_offsets[:-1]).sum().item())
    bytes_ = {
        "router_topk": t * h * 2 + (e + 1) * h * 2 + t * k * 6 + t * e * 2 + t * 2,
        "permute": t * h * 2 + n * h * 2 + n * 14,
        "combine": n * h * 2 + n * 8 + t * h * 2 + t * h * 2,
    }
    flops = {
        "routed_swiglu": 2 * n * h * 2 * i + 2 * n * i * h,
        "shared_swiglu": 2 * t * h * 2 * ish + 2 * t * ish * h,
    }
    return out, bytes_, flops, distinct


def token_sweep(lw, shape, peaks, counts=(1, 8, 64, 256, 1024)):
    """Decode-to-prefill sweep of the same layer: device time per pass at small
    token counts (four passes over rotated inputs captured in one CUDA graph, so
    launch gaps are what a graph-captured serving step would see), the roofline
    for the experts actually touched, and tokens/s."""
    from sparse_b200.layer import LayerRunner
    from sparse_b200 import synth
    dev = lw.device
    out = {}
    for t in counts:
        runner = LayerRunner(lw, shape.top_k, t)
        xs = [synth.make_hidden(t, shape.hidden, seed=50 + b).to(torch.bfloat16).to(dev) for b in range(4)]
        for b in range(4):
            runner.forward(xs[b])
        torch.cuda.synchronize()
        touched = int(torch.unique(runner.topk_idx[:t]).numel())
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            runner.forward(xs[0])
            with torch.cuda.graph(graph, stream=side):
                for b in range(4):
                    runner.forward(xs[b])
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        for _ in range(3):
            graph.replay()
        reps = 50
        ms = _time_region(lambda i: graph.replay(), reps, torch.cuda.current_stream(dev)) / (reps * 4)
        runner.check_status()
        flops = shape.flops_per_token() * t
        hbm = touched * shape.routed_expert_bytes_bf16 + 3 * shape.hidden * shape.shared_inter * 2 \
            + 2 * t * shape.hidden * 2
        roof = max(flops / (peaks["bf16_tflops"] * 1e12), hbm / (peaks["hbm_gbs"] * 1e9)) * 1e3
        out[str(t)] = {"ms": ms, "tokens_per_s": t / (ms * 1e-3), "experts_touched": touched,
                       "roofline_ms": roof, "frac": roof / ms, "launches": runner.last_launches}
    return out


def decode_stack(lw, shape, peaks, layers=24, counts=(1, 8, 16)):
    """A decode step through a 24-layer stack of MoE blocks, each layer with its
    own 1.1 GB of weights (so nothing survives in L2 from layer to layer), the
    output of a layer plus its input feeding the next, captured as ONE CUDA graph
    and replayed: what the MoE layers cost inside a graph-captured decode loop of
    a 24-layer model (attention not included)."""
    from sparse_b200.layer import LayerRunner
    from sparse_b200 import synth
    dev = lw.device
    stack = [lw] + [lw.clone() for _ in range(layers - 1)]
    out = {}
    for t in counts:
        runners = [LayerRunner(w_l, shape.top_k, t) for w_l in stack]
        x0 = synth.make_hidden(t, shape.hidden, seed=77).to(torch.bfloat16).to(dev)
        bufs = [torch.empty_like(x0) for _ in range(layers + 1)]
        outs = [torch.empty_like(x0) for _ in range(layers)]

        def step():
            bufs[0].copy_(x0)
            for li, r in enumerate(runners):
                r.forward(bufs[li], outs[li])
                torch.add(bufs[li], outs[li], out=bufs[li + 1])     # residual stream

        step()
        torch.cuda.synchronize()
        touched = sum(int(torch.unique(r.topk_idx[:t]).numel()) for r in runners)
        cap = torch.cuda.Stream(device=dev)
        cap.wait_stream(torch.cuda.current_stream(dev))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(cap):
            step()
            with torch.cuda.graph(graph, stream=cap):
                step()
        torch.cuda.current_stream(dev).wait_stream(cap)
        torch.cuda.synchronize()
        for _ in range(3):
            graph.replay()
        reps = 20
        ms = _time_region(lambda i: graph.replay(), reps, torch.cuda.current_stream(dev)) / reps
        for r in runners:
            r.check_status()
        hbm = touched * shape.routed_expert_bytes_bf16 + layers * 3 * shape.hidden * shape.shared_inter * 2
        floor_ms = hbm / (peaks["hbm_gbs"] * 1e9) * 1e3
        out[str(t)] = {"ms_per_step": ms, "tokens_per_s": t / (ms * 1e-3), "layers": layers,
                       "us_per_layer": ms * 1e3 / layers, "experts_touched": touched,
                       "hbm_floor_ms": floor_ms, "frac": floor_ms / ms}
    return out


class _Lin:
    """The two attributes of a linear layer that the block constructor reads."""
    def __init__(self, weight, bias=None):
        self.weight, self.bias = weight, bias


class _Mlp:
    def __init__(self, g, u, d):
        self.gate_proj, self.up_proj, self.down_proj = _Lin(g), _Lin(u), _Lin(d)


class _QwenLikeBlock:
    """Duck-typed stand-in for the framework MoE block the reference wraps."""
    def __init__(self, w):
        self.gate = _Lin(w.router, w.router_bias)
        self.experts = [_Mlp(w.gate[e], w.up[e], w.down[e]) for e in range(w.shape.num_experts)]
        self.shared_expert = _Mlp(w.sh_gate, w.sh_up, w.sh_down)
        self.shared_expert_gate = _Lin(w.sh_scalar_gate)
        self.norm_topk_prob = w.shape.norm_topk_prob


class _Env:
    def __init__(self, dev):
        self.rank, self.world, self.local_rank, self.device = 0, 1, dev.index or 0, dev


def offload_methods(args):
    """Opt-in (`--offload-methods`): decode steps (8 tokens) through a 4-layer
    stack of reference-style blocks whose experts live in pinned host memory with
    16 device slots per layer, under the reference's method switches (rr, epipe,
    rs, rs-epipe), next to the all-resident stack.  The RS predictor is a
    stand-in for a trained checkpoint: the next layer's own router applied to the
    current layer's input."""
    import gc
    import torch.nn as nn
    from sparse_b200 import synth
    from sparse_b200.config import method_settings
    from sparse_b200.context import Metrics, SparseContext
    from sparse_b200.moe_block import DistributedSparseMoeBlock
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    shape = synth.QWEN_MOE
    w = synth.make_weights(shape, weight_seed=0, zipf_s=ZIPF_S)
    src = _QwenLikeBlock(w)
    layers, cache, tokens, steps, warm = 4, 16, 8, 48, 16

    class NextRouterProbe(nn.Module):
        def __init__(self):
            super().__init__()
            self.wt = w.router.to(torch.bfloat16).float().t().contiguous().to(dev)
            self.b = w.router_bias.float().to(dev) if w.router_bias is not None else None

        def forward(self, x):
            z = x.float() @ self.wt
            return torch.softmax(z + self.b if self.b is not None else z, dim=-1)

    def build(method):
        SparseContext.initialize(layers, num_experts=shape.num_experts)
        metrics = Metrics()
        old = dict(os.environ)
        offload, planner = "gpu", "none"
        if method != "resident":
            flags, env = method_settings(method, ep_size=1)
            env["SPARSE_RS_CACHE_SAFE_MIN_SCORE_BY_RANK"] = "0.0"
            env["SPARSE_PREFETCH_MIN_CAND_SCORE"] = "0.0"
            os.environ.update(env)
            offload, planner = "cpu", flags["--planner-mode"]
        try:
            blocks = [DistributedSparseMoeBlock(
                layer_idx=l, mlp_block=src, scp_map={}, env=_Env(dev), num_layers=layers,
                num_experts=shape.num_experts, top_k=shape.top_k, dtype=torch.bfloat16, expert_offload=offload,
                expert_cache=cache, routing_mode="router", rs_dir="", rs_require_complete=False,
                rs_prob_to_logit_eps=1e-6, log_routing_stats=False, metrics=metrics, planner_mode=planner,
                prefetch_top_m=2, placement_mode="round_robin", max_tokens=64) for l in range(layers)]
        finally:
            os.environ.clear()
            os.environ.update(old)
        for l, b in enumerate(blocks):
            SparseContext.register_layer_block(l, b)
        if planner == "rs_prefetch":
            SparseContext.rs_bank = nn.ModuleList([NextRouterProbe() for _ in range(layers)])
            SparseContext.rs_bank_source_layers = list(range(-1, layers - 1))
        return blocks, metrics

    out = {}
    for method in ("resident", "rr", "epipe", "rs", "rs-epipe"):
        blocks, metrics = build(method)
        SparseContext.current_phase = "decode"
        t_acc, h0, m0, b0 = 0.0, 0, 0, 0
        for step in range(steps):
            SparseContext.begin_runtime_call(step)
            x = synth.make_hidden(tokens, shape.hidden, seed=5000 + step).to(torch.bfloat16).view(tokens, 1, -1).to(dev)
            torch.cuda.synchronize()
            if step == warm:
                h0, m0, b0 = metrics.cache_hit_count, metrics.cache_miss_count, metrics.expert_weight_h2d_bytes
            t0 = time.perf_counter()
            for blk in blocks:
                y, _ = blk(x)
                x = (x + y).contiguous()
            torch.cuda.synchronize()
            if step >= warm:
                t_acc += time.perf_counter() - t0
        for blk in blocks:
            blk.check_status()
        n = steps - warm
        hits, misses = metrics.cache_hit_count - h0, metrics.cache_miss_count - m0
        out[method] = {"ms_per_step": t_acc / n * 1e3, "us_per_layer": t_acc / n / layers * 1e6,
                       "tokens_per_s": tokens / (t_acc / n),
                       "cache_hit_rate": hits / max(1, hits + misses),
                       "h2d_mb_per_step": (metrics.expert_weight_h2d_bytes - b0) / n / 1e6,
                       "prefetch_issued": metrics.prefetch_issued_count,
                       "prefetch_used_before_demand": metrics.prefetch_complete_before_use_count,
                       "epipe_triggered": metrics.epipe_trigger_count}
        del blocks
        gc.collect()
        torch.cuda.empty_cache()
    emit({"metric": "offloaded_decode_step", "config": {
        "workload": "qwen1.5-moe-a2.7b-shaped MoE blocks, %d layers, %d tokens per decode step, experts in pinned "
                    "host memory, %d device slots per layer, zipf(1.2) router bias" % (layers, tokens, cache),
        "predictor": "stand-in: next layer's router applied to the current layer's input",
        "timing": "host wall clock per step (the offloaded path synchronises once per layer), %d steps after "
                  "%d warm-up steps" % (steps - warm, warm)}, "methods": out})


def cache_stress(args):
    """Opt-in (`--cache-stress`, launched like the bench at N > 1): decode steps of
    one token per GPU through a stack of Qwen-shaped MoE layers (MoE layers only,
    residual stream between them) with round-robin expert ownership, where every
    GPU also keeps a quarter of the experts it does NOT own in LRU cache slots
    filled from the owners' GPUs over NVLink.  Modes:

      owner   no caching: every non-owned expert's rows go to its owner (plain EP decode)
      rr      reactive LRU: a selected expert that is not cached is copied now,
              on the compute stream, then run locally (the copy time is exposed)
      rs      rr + a next-layer prefetch plan issued one layer ahead on a side
              stream; the predictor emits 8 guesses per layer of which each true
              expert survives with probability 0.7 (seeded)
      sparse  rs + readiness scheduling: what is not here (or still in flight)
              when the layer starts goes to its owner instead of being waited for

    Reports decode tokens/s (host wall clock: the path synchronises once per
    layer to read the routing back), exposed load time, hit rates and bytes."""
    import random
    import torch.distributed as dist
    from sparse_b200 import synth
    from sparse_b200.context import Metrics
    from sparse_b200.peer_cache import LocalCacheEpLayer, build_rank_layer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        raise SystemExit("--cache-stress needs at least 2 ranks (torch.distributed.run, one rank per GPU)")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist.init_process_group(backend="nccl", device_id=dev)
    shape = synth.QWEN_MOE
    layers_n, steps, warm = args.stress_layers, args.stress_steps, args.stress_warmup
    e_n, k = shape.num_experts, shape.top_k
    owner_of = [e % world for e in range(e_n)]
    non_owned = e_n - sum(1 for e in range(e_n) if e % world == rank)
    cache_slots = max(1, int(0.25 * (e_n - e_n / world)))
    w = synth.make_weights(shape, weight_seed=0, zipf_s=0.0)      # no router skew: the cache sees the whole expert set
    built = []
    for l in range(layers_n):
        lw, slab, owned, slot_at_owner = build_rank_layer(w, dev, rank, world, owner_of, cache_slots)
        slab.exchange(dist.group.WORLD)
        built.append((lw, slab, owned, slot_at_owner))
    torch.cuda.synchronize()
    dist.barrier()
    x0 = [synth.make_hidden(1, shape.hidden, seed=40000 + 131 * s_ + rank).to(torch.bfloat16).to(dev)
          for s_ in range(warm + steps)]

    def make_layers(miss, late, metrics):
        return [LocalCacheEpLayer(b[0], b[1], b[2], b[3], owner_of, k, 16, rank, world, dist.group.WORLD,
                                  cache_slots, miss=miss, late=late, metrics=metrics, layer_idx=l)
                for l, b in enumerate(built)]

    def predictor(truth_row, step, layer):
        rng = random.Random(1000003 * step + 1009 * layer + rank)
        guess = [e for e in truth_row if rng.random() < 0.7]
        others = [e for e in range(e_n) if e not in truth_row]
        rng.shuffle(others)
        guess += others[:8 - len(guess)]
        return {e: 1.0 - 0.05 * i for i, e in enumerate(guess)}

    def run(mode, truth=None):
        miss, late, prefetch = {"owner": ("owner", "owner", False), "rr": ("load", "wait", False),
                                "rs": ("load", "wait", True), "sparse": ("owner", "owner", True)}[mode]
        metrics = Metrics()
        lay = make_layers(miss, late, metrics)
        if mode == "owner":
            for ly in lay:
                ly.store.cache.capacity = 0          # nothing is ever admitted: plain owner routing
        record = [] if truth is None else None
        outs = None
        # the synthetic predictor's guesses are drawn before the clock starts: a real
        # predictor is a small MLP on the GPU, not Python on the timed path
        pred = None
        if prefetch:
            pred = [[predictor(truth[s_][l], s_, l) for l in range(layers_n)] for s_ in range(warm + steps)]
        torch.cuda.synchronize()
        dist.barrier()
        t_start = None
        snap = None
        for s_ in range(warm + steps):
            if s_ == warm:
                torch.cuda.synchronize()
                dist.barrier()
                snap = (metrics.load_exposed_ms, metrics.expert_weight_peer_bytes, metrics.cache_hit_count,
                        metrics.cache_miss_count, metrics.local_cached_item_count, metrics.owner_fallback_item_count,
                        metrics.prefetch_admitted_count, metrics.prefetch_complete_before_use_count,
                        metrics.prefetch_late_count)
                t_start = time.perf_counter()
            x = x0[s_]
            row = []
            if prefetch:
                lay[0].begin_step()
                lay[0].prefetch(pred[s_][0], budget=args.stress_budget)
            for l in range(layers_n):
                if prefetch and l + 1 < layers_n:
                    lay[l + 1].begin_step()
                    lay[l + 1].prefetch(pred[s_][l + 1], budget=args.stress_budget)
                y = lay[l].forward(x)
                if record is not None:
                    row.append(lay[l]._idx_host[0].tolist())     # already on the host
                # residual add + RMS norm, as the model does between its MoE blocks: without
                # the norm the hidden state of a 24-layer stack overflows bf16
                x = torch.nn.functional.rms_norm((x + y).float(), (shape.hidden,)).to(torch.bfloat16)
            if record is not None:
                record.append(row)
            outs = x
        torch.cuda.synchronize()
        wall = time.perf_counter() - t_start
        for ly in lay:
            ly.check_status()
            metrics.finalize_events()
        v = torch.tensor([wall], dtype=torch.float64, device=dev)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        wall = float(v.item())
        now = (metrics.load_exposed_ms, metrics.expert_weight_peer_bytes, metrics.cache_hit_count,
               metrics.cache_miss_count, metrics.local_cached_item_count, metrics.owner_fallback_item_count,
               metrics.prefetch_admitted_count, metrics.prefetch_complete_before_use_count,
               metrics.prefetch_late_count)
        d = [a - b for a, b in zip(now, snap)]
        tot = torch.tensor(d, dtype=torch.float64, device=dev)
        dist.all_reduce(tot)                                   # summed over ranks
        d = tot.tolist()
        res = {"decode_tokens_per_s": world * steps / wall, "ms_per_step": wall / steps * 1e3,
               "us_per_layer": wall / steps / layers_n * 1e6,
               "exposed_load_ms_per_step_per_gpu": d[0] / steps / world,
               "peer_weight_mb_per_step_per_gpu": d[1] / steps / world / 1e6,
               "cache_hits": int(d[2]), "cache_misses": int(d[3]),
               "items_run_locally_from_cache": int(d[4]), "items_sent_to_owner_for_lack_of_weights": int(d[5]),
               "prefetch_admitted": int(d[6]), "prefetch_ready_before_use": int(d[7]), "prefetch_late": int(d[8])}
        del lay
        return res, record, outs

    res_owner, truth, out_ref = run("owner")
    results = {"owner": res_owner}
    same = 1
    for mode in ("rr", "rs", "sparse"):
        results[mode], _, out_m = run(mode, truth)
        if not torch.equal(out_m, out_ref):
            same = 0
    flag = torch.tensor([same], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        emit({"metric": "cache_stress_decode_tokens_per_s", "n_gpus": world, "unit": "tokens/s",
              "config": {"workload": "qwen1.5-moe-a2.7b-shaped MoE layers only (no router skew), %d layers, 1 token per GPU per decode "
                                     "step, %d steps after %d warm-up steps, round-robin ownership at EP=%d, %d LRU "
                                     "slots per layer per GPU for non-owned experts (25%% of %d), weights copied "
                                     "from the owner GPU over NVLink" % (layers_n, steps, warm, world, cache_slots,
                                                                         non_owned),
                         "predictor": "synthetic: 8 guesses per layer, each true expert kept with probability 0.7 "
                                      "(seeded), prefetch budget %d per layer" % args.stress_budget,
                         "not_included": "attention and the 32768-token prefill of the full-model configuration"},
              "modes": results,
              "final_hidden_state_identical_in_all_modes": bool(int(flag.item())),
              "timing": "host wall clock, max over ranks (one host synchronisation per layer reads the routing back)"})
    dist.barrier()
    dist.destroy_process_group()


def model_decode(args):
    """Opt-in (`--model-decode qwen|deepseek`, launched like the bench at N > 1):
    prefill + greedy decode through the whole shaped model (attention, norms,
    MoE block in every layer, lm_head), random init, random token ids.
      qwen      24 layers, 8 sequences x 2048 prompt ids (seed 2), 128 new tokens
      deepseek  27 layers (layer 0 dense, MLA-shaped attention), 16 x 1024 (seed 3), 256 new tokens
    The sequences are sharded over the ranks (data-parallel attention), the
    experts by round-robin ownership.  Decode tokens/s as the reference counts
    it: generated tokens minus the first one per sequence, over the decode wall
    time (scripts/perf.py:2107-2120); every decode step is one CUDA-graph launch."""
    from sparse_b200 import synth
    from sparse_b200.context import Metrics
    from sparse_b200.model import DEEPSEEK_MODEL, QWEN_MODEL, RunningStats, ShapedMoeModel, greedy_decode_profiled

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist_
        dist = dist_
        dist.init_process_group(backend="nccl", device_id=dev)
    cfg, batch, prompt, new, seed = {"qwen": (QWEN_MODEL, 8, 2048, 128, 2),
                                     "deepseek": (DEEPSEEK_MODEL, 16, 1024, 256, 3)}[args.model_decode]
    if args.model_batch:
        batch = args.model_batch
    if args.model_prompt:
        prompt = args.model_prompt
    if args.model_new:
        new = args.model_new
    if batch % world != 0:
        raise SystemExit("--model-decode: %d sequences do not divide over %d ranks" % (batch, world))
    b_local = batch // world
    peaks = _peaks()
    model = ShapedMoeModel(cfg, dev, b_local, prompt + new + 1, seed=0, ep_rank=rank, ep_size=world,
                           process_group=None if world == 1 else dist.group.WORLD, chunk_tokens=4096)
    g = torch.Generator().manual_seed(seed)
    ids_all = torch.randint(0, cfg.vocab, (batch, prompt), generator=g)
    ids = ids_all[rank * b_local:(rank + 1) * b_local].to(dev)
    metrics = Metrics()
    metrics.decode_step_stats = RunningStats()
    sampler = ClockSampler(_physical_gpu_index(local_rank))
    # an untimed request first (the launchers' warm-up request): library handles,
    # lazily loaded kernels and the decode graph are set up outside the clock
    greedy_decode_profiled(model, ids, torch.ones_like(ids), 4, None, Metrics(), False)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    sampler.start()
    out = greedy_decode_profiled(model, ids, torch.ones_like(ids), new, None, metrics, True)
    sampler.stop()
    v = torch.tensor([metrics.wall_prefill_ms, metrics.wall_decode_ms], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
    prefill_ms, decode_ms = float(v[0].item()), float(v[1].item())
    # HBM bytes one decode step has to read on this GPU (last step's routing)
    touched = 0
    for ly in model.layers:
        if ly.block is not None:
            idx, _ = ly.block.topk(b_local)
            own = ly.block.weights.slot_of_expert
            touched += int(torch.unique(idx).numel()) if world == 1 else int((own >= 0).sum().item())
    shape = cfg.moe
    moe_layers = sum(1 for ly in model.layers if ly.block is not None)
    kv_bytes = cfg.layers * b_local * (prompt + new) * cfg.n_kv_heads * (cfg.qk_dim + cfg.v_dim) * 2
    attn_w = sum(sum(t.numel() * 2 for t in (getattr(ly, "wqkv", None), getattr(ly, "wq", None),
                                             getattr(ly, "wkv_a", None), getattr(ly, "wkv_b", None), ly.wo)
                     if t is not None) for ly in model.layers)
    dense_w = sum(ly.dense_w13.numel() * 2 + ly.dense_w2.numel() * 2 for ly in model.layers if ly.block is None)
    hbm = (touched * shape.routed_expert_bytes_bf16 + moe_layers * 3 * shape.hidden * shape.shared_inter * 2
           + kv_bytes + attn_w + dense_w + cfg.vocab * cfg.hidden * 2)
    floor_ms = hbm / (peaks["hbm_gbs"] * 1e9) * 1e3
    steps = new - 1
    if rank == 0:
        emit({"metric": "model_decode_tokens_per_s", "value": (batch * new - batch) / (decode_ms * 1e-3),
              "unit": "tokens/s", "n_gpus": world, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
              "config": {"workload": "%s, %d layers, %d sequences x %d random prompt ids (seed %d), %d greedy tokens, "
                                     "random init" % (cfg.name, cfg.layers, batch, prompt, seed, new),
                         "parallelism": "ep%d, sequences sharded %d per GPU, round-robin expert ownership" % (world, b_local),
                         "launch_mode": "one CUDA-graph launch per decode step (all layers, lm_head, argmax)",
                         "prefill_attention": "library fused attention over the cache, prompt in chunks of 4096 tokens"},
              "prefill_ms": prefill_ms, "prefill_tokens_per_s": batch * prompt / (prefill_ms * 1e-3),
              "decode_ms_per_step": decode_ms / steps,
              "decode_hbm_roofline": {"bytes_per_step_per_gpu": hbm, "floor_ms": floor_ms, "peak_gbs": peaks["hbm_gbs"],
                                      "frac": floor_ms / (decode_ms / steps),
                                      "what": "weights of the experts a step touches (on this GPU), shared experts, "
                                              "attention and dense weights, the cached keys/values, the lm_head"},
              "generated_sample": out[0, prompt:prompt + 8].tolist(),
              "clocks": sampler.summary()})
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_ours(args):
    from sparse_b200 import synth
    from sparse_b200.block import B200MoeBlock
    from sparse_b200.layer import LayerRunner, LayerWeights

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if args.gpus != 1 and world == 1:
            raise SystemExit("bench.py --gpus N>1 must be launched with torch.distributed.run (one rank per GPU)")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist_
        dist = dist_
        dist.init_process_group(backend="nccl", device_id=dev)

    peaks = _peaks()
    shape = synth.QWEN_MOE
    t = TOKENS_PER_GPU
    w = synth.make_weights(shape, weight_seed=0, zipf_s=ZIPF_S)

    def make_block(kind):
        """kind: balanced | rr | perm:<seed>  ->  (block, note)"""
        from sparse_b200.placement import Placement
        placement, note = None, "single GPU"
        if world > 1 and kind == "balanced":
            # Profile -> placement, as the reference's offline solver does for its
            # replicated placements: expert load of a seeded calibration batch
            # (not a bench input), hot experts replicated, sources spread over replicas.
            from sparse_b200 import ops
            from sparse_b200.placement import balanced_replicated_placement
            xc = synth.make_hidden(4096, shape.hidden, seed=424242).to(torch.bfloat16).to(dev)
            idx_c, _, _, _ = ops.router_topk(xc, w.router.to(torch.bfloat16).to(dev), shape.top_k,
                                             bias=None if w.router_bias is None else w.router_bias.float().to(dev))
            load = torch.bincount(idx_c.reshape(-1).long().cpu(), minlength=shape.num_experts).tolist()
            obj = balanced_replicated_placement([load], world)
            placement = Placement("scp_ep", 1, shape.num_experts, world, obj=obj, apply_decode=True)
            held = [len(placement.receive_experts(0, r, "prefill")) for r in range(world)]
            note = ("load-balanced replicated placement from a calibration batch's expert histogram; "
                    "experts held per rank %s" % held)
        elif world > 1 and kind.startswith("perm:"):
            # a seeded random permutation of the experts dealt round-robin, in the
            # non-replicated placement schema {"placement": {layer: {expert: rank}}}
            seed = int(kind.split(":", 1)[1])
            g = torch.Generator().manual_seed(seed)
            order = torch.randperm(shape.num_experts, generator=g).tolist()
            obj = {"placement": {"0": {str(e): pos % world for pos, e in enumerate(order)}}}
            placement = Placement("scp_ep", 1, shape.num_experts, world, obj=obj, apply_decode=True)
            note = "seeded random-permutation ownership (seed %d), one owner per expert" % seed
        elif world > 1:
            note = "round-robin ownership (e %% %d)" % world
        blk = B200MoeBlock.from_block_weights(w, dev, ep_rank=rank, ep_size=world, max_tokens=t,
                                              process_group=None if world == 1 else dist.group.WORLD,
                                              placement=placement, use_graphs=True)
        return blk, note

    block, placement_note = make_block(args.placement)
    xs_host = [synth.make_hidden(t, shape.hidden, seed=1 + 97 * rank + b).to(torch.bfloat16).pin_memory()
               for b in range(N_INPUT_BATCHES)]
    xs = [xh.to(dev) for xh in xs_host]
    out_host = torch.empty((t, shape.hidden), dtype=torch.bfloat16).pin_memory()
    stream = torch.cuda.current_stream(dev)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms):
        if dist is None:
            return ms
        v = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        return float(v.item())

    # ---- device-resident throughput ----
    # Every step is one graph launch: the step's kernels (two streams, device-side
    # barrier epochs at N>1) were recorded once per input buffer during warm-up.
    def step_dev(i, blk=None):
        (blk or block).forward_device(xs[i % N_INPUT_BATCHES])

    def timed_run(blk, steps, warmup):
        # warm-up: one un-recorded pass, then one recording (and replay) per input buffer
        for i in range(max(N_INPUT_BATCHES + 1, warmup)):
            step_dev(i, blk)
        barrier()
        total, per = _time_steps(lambda i: step_dev(i, blk), steps, stream)
        barrier()
        blk.check_status()
        return max_over_ranks(total), per

    sampler = ClockSampler(_physical_gpu_index(local_rank))
    sampler.start()
    ms_dev, per_step = timed_run(block, args.steps, args.warmup)
    launches = block.last_launches * args.steps

    # ---- end to end through the host-buffer API ----
    # Every step copies ITS input batch from pinned host memory and ITS result
    # back to pinned host memory; the block's host pipeline overlaps the copies
    # of neighbouring steps with the layer of the current one.
    outs_host = [out_host] + [torch.empty_like(out_host).pin_memory() for _ in range(2)]
    pipe = block.host_pipeline(depth=3)

    def step_e2e(i):
        pipe.submit(xs_host[i % N_INPUT_BATCHES], outs_host[i % 3])

    for i in range(3):
        step_e2e(i)
    pipe.drain()
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        step_e2e(i)
    pipe.drain()                              # the last result is in host memory
    ms_e2e_wall = (time.perf_counter() - t0) * 1e3
    ms_e2e = max_over_ranks(ms_e2e_wall)
    # one synchronous round trip (copy in, layer, copy out, wait): the latency of a single batch
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(5):
        block.forward_host(xs_host[i % N_INPUT_BATCHES], out_host)
    ms_e2e_sync = max_over_ranks((time.perf_counter() - t0) * 1e3 / 5)
    sampler.stop()
    barrier()

    # ---- the copies alone: what the host link allows with every rank copying at once ----
    # Same pinned buffers, same three streams' worth of overlap, no layer in between.
    cp_in, cp_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    x_cp = [torch.empty_like(xs[0]) for _ in range(3)]

    def copy_only(n):
        for i in range(n):
            with torch.cuda.stream(cp_in):
                x_cp[i % 3].copy_(xs_host[i % N_INPUT_BATCHES], non_blocking=True)
            with torch.cuda.stream(cp_out):
                outs_host[i % 3].copy_(xs[i % N_INPUT_BATCHES], non_blocking=True)
        cp_in.synchronize()
        cp_out.synchronize()

    copy_only(3)
    barrier()
    t0 = time.perf_counter()
    copy_only(args.steps)
    ms_copy = max_over_ranks((time.perf_counter() - t0) * 1e3)
    barrier()

    # ---- N > 1: one untimed step checked bit for bit against the single-GPU layer ----
    ep_parity = None
    if world > 1:
        ref_runner = LayerRunner(LayerWeights.from_block_weights(w, dev), shape.top_k, t)
        ok = 1
        for b in range(2):
            got = block.forward_device(xs[b]).clone()
            want, want_idx, _, _ = ref_runner.forward(xs[b])
            torch.cuda.synchronize()
            idx_b, _ = block.topk(t)
            if not (torch.equal(got, want) and torch.equal(idx_b, want_idx)):
                ok = 0
        block.check_status()
        flag = torch.tensor([ok], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ep_parity = {"ok": bool(int(flag.item())), "placement": args.placement,
                     "check": "2 batches per rank: output rows and expert indices of the EP step equal to the "
                              "single-GPU layer holding all 60 experts, torch.equal on every rank"}
        barrier()

    # ---- N > 1: the reference's own placements beside the default one ----
    other_placements = {}
    if world > 1 and not args.no_sweep:
        for kind in ("rr", "perm:2", "balanced"):
            if kind == args.placement:
                continue
            blk2, note2 = make_block(kind)
            n2 = max(10, min(args.steps, 50))
            ms2, per2 = timed_run(blk2, n2, N_INPUT_BATCHES + 1)
            got = blk2.forward_device(xs[0]).clone()
            want, _, _, _ = ref_runner.forward(xs[0])
            torch.cuda.synchronize()
            flag = torch.tensor([1 if torch.equal(got, want) else 0], dtype=torch.int32, device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            other_placements[kind] = {"ms_per_step": ms2 / n2, "tokens_per_s": t * world * n2 / (ms2 * 1e-3),
                                      "steps": n2, "step_ms": _step_stats(per2), "placement": note2,
                                      "ep_parity_ok": bool(int(flag.item()))}
            del blk2
            barrier()

    total_tokens = t * world * args.steps
    value = total_tokens / (ms_dev * 1e-3)
    e2e_value = total_tokens / (ms_e2e * 1e-3)

    line = {
        "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(N_INPUT_BATCHES + 1, args.warmup), "ms_per_step": ms_dev / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(world, placement_note),
        "step_ms": _step_stats(per_step),
        "launch_mode": "each step replayed from a CUDA graph recorded during warm-up (one per input buffer)",
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": t * shape.hidden * 2 * world,
                "d2h_bytes_per_step": t * shape.hidden * 2 * world,
                "timing": "host wall clock from the first submit to the last result in pinned host memory, max over ranks",
                "pipeline": "3 slots: copy-in, layer and copy-out of neighbouring steps overlap",
                "single_batch_latency_ms": ms_e2e_sync,
                "copy_only_bound": {"value": total_tokens / (ms_copy * 1e-3), "unit": "tokens/s",
                                    "what": "the same host->device and device->host copies of every step, all ranks "
                                            "at once, no layer: what the host links allow"}},
        "gpu_launches": launches,
        "clocks": sampler.summary(),
    }

    # ---- per-stage breakdown (all ranks run it; rank 0 reports) ----
    ep_marks = None
    if world > 1:
        ep_layer = block._ep
        reps = max(3, min(args.steps, 20))
        block.use_graphs = False              # the timing marks need the stage-by-stage path
        ep_layer.stage_events = []
        for i in range(reps):
            step_dev(i)
        barrier()
        ep_marks = ep_layer.stage_events
        ep_layer.stage_events = None
        recv_rows = int(ep_layer.r.recv_offsets[-1].item())
        # rows every rank received in that step, and its routed-GEMM time: the skew the barriers wait for
        rows_all = torch.zeros(world, dtype=torch.int64, device=dev)
        rows_all[rank] = recv_rows
        dist.all_reduce(rows_all)
        per = len(ep_marks) // reps
        my_gemm = 0.0
        for rep in range(reps):
            chunk = ep_marks[rep * per:(rep + 1) * per]
            for (n0, e0), (n1, e1) in zip(chunk[:-1], chunk[1:]):
                if n1 == "routed_swiglu":
                    my_gemm += e0.elapsed_time(e1) / reps
        gemm_all = torch.zeros(world, dtype=torch.float64, device=dev)
        gemm_all[rank] = my_gemm
        dist.all_reduce(gemm_all)
        rank_skew = {"received_rows": rows_all.tolist(), "routed_gemm_ms": [round(v, 4) for v in gemm_all.tolist()]}
        # where the two streams stand when, in the real (overlapped, eagerly launched) schedule of rank 0
        ep_layer.timeline = []
        for i in range(reps):
            step_dev(i)
        barrier()
        tl = ep_layer.timeline
        ep_layer.timeline = None
        per_tl = len(tl) // reps
        ep_timeline = {}
        for rep in range(1, reps):                         # the first pass warms the eager path up
            chunk = tl[rep * per_tl:(rep + 1) * per_tl]
            for name, ev in chunk[1:]:
                ep_timeline[name] = ep_timeline.get(name, 0.0) + chunk[0][1].elapsed_time(ev) / (reps - 1)

    # ---- decode-sized steps through the same block (all ranks) ----
    decode = {}
    block.use_graphs = False                  # the decode section times eager launches and its own graphs
    if not args.no_sweep:
        for td in (1, 8, 16):
            xd = [synth.make_hidden(td, shape.hidden, seed=900 + 31 * rank + b).to(torch.bfloat16).to(dev)
                  for b in range(4)]
            for i in range(5):
                block.forward_device(xd[i % 4])
            barrier()
            n_dec = 100
            ms = _time_region(lambda i: block.forward_device(xd[i % 4]), n_dec, stream)
            barrier()
            ms = max_over_ranks(ms) / n_dec
            block.check_status()
            # the same step captured once (4 passes over rotated inputs) and replayed
            cap = torch.cuda.Stream(device=dev)
            cap.wait_stream(stream)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(cap):
                block.forward_device(xd[0])
                with torch.cuda.graph(graph, stream=cap):
                    for b in range(4):
                        block.forward_device(xd[b])
            stream.wait_stream(cap)
            barrier()
            for _ in range(3):
                graph.replay()
            barrier()
            ms_g = _time_region(lambda i: graph.replay(), 25, stream)
            barrier()
            ms_g = max_over_ranks(ms_g) / 100
            block.check_status()
            decode[str(td)] = {"ms_per_layer": ms_g, "tokens_per_s": td * world / (ms_g * 1e-3),
                               "tokens_per_gpu": td, "launches": block.last_launches,
                               "launch_mode": "CUDA graph replay (4 layer passes per graph)",
                               "eager_ms_per_layer": ms}

    if rank == 0:
        stages = {}
        if world == 1:
            lw = block.weights
            stage_ms, stage_bytes, stage_flops, distinct = stage_breakdown(lw, shape, xs, args.steps)
        else:
            per = len(ep_marks) // reps
            stage_ms = {}
            for rep in range(reps):
                chunk = ep_marks[rep * per:(rep + 1) * per]
                for (n0, e0), (n1, e1) in zip(chunk[:-1], chunk[1:]):
                    stage_ms[n1] = stage_ms.get(n1, 0.0) + e0.elapsed_time(e1) / reps
            n_recv = recv_rows
            h, i, ish = shape.hidden, shape.inter, shape.shared_inter
            stage_bytes = {}
            stage_flops = {"routed_swiglu": 2 * n_recv * h * 2 * i + 2 * n_recv * i * h,
                           "shared_swiglu": 2 * t * h * 2 * ish + 2 * t * ish * h}
            distinct = block.weights.n_slots          # experts this rank holds (replicas included)
        for name, ms in stage_ms.items():
            ent = {"ms": ms}
            if name in stage_bytes:
                gbs = stage_bytes[name] / (ms * 1e-3) / 1e9
                ent.update({"bytes": stage_bytes[name], "gb_s": gbs, "frac_of_hbm_peak": gbs / peaks["hbm_gbs"]})
            if name in stage_flops:
                tf = stage_flops[name] / (ms * 1e-3) / 1e12
                ent.update({"flops": stage_flops[name], "tflop_s": tf, "frac_of_bf16_peak": tf / peaks["bf16_tflops"]})
            stages[name] = ent
        line["stages"] = stages
        gemm_flops = stage_flops["routed_swiglu"] + stage_flops["shared_swiglu"]
        gemm_ms = stage_ms["routed_swiglu"] + stage_ms["shared_swiglu"]
        achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12
        line["roofline"] = {
            "bound": "tensor", "kernel": "pair_gemm_kernel (tcgen05 cta_group::2; 4 launches per step, figures are per-launch averages)",
            "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
            "frac": achieved / peaks["bf16_tflops"], "peak_source": "%s (burst cuBLAS bf16)" % peaks["source"],
            "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH if world == 1 else None,
            "flops_per_step": gemm_flops, "ms_per_step": gemm_ms,
            "frac_of_sustained_peak": achieved / peaks["bf16_tflops_sustained"],
        }
        # whole-layer roofline per GPU: slower of dense compute at peak and
        # (HBM bytes at HBM peak + NVLink bytes at the measured 770 GB/s per direction)
        layer_flops = shape.flops_per_token() * t
        hbm_bytes = distinct * shape.routed_expert_bytes_bf16 + 3 * shape.hidden * shape.shared_inter * 2 \
            + 2 * t * shape.hidden * 2
        nvlink_bytes = 0 if world == 1 else t * shape.top_k * (world - 1) / world * shape.hidden * 2
        t_mem = hbm_bytes / (peaks["hbm_gbs"] * 1e9) + 2 * nvlink_bytes / 770e9
        t_roof = max(layer_flops / (peaks["bf16_tflops"] * 1e12), t_mem)
        line["layer_roofline"] = {"roofline_ms": t_roof * 1e3, "measured_ms": ms_dev / args.steps,
                                  "frac": t_roof * 1e3 / (ms_dev / args.steps),
                                  "distinct_experts": distinct,
                                  "nvlink_bytes_per_gpu_per_direction": nvlink_bytes,
                                  "nvlink_peak": "770 GB/s per direction (measured peer copy on this pool); with the "
                                                 "nominal 900 GB/s the bound moves by less than the flops term",
                                  "roofline_ms_at_900": max(layer_flops / (peaks["bf16_tflops"] * 1e12),
                                                            hbm_bytes / (peaks["hbm_gbs"] * 1e9)
                                                            + 2 * nvlink_bytes / 900e9) * 1e3}
        if ep_parity is not None:
            line["ep_parity"] = ep_parity
            line["rank_skew"] = rank_skew
            line["ep_timeline_ms"] = {k: round(v, 4) for k, v in ep_timeline.items()}
        if other_placements:
            line["placements"] = other_placements
        if decode:
            line["decode"] = decode
        if world == 1 and not args.no_sweep:
            line["sweep"] = token_sweep(block.weights, shape, peaks)
            line["decode_stack"] = decode_stack(block.weights, shape, peaks)
        if world == 1:
            line["parity"] = routing_parity_rates(w, shape, xs[0])
            if not args.no_sweep:
                tps_e, ms_e = torch_eager_tokens_per_s(w, shape, xs[0])
                line["torch_eager_gpu"] = {"value": tps_e, "unit": "tokens/s", "ms_per_step": ms_e,
                                           "what": "the reference block's op sequence (per-expert F.linear on cuBLAS, "
                                                   "torch.topk, index_add_) run eagerly on this GPU, same 4096 tokens"}
        if world == 1 and not args.no_cpu_baseline:
            tps, ms, cores = cpu_reference_tokens_per_s(3, 1)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                                    "sample": "first %d of the %d tokens, fp32, 3 steps after 1 warm-up" % (
                                        CPU_SAMPLE_TOKENS, t)}
        emit(line)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


_RESULT_FD = None


def emit(line):
    """The one JSON line, on the process's original stdout."""
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    # Libraries (NCCL's version banner, for one) write to file descriptor 1; the
    # contract is one JSON line there.  Everything else goes to stderr.
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="skip the decode-to-prefill token sweep")
    ap.add_argument("--placement", default="balanced",
                    help="expert placement at N>1: balanced (load-balanced replicated, default), rr "
                         "(round-robin) or perm:<seed> (seeded random permutation, one owner per expert)")
    ap.add_argument("--model-decode", default="", choices=["", "qwen", "deepseek"],
                    help="instead of the layer bench: prefill + greedy decode through the whole shaped model")
    ap.add_argument("--model-batch", type=int, default=0)
    ap.add_argument("--model-prompt", type=int, default=0)
    ap.add_argument("--model-new", type=int, default=0)
    ap.add_argument("--cache-stress", action="store_true",
                    help="instead of the layer bench: decode steps at N>1 with non-owned experts cached locally "
                         "(owner / rr / rs / sparse)")
    ap.add_argument("--stress-layers", type=int, default=24)
    ap.add_argument("--stress-steps", type=int, default=512)
    ap.add_argument("--stress-warmup", type=int, default=32)
    ap.add_argument("--stress-budget", type=int, default=2)
    ap.add_argument("--offload-methods", action="store_true",
                    help="instead of the layer bench: decode steps with host-resident experts under rr/epipe/rs/rs-epipe")
    args = ap.parse_args()
    import re
    if args.placement not in ("balanced", "rr") and not re.fullmatch(r"perm:\d+", args.placement):
        ap.error("--placement must be balanced, rr or perm:<seed>")
    if args.offload_methods:
        offload_methods(args)
        return
    if args.cache_stress:
        cache_stress(args)
        return
    if args.model_decode:
        model_decode(args)
        return
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
