"""Generate the golden vectors under tests/golden/ by running the REFERENCE.

Run in a container that has the reference checkout:

    python tests/golden/make_golden.py --reference <checkout of louislichen/SPARSE>

It imports the reference's `utils.eval_core`, wraps a stand-in inner MoE block
(the attribute layout of transformers 4.44: `gate`, `experts` ModuleList of
gate_proj/up_proj/down_proj/act_fn, `shared_expert` + `shared_expert_gate` or
`shared_experts`) in the reference's unmodified `DistributedSparseMoeBlock`
at world=1 on the CPU, feeds it the seeded synthetic tensors of
`sparse_b200.synth`, and stores what the reference returned.  The fixtures
hold outputs only (weights and inputs are re-drawn from the seeds): all
top-k indices and weights, the router logits, a sample of output rows and
per-row checksums of every output row.

The reference cannot travel to the GPU box; these files can.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from sparse_b200 import synth  # noqa: E402


class _MLP(nn.Module):
    def __init__(self, gw, uw, dw):
        super().__init__()
        i, h = gw.shape
        self.gate_proj = nn.Linear(h, i, bias=False)
        self.up_proj = nn.Linear(h, i, bias=False)
        self.down_proj = nn.Linear(i, h, bias=False)
        self.act_fn = nn.SiLU()
        with torch.no_grad():
            self.gate_proj.weight.copy_(gw)
            self.up_proj.weight.copy_(uw)
            self.down_proj.weight.copy_(dw)

    def forward(self, x):
        return self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))


class _GreedySoftmaxGate(nn.Module):
    """Stand-in for the DeepSeek-V2 gate, which the reference loads as
    third-party remote code and only calls: fp32 logits from fp32-cast inputs,
    fp32 softmax, greedy top-k, no renormalisation, scaling factor 1.  Returns
    (topk_idx, topk_weight) as `_routing_router` expects
    (utils/eval_core.py:9503-9517).  Ties: smaller expert id first."""

    def __init__(self, hidden, num_experts, top_k):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_experts, hidden))
        self.top_k = top_k

    def forward(self, hidden_states):
        h = hidden_states.shape[-1]
        x = hidden_states.reshape(-1, h)
        logits = torch.nn.functional.linear(x.float(), self.weight.float(), None)
        scores = logits.softmax(dim=-1, dtype=torch.float32)
        sv, si = torch.sort(scores, dim=-1, descending=True, stable=True)
        return si[:, :self.top_k].contiguous(), sv[:, :self.top_k].contiguous(), None


class _InnerBlock(nn.Module):
    """Duck-typed inner block (utils/eval_core.py:4342-4362)."""

    def __init__(self, w: synth.BlockWeights, qwen_style: bool):
        super().__init__()
        s = w.shape
        if qwen_style:
            self.gate = nn.Linear(s.hidden, s.num_experts, bias=w.router_bias is not None)
        else:
            self.gate = _GreedySoftmaxGate(s.hidden, s.num_experts, s.top_k)
        with torch.no_grad():
            self.gate.weight.copy_(w.router)
            if qwen_style and w.router_bias is not None:
                self.gate.bias.copy_(w.router_bias)
        self.experts = nn.ModuleList(
            [_MLP(w.gate[e], w.up[e], w.down[e]) for e in range(s.num_experts)])
        self.norm_topk_prob = bool(s.norm_topk_prob)
        self.top_k = s.top_k
        self.num_experts = s.num_experts
        if qwen_style:
            self.shared_expert = _MLP(w.sh_gate, w.sh_up, w.sh_down)
            self.shared_expert_gate = nn.Linear(s.hidden, 1, bias=False)
            with torch.no_grad():
                self.shared_expert_gate.weight.copy_(w.sh_scalar_gate)
        else:
            self.shared_experts = _MLP(w.sh_gate, w.sh_up, w.sh_down)


def build_reference_block(ec, w: synth.BlockWeights, dtype: torch.dtype):
    s = w.shape
    inner = _InnerBlock(w, qwen_style=s.shared_gate).to(dtype)
    ec.SparseContext.initialize(1, num_experts=s.num_experts)
    env = ec.DistEnv(rank=0, world=1, local_rank=0, device=torch.device("cpu"))
    blk = ec.DistributedSparseMoeBlock(
        layer_idx=0, mlp_block=inner, scp_map={}, env=env, num_layers=1,
        num_experts=s.num_experts, top_k=s.top_k, dtype=dtype,
        expert_offload="gpu", expert_cache=0, routing_mode="router", rs_dir="",
        rs_require_complete=False, rs_prob_to_logit_eps=1e-6,
        log_routing_stats=False, placement_mode="round_robin", topology=None)
    blk.eval()
    return blk


def sample_rows(t: int) -> np.ndarray:
    if t <= 32:
        return np.arange(t)
    head = np.arange(16)
    strided = np.linspace(16, t - 1, 16).astype(np.int64)
    return np.unique(np.concatenate([head, strided]))


def to_np(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


CASES = [
    # name, shape, dtype, tokens, zipf_s, input_seed
    ("qwen_fp32_t512", "QWEN_MOE", "float32", 512, 0.0, 1),
    ("qwen_bf16_t512", "QWEN_MOE", "bfloat16", 512, 0.0, 1),
    ("qwen_bf16_zipf_t1", "QWEN_MOE", "bfloat16", 1, 1.2, 1),
    ("qwen_bf16_zipf_t8", "QWEN_MOE", "bfloat16", 8, 1.2, 1),
    ("qwen_bf16_zipf_t64", "QWEN_MOE", "bfloat16", 64, 1.2, 1),
    ("qwen_bf16_zipf_t256", "QWEN_MOE", "bfloat16", 256, 1.2, 1),
    ("qwen_bf16_zipf_t4096", "QWEN_MOE", "bfloat16", 4096, 1.2, 1),
    ("deepseek_bf16_t64", "DEEPSEEK_V2_LITE", "bfloat16", 64, 0.0, 3),
    ("deepseek_bf16_t1000", "DEEPSEEK_V2_LITE", "bfloat16", 1000, 0.0, 3),
    ("tiny_bf16_t1", "TINY", "bfloat16", 1, 0.0, 5),
    ("tiny_bf16_t3", "TINY", "bfloat16", 3, 0.0, 5),
    ("tiny_bf16_t17", "TINY", "bfloat16", 17, 0.0, 5),
    ("tiny_bf16_t130", "TINY", "bfloat16", 130, 1.2, 5),
    ("tiny_fp32_t17", "TINY", "float32", 17, 0.0, 5),
]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import utils.eval_core as ec  # the reference

    torch.set_grad_enabled(False)
    cache = {}
    for name, shape_name, dtype_name, tokens, zipf_s, in_seed in CASES:
        if args.only and args.only not in name:
            continue
        shape = getattr(synth, shape_name)
        dtype = getattr(torch, dtype_name)
        key = (shape_name, zipf_s)
        if key not in cache:
            cache.clear()
            cache[key] = synth.make_weights(shape, weight_seed=0, zipf_s=zipf_s)
        w = cache[key]
        blk = build_reference_block(ec, w, dtype)
        x = synth.make_hidden(tokens, shape.hidden, seed=in_seed).to(dtype)
        res = blk(x.view(1, tokens, shape.hidden))
        if isinstance(res, tuple):
            out, logits = res
        else:
            out, logits = res, None
        # routing as the reference computed it on the same input
        topv, topi, logits2 = blk._routing_router(x)
        if logits is None:
            logits = logits2
        out = out.view(tokens, shape.hidden)
        rows = sample_rows(tokens)
        o64 = out.double()
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            shape=np.array(shape_name), dtype=np.array(dtype_name),
            tokens=np.array(tokens), zipf_s=np.array(zipf_s),
            input_seed=np.array(in_seed),
            topi=topi.numpy().astype(np.int16),
            topv=to_np(topv),
            logits=to_np(logits if logits.dtype == torch.float32 else logits.to(dtype)),
            rows=rows, out_rows=to_np(out[torch.from_numpy(rows)]),
            row_sum=o64.sum(1).numpy(), row_sqsum=(o64 * o64).sum(1).numpy())
        print(f"{name}: tokens={tokens} out_absmax={float(out.float().abs().max()):.4f}")


if __name__ == "__main__":
    main()
