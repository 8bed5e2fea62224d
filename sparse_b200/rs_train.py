"""Training next-layer RoutingScout predictors on this box.

The reference trains one small MLP per layer pair offline
(scripts/train_next_layer_rs.py:484-642): input = the hidden state entering
MoE layer l, label = the multi-hot of the experts the router of layer l+1
really chose for the same token ("next_layer_true_router_topk_multihot"), and
stores it as `rs_l{l+1}_inL{l}.pth` with the payload keys its runtime loader
reads (603-630).  This module does the same for the models of
`sparse_b200.model`:

    pairs = collect_pairs(model, prompt_ids, new_tokens)     # run the model, record (x_l, top-k_{l+1})
    report = train_bank(pairs, out_dir, num_experts, ...)    # one predictor per pair, checkpoints on disk
    rs.load_rs_bank(out_dir, ...)                            # what the serving path loads

Training is ordinary PyTorch (AdamW on a soft cross-entropy against the
normalised multi-hot label, early stopping on a held-out split, recall@k
reported as the reference does); the predictors are tiny fp32 MLPs and not
part of the bf16 hot path.
"""
from __future__ import annotations

import math
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from .rs import RoutingScoutResidualMLP


def collect_pairs(model, input_ids: torch.Tensor, new_tokens: int) -> Dict[Tuple[int, int], Tuple[torch.Tensor, torch.Tensor]]:
    """Run prefill + `new_tokens` eager decode steps and record, for every pair of
    consecutive MoE layers (l, l+1), the rows entering layer l's MoE block and
    the experts layer l+1's router chose for the same tokens.
    Returns {(l, l+1): (X [N,H] fp32 on CPU, I [N,K] int64 on CPU)}."""
    trace: List[Tuple[int, torch.Tensor, torch.Tensor]] = []
    model.trace = trace
    try:
        logits = model.prefill(input_ids.to(model.device))
        model.cur_ids.copy_(torch.argmax(logits, dim=-1))
        for _ in range(max(0, new_tokens - 1)):
            model.decode_step(use_graph=False)
        torch.cuda.synchronize(model.device)
    finally:
        model.trace = None
    by_call: Dict[int, List[Tuple[torch.Tensor, torch.Tensor]]] = {}
    for layer, x, idx in trace:
        by_call.setdefault(layer, []).append((x, idx))
    layers = sorted(by_call)
    out = {}
    for a, b in zip(layers[:-1], layers[1:]):
        xs = torch.cat([x for x, _ in by_call[a]]).float().cpu()
        ids = torch.cat([i for _, i in by_call[b]]).long().cpu()
        if xs.shape[0] == ids.shape[0]:
            out[(a, b)] = (xs, ids)
    return out


def _soft_ce(probs: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    return -(target * torch.log(probs.clamp_min(1e-9))).sum(dim=-1).mean()


def recall_at_k(probs: torch.Tensor, true_ids: torch.Tensor, k: int) -> float:
    """Share of the truly chosen experts that are among the k highest-scored predictions."""
    top = torch.topk(probs, min(k, probs.shape[1]), dim=-1).indices
    hit = (top.unsqueeze(2) == true_ids.unsqueeze(1)).any(dim=1)
    return float(hit.float().mean())


def train_pair(x: torch.Tensor, true_ids: torch.Tensor, num_experts: int, hidden_dim: int = 512,
               num_hidden_layers: int = 2, epochs: int = 30, lr: float = 1e-3, weight_decay: float = 1e-2,
               batch_size: int = 1024, patience: int = 5, seed: int = 0, device: Optional[torch.device] = None,
               eval_ks: Sequence[int] = (4, 8)):
    """One predictor: x [N,H] fp32, true_ids [N,K].  Returns (module in eval mode on CPU, metrics)."""
    device = device or torch.device("cuda" if torch.cuda.is_available() else "cpu")
    g = torch.Generator().manual_seed(seed)
    n = x.shape[0]
    perm = torch.randperm(n, generator=g)
    n_val = max(1, n // 10)
    val, tr = perm[:n_val], perm[n_val:]
    torch.manual_seed(seed)
    model = RoutingScoutResidualMLP(x.shape[1], num_experts, hidden_dim, num_hidden_layers, dropout=0.05).to(device)
    opt = torch.optim.AdamW(model.parameters(), lr=lr, weight_decay=weight_decay)
    k = true_ids.shape[1]
    target = torch.zeros((n, num_experts)).scatter_(1, true_ids, 1.0 / k)
    xd, td, idd = x.to(device), target.to(device), true_ids.to(device)
    best, best_state, best_epoch, left = math.inf, None, -1, patience
    for epoch in range(epochs):
        model.train()
        order = tr[torch.randperm(tr.numel(), generator=g)]
        for s in range(0, order.numel(), batch_size):
            b = order[s:s + batch_size].to(device)
            opt.zero_grad(set_to_none=True)
            loss = _soft_ce(model(xd[b]), td[b])
            loss.backward()
            opt.step()
        model.eval()
        with torch.no_grad():
            v = val.to(device)
            val_loss = float(_soft_ce(model(xd[v]), td[v]))
        if val_loss < best:
            best, best_epoch, left = val_loss, epoch, patience
            best_state = {k_: t.detach().cpu().clone() for k_, t in model.state_dict().items()}
        else:
            left -= 1
            if left <= 0:
                break
    model.load_state_dict(best_state, strict=True)
    model.eval()
    with torch.no_grad():
        v = val.to(device)
        pv = model(xd[v])
        metrics = {"loss": best, "best_epoch": best_epoch, "n_train": int(tr.numel()), "n_val": int(val.numel())}
        for kk in eval_ks:
            metrics["recall@%d" % kk] = recall_at_k(pv, idd[v], kk)
    return model.cpu(), metrics


def save_checkpoint(out_dir: str, module: nn.Module, source_layer: int, target_layer: int, input_dim: int,
                    num_experts: int, hidden_dim: int, num_hidden_layers: int, top_k: int, metrics: Dict) -> str:
    """The reference's payload (scripts/train_next_layer_rs.py:603-630) and file name."""
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, "rs_l%d_inL%d.pth" % (target_layer, source_layer))
    torch.save({
        "model_type": "next_layer_residual_logits_rs", "task": "router_prob", "state_dict": module.state_dict(),
        "input_dim": int(input_dim), "hidden_dim": int(hidden_dim), "num_hidden_layers": int(num_hidden_layers),
        "num_experts": int(num_experts), "source_layer": int(source_layer), "target_layer": int(target_layer),
        "lead_layers": int(target_layer - source_layer), "top_k": int(top_k),
        "label_type": "next_layer_true_router_topk_multihot", "feature_mode": "hidden",
        "target_distribution": "multihot", "loss_mode": "soft_ce", "best_epoch": int(metrics.get("best_epoch", -1)),
        "best_val": float(metrics.get("loss", 0.0)), "metrics": dict(metrics), "split_sha256": "",
        "profile_manifest_sha256": "", "profile_provenance": "collected on this box by sparse_b200.rs_train",
    }, path)
    return path


def train_bank(pairs: Dict[Tuple[int, int], Tuple[torch.Tensor, torch.Tensor]], out_dir: str, num_experts: int,
               hidden_dim: int = 512, num_hidden_layers: int = 2, **train_kw) -> List[Dict]:
    """Train and save one predictor per (source, target) pair; returns one report row per pair."""
    rows = []
    for (src, dst), (x, ids) in sorted(pairs.items()):
        mod, metrics = train_pair(x, ids, num_experts, hidden_dim, num_hidden_layers, seed=1009 * src + dst, **train_kw)
        path = save_checkpoint(out_dir, mod, src, dst, x.shape[1], num_experts, hidden_dim, num_hidden_layers,
                               ids.shape[1], metrics)
        rows.append(dict(metrics, source_layer=src, target_layer=dst, ckpt=path))
    return rows
