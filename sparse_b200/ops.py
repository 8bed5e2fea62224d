"""Tensor-level wrappers over the C ABI.

PyTorch is used for device memory and streams only; every computation below
is one call into libsparse_b200.  All functions run on the current CUDA stream
of the tensors' device and never synchronise.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import lib, check

_DT = {torch.bfloat16: _lib.SB_DTYPE_BF16, torch.float32: _lib.SB_DTYPE_F32}


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError("sparse_b200 ops need CUDA tensors (there is no CPU path)")
    if not t.is_contiguous():
        raise RuntimeError("sparse_b200 ops need contiguous tensors")
    return t.data_ptr()


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def pad_rows(n: int) -> int:
    """Row capacity the grouped GEMM wants for n rows (a whole number of tiles)."""
    return max(1, (max(n, 1) + _lib.SB_TILE_M - 1) // _lib.SB_TILE_M) * _lib.SB_TILE_M


def router_topk(x: torch.Tensor, wg: torch.Tensor, top_k: int,
                bias: Optional[torch.Tensor] = None,
                w_shared_gate: Optional[torch.Tensor] = None,
                renorm: bool = False, fp32_logits: bool = False,
                want_logits: bool = True):
    """-> (idx int32 [T,K], weights [T,K], logits [T,E] | None, shared_scale [T] | None)."""
    t, h = x.shape
    e = wg.shape[0]
    dev, dt = x.device, x.dtype
    idx = torch.empty((t, top_k), dtype=torch.int32, device=dev)
    w = torch.empty((t, top_k), dtype=dt, device=dev)
    logits = None
    if want_logits:
        logits = torch.empty((t, e), dtype=torch.float32 if fp32_logits else dt, device=dev)
    shared = torch.empty((t,), dtype=dt, device=dev) if w_shared_gate is not None else None
    bias_f = None
    if bias is not None:
        bias_f = bias.to(dt).to(torch.float32).contiguous()
    with torch.cuda.device(dev):
        check(lib.sb_router_topk(_ptr(x), _ptr(wg), _ptr(bias_f), _ptr(w_shared_gate), t, h, e,
                                 top_k, int(renorm), _DT[dt], int(fp32_logits), _ptr(idx), _ptr(w),
                                 _ptr(logits), _ptr(shared), _stream(x)), "sb_router_topk")
    return idx, w, logits, shared


def softmax_topk(logits: torch.Tensor, top_k: int, renorm: bool = False):
    t, e = logits.shape
    idx = torch.empty((t, top_k), dtype=torch.int32, device=logits.device)
    w = torch.empty((t, top_k), dtype=logits.dtype, device=logits.device)
    with torch.cuda.device(logits.device):
        check(lib.sb_softmax_topk(_ptr(logits), t, e, top_k, int(renorm), _DT[logits.dtype],
                                  _ptr(idx), _ptr(w), _stream(logits)), "sb_softmax_topk")
    return idx, w


class Permutation:
    """Outputs of `permute` (all device tensors)."""
    __slots__ = ("rows", "expert_offsets", "slot_of_item", "item_of_slot", "slot_scale",
                 "tile_table", "n_items", "r_cap")


def permute(x: torch.Tensor, item_expert: torch.Tensor, num_experts: int,
            items_per_row: int, item_scale: Optional[torch.Tensor] = None) -> Permutation:
    n = item_expert.numel()
    h = x.shape[1]
    dev = x.device
    p = Permutation()
    p.n_items, p.r_cap = n, pad_rows(n)
    p.rows = torch.empty((p.r_cap, h), dtype=torch.bfloat16, device=dev)
    p.expert_offsets = torch.empty((num_experts + 1,), dtype=torch.int32, device=dev)
    p.slot_of_item = torch.empty((max(n, 1),), dtype=torch.int32, device=dev)
    p.item_of_slot = torch.empty((max(n, 1),), dtype=torch.int32, device=dev)
    p.slot_scale = (torch.empty((p.r_cap,), dtype=torch.bfloat16, device=dev)
                    if item_scale is not None else None)
    p.tile_table = torch.empty((lib.sb_tile_table_ints(n, num_experts),), dtype=torch.int32, device=dev)
    ws_bytes = lib.sb_permute_workspace_bytes(n, num_experts)
    ws = torch.empty((ws_bytes,), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        check(lib.sb_permute(_ptr(x), _ptr(item_expert), _ptr(item_scale), n, items_per_row, h,
                             num_experts, _ptr(ws), ws_bytes, _ptr(p.rows), _ptr(p.expert_offsets),
                             _ptr(p.slot_of_item), _ptr(p.item_of_slot), _ptr(p.slot_scale),
                             _ptr(p.tile_table), _stream(x)), "sb_permute")
    return p


def grouped_swiglu(rows: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor,
                   tile_table: Optional[torch.Tensor] = None, dense_rows: int = 0,
                   slot_of_expert: Optional[torch.Tensor] = None,
                   row_scale: Optional[torch.Tensor] = None,
                   status: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """rows [R_cap,H]; w13 [S,2I,H]; w2 [S,H,I] -> (out [R_cap,H], h [R_cap,I])."""
    r_cap, h = rows.shape
    s, two_i, _ = w13.shape
    i = two_i // 2
    dev = rows.device
    hbuf = torch.empty((r_cap, i), dtype=torch.bfloat16, device=dev)
    out = torch.empty((r_cap, h), dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        check(lib.sb_grouped_swiglu(_ptr(rows), _ptr(tile_table), dense_rows, _ptr(w13), _ptr(w2),
                                    _ptr(slot_of_expert), _ptr(row_scale), r_cap, h, i, s,
                                    _ptr(hbuf), _ptr(out), _ptr(status), _stream(rows)),
              "sb_grouped_swiglu")
    return out, hbuf


def combine(rows_out: torch.Tensor, slot_of_item: torch.Tensor, idx: torch.Tensor,
            shared_out: Optional[torch.Tensor], tokens: int,
            shared_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`shared_scale` [T] bf16: the shared expert's scalar gate, applied to `shared_out`'s
    rows on the way (sb_combine_gated)."""
    h = rows_out.shape[1]
    k = idx.shape[1]
    out = torch.empty((tokens, h), dtype=torch.bfloat16, device=rows_out.device)
    with torch.cuda.device(rows_out.device):
        if shared_scale is None:
            check(lib.sb_combine(_ptr(rows_out), _ptr(slot_of_item), _ptr(idx), _ptr(shared_out), tokens,
                                 h, k, _ptr(out), _stream(rows_out)), "sb_combine")
        else:
            check(lib.sb_combine_gated(_ptr(rows_out), _ptr(slot_of_item), _ptr(idx), _ptr(shared_out),
                                       _ptr(shared_scale), tokens, h, k, _ptr(out), _stream(rows_out)),
                  "sb_combine_gated")
    return out


def slot_copy_async(dst: torch.Tensor, src: torch.Tensor, stream: torch.cuda.Stream,
                    kind: int) -> None:
    """Copy `src` (pinned host, peer or local device tensor) into the cache slot `dst`."""
    if dst.numel() * dst.element_size() != src.numel() * src.element_size():
        raise RuntimeError("slot copy size mismatch")
    if not dst.is_contiguous() or not src.is_contiguous():
        raise RuntimeError("slot copy needs contiguous tensors")
    check(lib.sb_slot_copy_async(dst.data_ptr(), src.data_ptr(), dst.numel() * dst.element_size(),
                                 kind, dst.device.index, stream.cuda_stream), "sb_slot_copy_async")
