"""ctypes binding of libsparse_b200.so (the C ABI in include/sparse_b200.h).

There is no fallback: if the library is missing the import of this module
raises, and every op raises `RuntimeError` with the library's own message on a
non-zero status.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Tuple

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libsparse_b200.so")

SB_OK = 0
SB_DTYPE_BF16 = 0
SB_DTYPE_F32 = 1
SB_COPY_HOST_TO_DEVICE = 0
SB_COPY_PEER_TO_DEVICE = 1
SB_COPY_DEVICE_LOCAL = 2
SB_TILE_M = 128

i32, vp, sz = C.c_int32, C.c_void_p, C.c_size_t


class MoeLayer(C.Structure):
    """Mirror of `struct sb_moe_layer`."""
    _fields_ = [
        ("T", i32), ("H", i32), ("E", i32), ("K", i32), ("I", i32), ("I_shared", i32),
        ("renorm", i32), ("n_slots", i32), ("router_fp32_logits", i32), ("reserved_", i32),
        ("x", vp), ("router_w", vp), ("router_bias", vp), ("shared_gate_w", vp),
        ("w13", vp), ("w2", vp), ("slot_of_expert", vp),
        ("shared_w13", vp), ("shared_w2", vp),
        ("out", vp), ("logits", vp), ("topk_idx", vp), ("topk_w", vp),
        ("ws", vp), ("ws_bytes", sz),
    ]


# name -> (restype, argtypes); this table is also what the symbol-export test walks.
# rows up to which `sb_moe_layer_forward` takes the weight-streaming path (SB_DECODE_MAX_TOKENS)
DECODE_MAX_TOKENS = 16

SIGNATURES: Dict[str, Tuple[object, list]] = {
    "sb_abi_version": (i32, []),
    "sb_last_error_string": (C.c_char_p, []),
    "sb_device_sm_count": (i32, []),
    "sb_last_launch_count": (i32, []),
    "sb_init": (i32, [i32]),
    "sb_set_tuning": (i32, [C.c_char_p, i32]),
    "sb_tile_rows": (i32, []),
    "sb_w13_interleaved": (i32, []),
    "sb_router_topk": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp]),
    "sb_softmax_topk": (i32, [vp, i32, i32, i32, i32, i32, vp, vp, vp]),
    "sb_permute_workspace_bytes": (sz, [i32, i32]),
    "sb_tile_table_ints": (sz, [i32, i32]),
    "sb_permute": (i32, [vp, vp, vp, i32, i32, i32, i32, vp, sz, vp, vp, vp, vp, vp, vp, vp]),
    "sb_permute_noalloc": (i32, [vp, vp, vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp]),
    "sb_grouped_swiglu": (i32, [vp, vp, i32, vp, vp, vp, vp, i32, i32, i32, i32, vp, vp, vp, vp]),
    "sb_decode_experts": (i32, [vp, vp, i32, vp, vp, vp, vp, vp, i32, i32, i32, vp, vp, vp, vp, vp, i32, i32,
                                vp, vp, vp, vp]),
    "sb_decode_experts_to": (i32, [vp, vp, i32, vp, vp, vp, vp, vp, i32, i32, i32, vp, vp, i32, vp, vp]),
    "sb_grouped_swiglu_mixed": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, vp, i32, vp, vp, vp, vp,
                                      i32, i32, vp, vp, vp, vp, vp]),
    "sb_route_decode": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp,
                              vp, vp]),
    "sb_combine": (i32, [vp, vp, vp, vp, i32, i32, i32, vp, vp]),
    "sb_combine_gated": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, vp, vp]),
    "sb_slot_copy_async": (i32, [vp, vp, sz, i32, i32, vp]),
    "sb_peer_alloc": (i32, [sz, C.POINTER(vp)]),
    "sb_peer_free": (i32, [vp]),
    "sb_ipc_export": (i32, [vp, vp]),
    "sb_ipc_import": (i32, [vp, C.POINTER(vp)]),
    "sb_ipc_close": (i32, [vp]),
    "sb_ep_publish_counts": (i32, [vp, i32, i32, i32, C.POINTER(vp), vp]),
    "sb_ep_barrier": (i32, [C.POINTER(vp), i32, i32, C.c_uint32, vp, vp]),
    "sb_ep_barrier_seq": (i32, [C.POINTER(vp), i32, i32, vp, vp, vp]),
    "sb_ep_barrier_timed": (i32, [C.POINTER(vp), i32, i32, vp, C.c_uint64, vp, vp]),
    "sb_ep_exchange_dispatch": (i32, [vp, C.POINTER(vp), C.POINTER(vp), vp, vp, i32, i32, i32, i32, vp, vp, vp,
                                      vp, vp, vp, vp, i32, i32, i32, C.POINTER(vp), C.POINTER(vp), vp, vp,
                                      C.POINTER(vp), C.POINTER(vp), i32, vp, vp, vp]),
    "sb_ep_exchange_dispatch_local": (i32, [vp, C.POINTER(vp), C.POINTER(vp), vp, vp, i32, i32, i32, i32, vp, vp,
                                            vp, vp, vp, vp, vp, i32, i32, i32, C.POINTER(vp), C.POINTER(vp), vp, vp,
                                            C.POINTER(vp), C.POINTER(vp), i32, vp, vp, vp, vp, vp, vp]),
    "sb_ep_plan": (i32, [vp, vp, i32, i32, i32, i32, vp, vp, vp, vp]),
    "sb_ep_dispatch": (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32,
                             C.POINTER(vp), C.POINTER(vp), vp, vp, i32, C.POINTER(vp), vp]),
    "sb_ep_return_rows": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "sb_grouped_swiglu_passes": (i32, [vp, vp, i32, vp, vp, vp, vp, i32, i32, i32, i32, vp, vp, i32, i32, vp, vp]),
    "sb_ep_resolve_return": (i32, [vp, vp, i32, C.POINTER(vp), i32, i32, i32, i32, vp, vp]),
    "sb_grouped_swiglu_scatter": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, vp, vp, vp]),
    "sb_ep_combine": (i32, [C.POINTER(vp), vp, vp, vp, vp, i32, i32, i32, i32, vp, vp]),
    "sb_add_rmsnorm": (i32, [vp, vp, vp, vp, C.c_float, i32, i32, vp, vp]),
    "sb_rope_append": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, C.c_float, i32, vp, vp, i32, i32, i32,
                             vp]),
    "sb_attn_decode_workspace_bytes": (sz, [i32, i32, i32, i32]),
    "sb_attn_decode": (i32, [vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, C.c_float, i32, vp, sz, vp, vp]),
    "sb_moe_layer_struct_bytes": (sz, []),
    "sb_moe_layer_workspace_bytes": (sz, [i32, i32, i32, i32, i32, i32]),
    "sb_moe_layer_forward": (i32, [C.POINTER(MoeLayer), vp, vp]),
}


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m sparse_b200.build` "
            "(needs nvcc); sparse_b200 has no non-CUDA fallback")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)       # AttributeError if a symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()
if lib.sb_moe_layer_struct_bytes() != C.sizeof(MoeLayer):
    raise ImportError("sparse_b200: struct sb_moe_layer of the library and its ctypes mirror differ")


def apply_tuning_from_env(var: str = "SPARSE_B200_TUNING") -> None:
    """`key=value,key=value` from the environment -> `sb_set_tuning` (the reference's
    knobs are environment variables read by the block, utils/eval_core.py:4939-4968;
    these only change scheduling, never results).  A bad entry raises."""
    for item in filter(None, (t.strip() for t in os.environ.get(var, "").split(","))):
        key, _, value = item.partition("=")
        status = lib.sb_set_tuning(key.strip().encode(), int(value))
        if status != SB_OK:
            msg = lib.sb_last_error_string()
            raise ValueError(f"{var}: {item!r} refused: {msg.decode() if msg else status}")


apply_tuning_from_env()

_initialised = set()


def init_device(index: int) -> None:
    """`sb_init` once per device index (creates the library's side stream there)."""
    if index not in _initialised:
        check(lib.sb_init(int(index)), "sb_init")
        _initialised.add(index)


def check(status: int, what: str) -> None:
    if status != SB_OK:
        msg = lib.sb_last_error_string()
        raise RuntimeError(f"{what} failed with status {status}: {msg.decode() if msg else ''}")
