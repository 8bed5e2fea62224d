import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """Golden fixture written by tests/golden/make_golden.py -> dict of tensors."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    dtype = getattr(torch, str(z["dtype"]))

    def dec(a):
        t = torch.from_numpy(np.ascontiguousarray(a))
        if a.dtype == np.uint16:
            return t.view(torch.int16).view(torch.bfloat16)
        return t

    return {
        "shape": str(z["shape"]), "dtype": dtype, "tokens": int(z["tokens"]),
        "zipf_s": float(z["zipf_s"]), "input_seed": int(z["input_seed"]),
        "topi": torch.from_numpy(z["topi"].astype(np.int64)),
        "topv": dec(z["topv"]), "logits": dec(z["logits"]),
        "rows": torch.from_numpy(z["rows"].astype(np.int64)),
        "out_rows": dec(z["out_rows"]),
        "row_sum": torch.from_numpy(z["row_sum"]), "row_sqsum": torch.from_numpy(z["row_sqsum"]),
    }


_WEIGHT_CACHE = {}


def block_weights(shape_name, zipf_s):
    """Seeded fp32 master weights, cached for the session (one shape at a time
    to bound memory)."""
    from sparse_b200 import synth
    key = (shape_name, float(zipf_s))
    if key not in _WEIGHT_CACHE:
        for k in list(_WEIGHT_CACHE):
            if k[0] != shape_name:
                del _WEIGHT_CACHE[k]
        if zipf_s:
            base = block_weights(shape_name, 0.0)
            import copy
            w = copy.copy(base)
            w.router_bias = synth.zipf_router_bias(base.shape.num_experts, zipf_s, 7)
            _WEIGHT_CACHE[key] = w
        else:
            _WEIGHT_CACHE[key] = synth.make_weights(getattr(synth, shape_name), weight_seed=0)
    return _WEIGHT_CACHE[key]


def rel_l2(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))
