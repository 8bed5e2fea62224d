"""The reference's module paths, importable.

The reference's callers import `utils.eval_core`, `utils.rs_staging`,
`utils.rs_overlap` and `utils.runtime.config`, and launch `scripts/perf.py`
(scripts/perf.py:24-42 of the reference).  Putting this directory first on
`sys.path` (or on PYTHONPATH) makes those names resolve to this package:

    import sparse_b200.compat as compat; compat.activate()
    from utils.eval_core import DistributedSparseMoeBlock, greedy_decode_profiled

Each shim module re-exports the B200 implementation under the reference's
symbol names; names of subsystems that are not built raise a clear
NotImplementedError when used, never silently do something else.
"""
import os
import sys

COMPAT_DIR = os.path.dirname(os.path.abspath(__file__))


def activate() -> str:
    """Put the shim directory first on sys.path; returns it."""
    if COMPAT_DIR in sys.path:
        sys.path.remove(COMPAT_DIR)
    sys.path.insert(0, COMPAT_DIR)
    for name in [m for m in sys.modules if m == "utils" or m.startswith("utils.")]:
        mod = sys.modules[name]
        if not str(getattr(mod, "__file__", "") or "").startswith(COMPAT_DIR):
            del sys.modules[name]          # another `utils` package was imported first
    return COMPAT_DIR
