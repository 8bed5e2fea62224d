"""CPU: the C-ABI library loads without a GPU, exports every declared symbol,
and rejects bad arguments before touching a device."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT


def _declared():
    with open(os.path.join(ROOT, "include", "sparse_b200.h")) as fh:
        src = fh.read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(sb_[a-z0-9_]+)\s*\(", src)))


def test_every_declared_symbol_is_exported_and_bound():
    from sparse_b200 import _lib
    names = _declared()
    assert len(names) >= 12
    for n in names:
        assert hasattr(_lib.lib, n), f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(names)
    assert _lib.lib.sb_abi_version() == 2


def test_size_queries_need_no_device():
    from sparse_b200._lib import lib
    assert lib.sb_permute_workspace_bytes(16384, 60) >= 128 * 60 * 4
    assert lib.sb_permute_workspace_bytes(0, 60) > 0
    assert lib.sb_tile_table_ints(16384, 60) == 4 + (128 + 60) * 4
    a = lib.sb_moe_layer_workspace_bytes(4096, 2048, 60, 4, 1408, 5632)
    b = lib.sb_moe_layer_workspace_bytes(8192, 2048, 60, 4, 1408, 5632)
    assert 0 < a < b
    # rows + intermediate + outputs of T=4096: a few hundred MB, not GB
    assert 200e6 < a < 600e6


def test_bad_arguments_are_rejected_with_a_message():
    from sparse_b200._lib import lib
    rc = lib.sb_router_topk(None, None, None, None, 4, 2048, 60, 0, 0, 0, 0, None, None, None, None, None)
    assert rc == -1 and b"sb_router_topk" in lib.sb_last_error_string()
    rc = lib.sb_router_topk(None, None, None, None, 4, 2047, 60, 4, 0, 0, 0, None, None, None, None, None)
    assert rc == -1
    rc = lib.sb_combine(None, None, None, None, 4, 2048, 9, None, None)
    assert rc == -1 and b"sb_combine" in lib.sb_last_error_string()
    assert lib.sb_combine_gated(None, None, None, None, None, 4, 2048, 9, None, None) == -1
    assert lib.sb_combine_gated(None, None, None, None, None, 0, 2048, 4, None, None) == 0
    rc = lib.sb_grouped_swiglu(None, None, 0, None, None, None, None, 128, 2000, 1408, 1, None, None, None, None)
    assert rc == -4 and b"multiples of 64" in lib.sb_last_error_string()
    rc = lib.sb_permute(None, None, None, 8, 1, 2048, 300, None, 0, None, None, None, None, None, None, None)
    assert rc == -1
    rc = lib.sb_slot_copy_async(None, None, 16, 0, -1, None)
    assert rc == -1
    # T == 0 is a no-op, not an error
    assert lib.sb_router_topk(None, None, None, None, 0, 2048, 60, 4, 0, 0, 0, None, None, None, None, None) == 0
    assert lib.sb_combine(None, None, None, None, 0, 2048, 4, None, None) == 0


def test_struct_layout_matches_header():
    from sparse_b200._lib import MoeLayer, lib
    assert C.sizeof(MoeLayer) == lib.sb_moe_layer_struct_bytes()


def test_decode_limit_matches_header():
    import re
    from sparse_b200 import _lib
    text = open(os.path.join(ROOT, "include", "sparse_b200.h")).read()
    m = re.search(r"#define\s+SB_DECODE_MAX_TOKENS\s+(\d+)", text)
    assert m and int(m.group(1)) == _lib.DECODE_MAX_TOKENS


def test_tuning_knob_argument_checks():
    """No GPU needed: keys and ranges of sb_set_tuning."""
    from sparse_b200 import _lib
    lib = _lib.lib
    assert lib.sb_set_tuning(b"sched", 0) == 0 and lib.sb_set_tuning(b"dense_group", 1) == 0
    assert lib.sb_set_tuning(b"router_overlap", 1) == 0
    assert lib.sb_set_tuning(b"kslabs", 2) == 0 and lib.sb_set_tuning(b"dispatch_ctas", 1) == 0
    for key, bad in ((b"sched", -1), (b"sched", 3), (b"dense_group", 0), (b"dense_group", 65), (b"router_overlap", 2),
                     (b"kslabs", 0), (b"kslabs", 3), (b"dispatch_ctas", 0), (b"dispatch_ctas", 9)):
        assert lib.sb_set_tuning(key, bad) != 0
    assert lib.sb_set_tuning(b"unknown", 0) != 0 and lib.sb_set_tuning(None, 0) != 0


def test_tuning_from_the_environment(monkeypatch):
    """SPARSE_B200_TUNING="key=value,..." is applied through sb_set_tuning; a bad entry raises."""
    from sparse_b200 import _lib
    monkeypatch.setenv("SPARSE_B200_TUNING", "kslabs=1, dispatch_ctas=4")
    _lib.apply_tuning_from_env()
    monkeypatch.setenv("SPARSE_B200_TUNING", "kslabs=7")
    with pytest.raises(ValueError):
        _lib.apply_tuning_from_env()
    monkeypatch.setenv("SPARSE_B200_TUNING", "kslabs=2,dispatch_ctas=1")
    _lib.apply_tuning_from_env()
