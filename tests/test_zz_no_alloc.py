"""`sb_permute_noalloc`: the expert-sorted permutation for hosts that cannot
allocate device scratch (a serving loop where cudaMalloc would stall the
device, or a process whose memory pool already owns the GPU's memory).

The entry point keeps its scratch in an array inside the library instead of
taking a workspace pointer.  Checked here through the C ABI: it gives exactly
the outputs of `sb_permute` (integer and byte data, so equality, no
tolerance), on two calls in a row that share the array, with a different
problem size the second time so that leftovers of the first call would show.
This file sorts last so a `-x` run has executed every other test before it.
"""
import pytest
import torch

from sparse_b200._lib import lib


def _outputs(n, h, e, dev):
    r_cap = max(128, (n + 127) // 128 * 128)
    return {
        "rows": torch.zeros((r_cap, h), dtype=torch.bfloat16, device=dev),
        "offs": torch.zeros((e + 1,), dtype=torch.int32, device=dev),
        "slot_of_item": torch.zeros((n,), dtype=torch.int32, device=dev),
        "item_of_slot": torch.zeros((n,), dtype=torch.int32, device=dev),
        "slot_scale": torch.zeros((r_cap,), dtype=torch.bfloat16, device=dev),
        "tiles": torch.zeros((lib.sb_tile_table_ints(n, e),), dtype=torch.int32, device=dev),
    }


def _run_pair(n_tok, k, h, e, seed, dev):
    torch.manual_seed(seed)
    n = n_tok * k
    ids = torch.randint(0, e, (n,), dtype=torch.int32)
    ids[::7] = e - 1                                 # some skew, some empty experts likely
    x = torch.randn(n_tok, h).to(torch.bfloat16).to(dev)
    scale = torch.rand(n).to(torch.bfloat16).to(dev)
    ids = ids.to(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    a = _outputs(n, h, e, dev)
    ws_bytes = lib.sb_permute_workspace_bytes(n, e)
    ws = torch.empty((ws_bytes,), dtype=torch.uint8, device=dev)
    rc = lib.sb_permute(x.data_ptr(), ids.data_ptr(), scale.data_ptr(), n, k, h, e, ws.data_ptr(),
                        ws_bytes, a["rows"].data_ptr(), a["offs"].data_ptr(),
                        a["slot_of_item"].data_ptr(), a["item_of_slot"].data_ptr(),
                        a["slot_scale"].data_ptr(), a["tiles"].data_ptr(), stream)
    assert rc == 0, lib.sb_last_error_string()

    b = _outputs(n, h, e, dev)
    rc = lib.sb_permute_noalloc(x.data_ptr(), ids.data_ptr(), scale.data_ptr(), n, k, h, e,
                                b["rows"].data_ptr(), b["offs"].data_ptr(),
                                b["slot_of_item"].data_ptr(), b["item_of_slot"].data_ptr(),
                                b["slot_scale"].data_ptr(), b["tiles"].data_ptr(), stream)
    assert rc == 0, lib.sb_last_error_string()
    torch.cuda.synchronize()
    n_tiles = int(a["tiles"][0].item())
    assert int(b["tiles"][0].item()) == n_tiles
    for key in ("offs", "slot_of_item", "item_of_slot"):
        assert torch.equal(a[key], b[key]), key
    assert torch.equal(a["rows"][:n], b["rows"][:n])
    assert torch.equal(a["slot_scale"][:n], b["slot_scale"][:n])
    assert torch.equal(a["tiles"][:4 + 4 * n_tiles], b["tiles"][:4 + 4 * n_tiles])


@pytest.mark.gpu
def test_noalloc_matches_workspace_variant_on_two_calls_in_a_row():
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    _run_pair(n_tok=9000, k=4, h=128, e=60, seed=1, dev=dev)    # larger first (beyond the one-CTA path, so the scratch is used) ...
    _run_pair(n_tok=37, k=2, h=64, e=8, seed=2, dev=dev)        # ... then small: stale cells must not matter
    _run_pair(n_tok=9000, k=4, h=128, e=60, seed=3, dev=dev)


def test_noalloc_refuses_sizes_beyond_its_scratch():
    # 131072 scratch ints: ceil(n/128)*E above that is refused before any device work
    rc = lib.sb_permute_noalloc(None, None, None, 128 * 2049, 1, 64, 64, None, None, None, None,
                                None, None, None)
    assert rc == -2
    msg = lib.sb_last_error_string()
    assert b"sb_permute_noalloc" in msg and b"131072" in msg
