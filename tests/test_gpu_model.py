"""GPU: the kernels of the decode loop around the MoE layers (RMSNorm with the
residual add, rotary embedding + cache append, decode attention) against plain
PyTorch fp32 restatements, and the model harness against itself: decoding a
token with the cache gives what a longer prefill gives, a replayed CUDA graph
gives the bits of the eager step."""
import math

import pytest
import torch

from sparse_b200 import _lib
from sparse_b200._lib import lib, check

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _stream():
    return torch.cuda.current_stream(torch.device(DEV)).cuda_stream


@pytest.mark.parametrize("t,h,with_delta", [(1, 256, True), (7, 2048, True), (300, 2048, False), (5, 512, False)])
def test_add_rmsnorm(t, h, with_delta):
    torch.manual_seed(t + h)
    bf = torch.bfloat16
    resid = torch.randn(t, h).to(bf).to(DEV)
    delta = torch.randn(t, h).to(bf).to(DEV) if with_delta else None
    w = (1.0 + 0.1 * torch.randn(h)).to(bf).to(DEV)
    eps = 1e-6
    hsum = (resid.float() + delta.float()).to(bf) if with_delta else resid.clone()
    x = hsum.float()
    want = w.float() * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)).to(bf).float()
    out = torch.empty_like(resid)
    r = resid.clone()
    check(lib.sb_add_rmsnorm(r.data_ptr(), delta.data_ptr() if with_delta else None, None, w.data_ptr(), eps, t, h,
                             out.data_ptr(), _stream()), "sb_add_rmsnorm")
    torch.cuda.synchronize()
    assert torch.equal(r, hsum), "the residual stream is the bf16 sum"
    # rsqrt and the fp32 mean may round differently: one bf16 step at most
    assert float((out.float() - want).abs().max()) <= 2.0 ** -7 * float(want.abs().max())
    assert float((out.float() == want.to(bf).float()).float().mean()) > 0.98


def _rope_ref(x, pos, rope_dim, theta):
    """x [T, heads, d]; rotate pairs (i, i + rope_dim/2) of the first rope_dim elements."""
    half = rope_dim // 2
    inv = theta ** (-2.0 * torch.arange(half, dtype=torch.float32, device=x.device) / rope_dim)
    ang = pos.float().unsqueeze(1) * inv.unsqueeze(0)
    cs, sn = ang.cos().to(torch.bfloat16).float(), ang.sin().to(torch.bfloat16).float()
    cs, sn = cs.unsqueeze(1), sn.unsqueeze(1)
    a, b = x[..., :half].float(), x[..., half:rope_dim].float()
    ra = (a * cs).to(torch.bfloat16).float() + (-b * sn).to(torch.bfloat16).float()
    rb = (b * cs).to(torch.bfloat16).float() + (a * sn).to(torch.bfloat16).float()
    out = x.clone()
    out[..., :half] = ra.to(torch.bfloat16)
    out[..., half:rope_dim] = rb.to(torch.bfloat16)
    return out


@pytest.mark.parametrize("n_q,n_kv,dk,dv,rope_dim", [(16, 16, 128, 128, 128), (16, 16, 192, 128, 64), (4, 2, 64, 64, 64)])
def test_rope_append(n_q, n_kv, dk, dv, rope_dim):
    torch.manual_seed(dk)
    bf = torch.bfloat16
    b, s_max, t = 3, 40, 11
    q = torch.randn(t, n_q, dk).to(bf).to(DEV)
    k = torch.randn(t, n_kv, dk).to(bf).to(DEV)
    v = torch.randn(t, n_kv, dv).to(bf).to(DEV)
    seq = torch.randint(0, b, (t,), dtype=torch.int32)
    pos = torch.randperm(s_max)[:t].to(torch.int32)          # distinct rows
    seq_d, pos_d = seq.to(DEV), pos.to(DEV)
    ck = torch.zeros(b, s_max, n_kv, dk, dtype=bf, device=DEV)
    cv = torch.zeros(b, s_max, n_kv, dv, dtype=bf, device=DEV)
    want_q = _rope_ref(q, pos_d, rope_dim, 10000.0)
    want_k = _rope_ref(k, pos_d, rope_dim, 10000.0)
    qq = q.clone()
    check(lib.sb_rope_append(qq.data_ptr(), k.data_ptr(), v.data_ptr(), seq_d.data_ptr(), pos_d.data_ptr(), t, n_q,
                             n_kv, dk, dv, rope_dim, 10000.0, s_max, ck.data_ptr(), cv.data_ptr(), 0, 0, 0, _stream()),
          "sb_rope_append")
    torch.cuda.synchronize()
    # sin/cos of the device's fast path against libm's: a bf16 step on a few elements at most
    for got, want in ((qq, want_q), (ck[seq.long(), pos.long()], want_k)):
        d = (got.float() - want.float()).abs()
        assert float(d.max()) <= 2.0 ** -6 * float(want.float().abs().max())
        assert float((d == 0).float().mean()) > 0.97
    assert torch.equal(cv[seq.long(), pos.long()], v)
    untouched = torch.ones(b, s_max, dtype=torch.bool)
    untouched[seq.long(), pos.long()] = False
    assert float(ck[untouched.to(DEV)].abs().max()) == 0.0


@pytest.mark.parametrize("n_q,n_kv,dk,dv,lens,n_split", [
    (16, 16, 128, 128, [1, 17, 300, 2048], 5), (16, 16, 192, 128, [64, 1000], 12), (4, 2, 64, 64, [3, 0, 9], 1)])
def test_attn_decode(n_q, n_kv, dk, dv, lens, n_split):
    torch.manual_seed(dk + n_split)
    bf = torch.bfloat16
    b, s_max = len(lens), max(max(lens), 1) + 5
    q = torch.randn(b, n_q, dk).to(bf).to(DEV)
    ck = torch.randn(b, s_max, n_kv, dk).to(bf).to(DEV)
    cv = torch.randn(b, s_max, n_kv, dv).to(bf).to(DEV)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    ws = torch.empty(lib.sb_attn_decode_workspace_bytes(b, n_q, dv, n_split), dtype=torch.uint8, device=DEV)
    out = torch.empty(b, n_q, dv, dtype=bf, device=DEV)
    scale = 1.0 / math.sqrt(dk)
    check(lib.sb_attn_decode(q.data_ptr(), 0, ck.data_ptr(), cv.data_ptr(), seq_lens.data_ptr(), b, n_q, n_kv, dk, dv,
                             s_max, scale, n_split, ws.data_ptr(), ws.numel(), out.data_ptr(), _stream()),
          "sb_attn_decode")
    torch.cuda.synchronize()
    rep = n_q // n_kv
    for i, n in enumerate(lens):
        if n == 0:
            assert float(out[i].abs().max()) == 0.0
            continue
        kk = ck[i, :n].float().repeat_interleave(rep, dim=1)         # [n, n_q, dk]
        vv = cv[i, :n].float().repeat_interleave(rep, dim=1)
        s = torch.einsum("hd,nhd->hn", q[i].float(), kk) * scale
        want = torch.einsum("hn,nhd->hd", torch.softmax(s, dim=-1), vv)
        got = out[i].float()
        assert float((got - want).abs().max()) < 2e-2
        assert float((got - want).norm() / want.norm()) < 5e-3


def test_kernels_take_column_slices_of_a_fused_projection():
    """q, k, v as strided column slices of one [T, q+k+v] buffer give the bits of packed tensors."""
    torch.manual_seed(4)
    bf = torch.bfloat16
    n_q, n_kv, dk, dv, t, b, s_max = 4, 2, 64, 64, 5, 5, 16
    fused = torch.randn(t, n_q * dk + n_kv * dk + n_kv * dv).to(bf).to(DEV)
    q, k, v = fused[:, :n_q * dk], fused[:, n_q * dk:n_q * dk + n_kv * dk], fused[:, n_q * dk + n_kv * dk:]
    seq = torch.arange(t, dtype=torch.int32, device=DEV)
    pos = torch.full((t,), 3, dtype=torch.int32, device=DEV)
    outs = []
    for packed in (False, True):
        buf = fused.clone()
        qq = buf[:, :n_q * dk]
        kk, vv = buf[:, n_q * dk:n_q * dk + n_kv * dk], buf[:, n_q * dk + n_kv * dk:]
        if packed:
            qq, kk, vv = qq.contiguous(), kk.contiguous(), vv.contiguous()
        ck = torch.zeros(b, s_max, n_kv, dk, dtype=bf, device=DEV)
        cv = torch.zeros(b, s_max, n_kv, dv, dtype=bf, device=DEV)
        check(lib.sb_rope_append(qq.data_ptr(), kk.data_ptr(), vv.data_ptr(), seq.data_ptr(), pos.data_ptr(), t, n_q,
                                 n_kv, dk, dv, dk, 10000.0, s_max, ck.data_ptr(), cv.data_ptr(), qq.stride(0),
                                 kk.stride(0), vv.stride(0), _stream()), "sb_rope_append")
        lens = torch.full((b,), 4, dtype=torch.int32, device=DEV)
        ws = torch.empty(lib.sb_attn_decode_workspace_bytes(b, n_q, dv, 2), dtype=torch.uint8, device=DEV)
        out = torch.empty(b, n_q * dv, dtype=bf, device=DEV)
        check(lib.sb_attn_decode(qq.data_ptr(), qq.stride(0), ck.data_ptr(), cv.data_ptr(), lens.data_ptr(), b, n_q,
                                 n_kv, dk, dv, s_max, 0.125, 2, ws.data_ptr(), ws.numel(), out.data_ptr(), _stream()),
              "sb_attn_decode")
        torch.cuda.synchronize()
        outs.append((qq.clone().contiguous(), ck.clone(), cv.clone(), out.clone()))
    for a, c in zip(outs[0], outs[1]):
        assert torch.equal(a, c)


def _tiny_model(batch, max_seq, **kw):
    from sparse_b200.model import ShapedMoeModel, TINY_MODEL
    return ShapedMoeModel(TINY_MODEL, torch.device(DEV), batch, max_seq, seed=3, **kw)


def test_decode_with_cache_agrees_with_longer_prefill():
    torch.manual_seed(0)
    b, s = 3, 37
    ids = torch.randint(0, 512, (b, s + 1), device=DEV)
    m1 = _tiny_model(b, 64)
    full = m1.prefill(ids)                                  # logits after s+1 tokens
    m2 = _tiny_model(b, 64)
    m2.prefill(ids[:, :s])
    m2.cur_ids.copy_(ids[:, s])
    m2._decode_body()                                       # consumes token s with the cache
    torch.cuda.synchronize()
    # the decode step's own logits are not returned; compare what it chose with the long prefill's choice
    want_next = full.argmax(dim=-1)
    assert torch.equal(m2.cur_ids, want_next)
    assert bool((m2.cur_pos == s + 1).all())
    # the cache rows written by the decode step equal the ones the long prefill wrote
    for l1, l2 in zip(m1.layers, m2.layers):
        a, c = l1.cache_k[:, s].float(), l2.cache_k[:, s].float()
        assert float((a - c).norm() / a.norm()) < 2e-2
    m1.check_status(); m2.check_status()


def test_graph_replayed_decode_equals_eager_decode():
    from sparse_b200.context import Metrics
    from sparse_b200.model import RunningStats, greedy_decode_profiled
    torch.manual_seed(1)
    b, s, new = 4, 20, 12
    ids = torch.randint(0, 512, (b, s), device=DEV)
    outs = []
    for use_graph in (False, True):
        m = _tiny_model(b, 64)
        metrics = Metrics()
        metrics.decode_step_stats = RunningStats()
        out = greedy_decode_profiled(m, ids, torch.ones_like(ids), new, None, metrics, True, use_graph=use_graph,
                                     per_step_sync=not use_graph)
        assert out.shape == (b, s + new) and torch.equal(out[:, :s], ids)
        assert metrics.wall_prefill_ms > 0 and metrics.wall_decode_ms > 0 and metrics.wall_ttft_ms > 0
        if not use_graph:
            assert len(metrics.decode_step_stats.values_ms) == new - 1
        outs.append(out)
    assert torch.equal(outs[0], outs[1])


def test_chunked_prefill_equals_single_chunk_prefill():
    torch.manual_seed(2)
    b, s = 2, 50
    ids = torch.randint(0, 512, (b, s), device=DEV)
    one = _tiny_model(b, 64, chunk_tokens=4096).prefill(ids)
    many = _tiny_model(b, 64, chunk_tokens=2 * 16).prefill(ids)         # chunks of 16 positions
    assert torch.equal(one.argmax(-1), many.argmax(-1))
    assert float((one - many).abs().max()) < 5e-2 * float(one.abs().max())


def test_deepseek_shaped_attention_layout_runs():
    """MLA-shaped attention (qk 192 = rope 64 + nope 128, v 128, latent 512) and a dense first layer."""
    from sparse_b200 import synth
    from sparse_b200.model import ModelConfig, ShapedMoeModel
    cfg = ModelConfig("mla-small", 2, 256, 16, 16, 192, 128, 64, 1.0e4, 1e-6, 512, synth.TINY, {0: 320}, "mla", 512, False)
    m = ShapedMoeModel(cfg, torch.device(DEV), 2, 48, seed=5)
    ids = torch.randint(0, 512, (2, 30), device=DEV)
    full = m.prefill(ids)
    m2 = ShapedMoeModel(cfg, torch.device(DEV), 2, 48, seed=5)
    m2.prefill(ids[:, :29])
    m2.cur_ids.copy_(ids[:, 29])
    m2._decode_body()
    torch.cuda.synchronize()
    assert torch.equal(m2.cur_ids, full.argmax(dim=-1))
    m.check_status(); m2.check_status()
