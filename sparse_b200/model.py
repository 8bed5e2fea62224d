"""A shaped MoE language model around the MoE blocks, and the greedy decode loop.

What the reference gets from Transformers (`build_model_and_tokenizer`,
utils/eval_core.py:17759-18221: load the model, swap every `layer.mlp` for a
`DistributedSparseMoeBlock`) and drives with `greedy_decode_profiled`
(utils/eval_core.py:18464-18607: one prefill, then one model call per
generated token with a growing key/value cache), built here for randomly
initialised models of the two benchmark shapes:

* Qwen1.5-MoE-A2.7B-shaped: 24 layers, hidden 2048, 16 heads of 128 with RoPE,
  RMSNorm, vocabulary 151936, the Qwen MoE block in every layer;
* DeepSeek-V2-Lite-shaped: 27 layers, layer 0 a dense SwiGLU FFN (10944), MLA
  attention (16 heads, kv_lora_rank 512, qk_nope 128, qk_rope 64, v 128) with
  keys and values decompressed into the cache per head, vocabulary 102400.

Per decode step every layer runs: RMSNorm (fused with the residual add) ->
q/k/v projections (library GEMMs) -> rotary embedding + cache append ->
decode attention over the cache -> output projection -> RMSNorm -> MoE block.
All of it is stream-ordered with nothing read back, so the whole step (all
layers, the lm_head GEMM and the argmax) is recorded once into a CUDA graph
and replayed per token; positions and token ids live in device buffers that
the graph itself advances.  Prefill runs the same layers on chunks of the
prompt with the library's fused attention over the cache.

Under expert parallelism every rank holds the whole model except the experts
it does not own, and its own share of the sequences (data-parallel attention,
expert-parallel MoE), as the reference's EP group does.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from . import _lib, ops, synth
from ._lib import lib, check
from .block import B200MoeBlock
from .context import Metrics, SparseContext
from .layer import LayerWeights


@dataclass
class ModelConfig:
    name: str
    layers: int
    hidden: int
    n_heads: int
    n_kv_heads: int
    qk_dim: int                 # per-head query/key width (rope part first)
    v_dim: int
    rope_dim: int
    rope_theta: float
    rms_eps: float
    vocab: int
    moe: synth.BlockShape
    dense_layers: Dict[int, int] = field(default_factory=dict)     # layer -> dense FFN width
    attention: str = "mha"      # "mha" or "mla"
    kv_lora_rank: int = 0
    qkv_bias: bool = False


QWEN_MODEL = ModelConfig("qwen1.5-moe-a2.7b-shaped", 24, 2048, 16, 16, 128, 128, 128, 1.0e6, 1e-6, 151936,
                         synth.QWEN_MOE, {}, "mha", 0, True)
DEEPSEEK_MODEL = ModelConfig("deepseek-v2-lite-shaped", 27, 2048, 16, 16, 192, 128, 64, 1.0e4, 1e-6, 102400,
                             synth.DEEPSEEK_V2_LITE, {0: 10944}, "mla", 512, False)
TINY_MODEL = ModelConfig("tiny", 2, 256, 4, 4, 64, 64, 64, 1.0e4, 1e-6, 512, synth.TINY, {}, "mha", 0, True)


def _normal(shape, device, seed: int, std: float = 0.02) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return torch.empty(shape, dtype=torch.float32, device=device).normal_(0.0, std, generator=g).to(torch.bfloat16)


def random_layer_weights(shape: synth.BlockShape, device: torch.device, seed: int, owned: Sequence[int]) -> LayerWeights:
    """MoE weights drawn on the device: N(0, 0.02), one seed per tensor so that an
    expert has the same weights on whichever rank holds it."""
    lw = LayerWeights(shape.hidden, shape.inter, shape.num_experts, max(1, len(owned)), shape.shared_inter, device)
    lw.set_router(_normal((shape.num_experts, shape.hidden), device, seed * 1000003 + 1))
    slot_of = [-1] * shape.num_experts
    for slot, e in enumerate(owned):
        lw.w13[slot].copy_(_normal((2 * shape.inter, shape.hidden), device, seed * 1000003 + 100 + 2 * e))
        lw.w2[slot].copy_(_normal((shape.hidden, shape.inter), device, seed * 1000003 + 101 + 2 * e))
        slot_of[e] = slot
    lw.set_slot_map(slot_of)
    if shape.shared_inter:
        lw.shared_w13[0].copy_(_normal((2 * shape.shared_inter, shape.hidden), device, seed * 1000003 + 2))
        lw.shared_w2[0].copy_(_normal((shape.hidden, shape.shared_inter), device, seed * 1000003 + 3))
        if shape.shared_gate:
            lw.shared_gate_w = _normal((shape.hidden,), device, seed * 1000003 + 4).contiguous()
    return lw


class _Layer:
    pass


class ShapedMoeModel:
    """Random-init model of a `ModelConfig` on one GPU (one rank of an EP group)."""

    def __init__(self, cfg: ModelConfig, device: torch.device, batch: int, max_seq: int, seed: int = 0,
                 ep_rank: int = 0, ep_size: int = 1, process_group=None, owner_of: Optional[Sequence[int]] = None,
                 chunk_tokens: int = 4096):
        self.cfg, self.device, self.batch, self.max_seq = cfg, device, batch, max_seq
        self.ep_rank, self.ep_size = ep_rank, ep_size
        h, bf = cfg.hidden, torch.bfloat16
        dev_index = device.index if device.index is not None else torch.cuda.current_device()
        _lib.init_device(dev_index)
        self.chunk_tokens = max(batch, chunk_tokens // batch * batch)     # tokens per prefill chunk (all sequences)
        moe_tokens = max(self.chunk_tokens, batch)
        self.embed = _normal((cfg.vocab, h), device, seed * 7919 + 11)
        self.lm_head = _normal((cfg.vocab, h), device, seed * 7919 + 12)
        self.final_norm = torch.ones((h,), dtype=bf, device=device)
        e_n = cfg.moe.num_experts
        if owner_of is None:
            owner_of = [e % ep_size for e in range(e_n)]
        owned = [e for e in range(e_n) if owner_of[e] == ep_rank] if ep_size > 1 else list(range(e_n))
        self.layers: List[_Layer] = []
        nh, nkv, dk, dv = cfg.n_heads, cfg.n_kv_heads, cfg.qk_dim, cfg.v_dim
        for l in range(cfg.layers):
            ly = _Layer()
            s0 = seed * 7919 + 1000 * (l + 1)
            ly.ln1 = torch.ones((h,), dtype=bf, device=device)
            ly.ln2 = torch.ones((h,), dtype=bf, device=device)
            if cfg.attention == "mla":
                nope = dk - cfg.rope_dim
                ly.wq = _normal((nh * dk, h), device, s0 + 1)
                ly.wkv_a = _normal((cfg.kv_lora_rank + cfg.rope_dim, h), device, s0 + 2)
                ly.kv_norm = torch.ones((cfg.kv_lora_rank,), dtype=bf, device=device)
                ly.wkv_b = _normal((nh * (nope + dv), cfg.kv_lora_rank), device, s0 + 3)
                ly.bqkv = None
            else:
                ly.wqkv = _normal((nh * dk + nkv * dk + nkv * dv, h), device, s0 + 1)
                ly.bqkv = _normal((nh * dk + nkv * dk + nkv * dv,), device, s0 + 2) if cfg.qkv_bias else None
            ly.wo = _normal((h, nh * dv), device, s0 + 4)
            ly.cache_k = torch.zeros((batch, max_seq, nkv, dk), dtype=bf, device=device)
            ly.cache_v = torch.zeros((batch, max_seq, nkv, dv), dtype=bf, device=device)
            if l in cfg.dense_layers:
                inter = cfg.dense_layers[l]
                ly.dense_w13 = _normal((1, 2 * inter, h), device, s0 + 5)
                ly.dense_w2 = _normal((1, h, inter), device, s0 + 6)
                ly.block = None
            else:
                lw = random_layer_weights(cfg.moe, device, s0 + 7, owned)
                owner = None if ep_size == 1 else list(owner_of)
                ly.block = B200MoeBlock(lw, cfg.moe.top_k, moe_tokens, norm_topk_prob=cfg.moe.norm_topk_prob,
                                        fp32_router_logits=cfg.attention == "mla", ep_rank=ep_rank, ep_size=ep_size,
                                        process_group=process_group, owner=owner)
            self.layers.append(ly)
        # enough key splits for about six CTAs per SM: a CTA streams its keys with
        # a few hundred bytes in flight per warp, so bandwidth comes from CTA count
        sms = max(1, int(lib.sb_device_sm_count()) or 148)
        self.n_split = max(1, min(64, (6 * sms + batch * nh - 1) // (batch * nh)))
        ws = lib.sb_attn_decode_workspace_bytes(batch, nh, dv, self.n_split)
        self.attn_ws = torch.empty((ws,), dtype=torch.uint8, device=device)
        # decode-step state advanced by the graph itself
        self.cur_ids = torch.zeros((batch,), dtype=torch.int64, device=device)
        self.cur_pos = torch.zeros((batch,), dtype=torch.int32, device=device)
        self.seq_ids = torch.arange(batch, dtype=torch.int32, device=device)
        self.seq_lens = torch.zeros((batch,), dtype=torch.int32, device=device)
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self.status_checked = False

    # -- pieces ----------------------------------------------------------------------------
    def _s(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _norm(self, resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(resid)
        check(lib.sb_add_rmsnorm(resid.data_ptr(), delta.data_ptr() if delta is not None else None, None,
                                 weight.data_ptr(), self.cfg.rms_eps, resid.shape[0], resid.shape[1],
                                 out.data_ptr(), self._s()), "sb_add_rmsnorm")
        return out

    def _qkv(self, ly: _Layer, x: torch.Tensor):
        cfg = self.cfg
        nh, nkv, dk, dv, t = cfg.n_heads, cfg.n_kv_heads, cfg.qk_dim, cfg.v_dim, x.shape[0]
        if cfg.attention == "mla":
            nope, rope = dk - cfg.rope_dim, cfg.rope_dim
            q = F.linear(x, ly.wq)                                     # per head: [rope | nope]
            kv_a = F.linear(x, ly.wkv_a)
            c_kv = kv_a[:, :cfg.kv_lora_rank].contiguous()
            k_pe = kv_a[:, cfg.kv_lora_rank:]
            c_kv = self._norm(c_kv, None, ly.kv_norm)
            kv = F.linear(c_kv, ly.wkv_b).view(t, nh, nope + dv)
            k = torch.cat([k_pe.unsqueeze(1).expand(t, nh, rope), kv[:, :, :nope]], dim=2).reshape(t, nh * dk)
            v = kv[:, :, nope:].reshape(t, nh * dv)
            return q, k, v
        # column slices of the fused projection: the kernels take the token stride
        qkv = F.linear(x, ly.wqkv, ly.bqkv)
        return qkv[:, :nh * dk], qkv[:, nh * dk:nh * dk + nkv * dk], qkv[:, nh * dk + nkv * dk:]

    def _rope_append(self, ly: _Layer, q, k, v, seq_of_token, pos_of_token) -> None:
        cfg = self.cfg
        check(lib.sb_rope_append(q.data_ptr(), k.data_ptr(), v.data_ptr(), seq_of_token.data_ptr(),
                                 pos_of_token.data_ptr(), q.shape[0], cfg.n_heads, cfg.n_kv_heads, cfg.qk_dim,
                                 cfg.v_dim, cfg.rope_dim, cfg.rope_theta, self.max_seq, ly.cache_k.data_ptr(),
                                 ly.cache_v.data_ptr(), q.stride(0), k.stride(0), v.stride(0), self._s()),
              "sb_rope_append")

    # When set to a list, every MoE call appends (layer index, input rows, chosen experts):
    # what `rs_train.collect_pairs` turns into predictor training data.
    trace = None

    def _mlp(self, ly: _Layer, x: torch.Tensor) -> torch.Tensor:
        if ly.block is None:
            out, _ = ops.grouped_swiglu(x, ly.dense_w13, ly.dense_w2, dense_rows=x.shape[0])
            return out[:x.shape[0]]
        out = torch.empty_like(x)
        ly.block.forward_device(x, out)
        if self.trace is not None:
            self.trace.append((self.layers.index(ly), x.clone(), ly.block.topk(x.shape[0])[0].clone()))
        return out

    # -- prefill -----------------------------------------------------------------------------
    def _prefill_chunk(self, ids: torch.Tensor, past: int) -> torch.Tensor:
        """ids [B, Tc] at positions past..past+Tc-1 -> hidden state of every token [B*Tc, H] (before the final norm)."""
        cfg, b, tc = self.cfg, ids.shape[0], ids.shape[1]
        nh, nkv, dk, dv = cfg.n_heads, cfg.n_kv_heads, cfg.qk_dim, cfg.v_dim
        t = b * tc
        resid = self.embed.index_select(0, ids.reshape(-1))
        seq = self.seq_ids[:b].repeat_interleave(tc)
        pos = (torch.arange(tc, dtype=torch.int32, device=self.device) + past).repeat(b)
        kv_len = past + tc
        mask = None
        if past > 0:
            i = torch.arange(tc, device=self.device).unsqueeze(1)
            j = torch.arange(kv_len, device=self.device).unsqueeze(0)
            mask = j <= (i + past)
        delta = None
        for ly in self.layers:
            x = self._norm(resid, delta, ly.ln1)
            q, k, v = self._qkv(ly, x)
            self._rope_append(ly, q, k, v, seq, pos)
            qh = q.reshape(b, tc, nh, dk).transpose(1, 2)
            kh = ly.cache_k[:b, :kv_len].transpose(1, 2)
            vh = ly.cache_v[:b, :kv_len].transpose(1, 2)
            if nkv != nh:
                kh = kh.repeat_interleave(nh // nkv, dim=1)
                vh = vh.repeat_interleave(nh // nkv, dim=1)
            if dv != dk:
                vh = F.pad(vh, (0, dk - dv))
            att = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask, is_causal=mask is None,
                                                 scale=1.0 / math.sqrt(dk))
            att = att[..., :dv].transpose(1, 2).reshape(t, nh * dv)
            attn_out = F.linear(att, ly.wo)
            x2 = self._norm(resid, attn_out, ly.ln2)
            delta = self._mlp(ly, x2)
        check(lib.sb_add_rmsnorm(resid.data_ptr(), delta.data_ptr(), None, None, cfg.rms_eps, t, cfg.hidden, None,
                                 self._s()), "sb_add_rmsnorm")
        return resid

    def prefill(self, input_ids: torch.Tensor) -> torch.Tensor:
        """input_ids [B, S] -> logits of the last position [B, V] (fp32); fills the cache."""
        b, s = input_ids.shape
        if b != self.batch or s >= self.max_seq:
            raise RuntimeError("model was built for batch %d and fewer than %d positions" % (self.batch, self.max_seq))
        per_seq = max(1, self.chunk_tokens // b)
        last = None
        for p0 in range(0, s, per_seq):
            chunk = input_ids[:, p0:p0 + per_seq].contiguous()
            hidden = self._prefill_chunk(chunk, p0)
            last = hidden.view(b, chunk.shape[1], -1)[:, -1, :].contiguous()
        normed = self._norm(last, None, self.final_norm)
        self.cur_pos.fill_(s)
        return F.linear(normed, self.lm_head).float()

    # -- decode ------------------------------------------------------------------------------
    def _decode_body(self) -> None:
        """One token per sequence: reads cur_ids/cur_pos, appends to the cache,
        writes the next ids back and advances the positions."""
        cfg, b = self.cfg, self.batch
        nh, nkv, dk, dv = cfg.n_heads, cfg.n_kv_heads, cfg.qk_dim, cfg.v_dim
        resid = self.embed.index_select(0, self.cur_ids)
        torch.add(self.cur_pos, 1, out=self.seq_lens)
        delta = None
        for ly in self.layers:
            x = self._norm(resid, delta, ly.ln1)
            q, k, v = self._qkv(ly, x)
            self._rope_append(ly, q, k, v, self.seq_ids, self.cur_pos)
            att = torch.empty((b, nh * dv), dtype=torch.bfloat16, device=self.device)
            check(lib.sb_attn_decode(q.data_ptr(), q.stride(0), ly.cache_k.data_ptr(), ly.cache_v.data_ptr(),
                                     self.seq_lens.data_ptr(), b, nh, nkv, dk, dv, self.max_seq,
                                     1.0 / math.sqrt(dk), self.n_split, self.attn_ws.data_ptr(),
                                     self.attn_ws.numel(), att.data_ptr(), self._s()), "sb_attn_decode")
            attn_out = F.linear(att, ly.wo)
            x2 = self._norm(resid, attn_out, ly.ln2)
            delta = self._mlp(ly, x2)
        normed = self._norm(resid, delta, self.final_norm)
        logits = F.linear(normed, self.lm_head)
        self.cur_ids.copy_(torch.argmax(logits.float(), dim=-1))
        self.cur_pos.add_(1)

    def decode_step(self, use_graph: bool = True) -> torch.Tensor:
        """Advance every sequence by one token; returns the new ids (a view of the
        device buffer the next step reads)."""
        if not use_graph:
            self._decode_body()
            return self.cur_ids
        if self._graph is None:
            stream = torch.cuda.current_stream(self.device)
            # state the recording must not disturb
            ids0, pos0 = self.cur_ids.clone(), self.cur_pos.clone()
            self._decode_body()                      # un-recorded pass: one-time set-up happens here
            self.cur_ids.copy_(ids0)
            self.cur_pos.copy_(pos0)
            cap = torch.cuda.Stream(device=self.device)
            cap.wait_stream(stream)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(cap):
                with torch.cuda.graph(graph, stream=cap, capture_error_mode="thread_local"):
                    self._decode_body()
            stream.wait_stream(cap)
            self._graph = graph
        self._graph.replay()
        return self.cur_ids

    def check_status(self) -> None:
        for ly in self.layers:
            if ly.block is not None:
                ly.block.check_status()


class RunningStats:
    """Per-step latencies with the summary keys of the reference (utils/eval_core.py:1252-1278)."""

    def __init__(self):
        self.values_ms: List[float] = []

    def add_ms(self, v: float) -> None:
        self.values_ms.append(float(v))

    def reset(self) -> None:
        self.values_ms.clear()

    def summary(self, prefix: str = "") -> Dict[str, float]:
        if not self.values_ms:
            return {prefix + k: 0.0 for k in ("avg_ms", "p50_ms", "p95_ms", "p99_ms", "max_ms")}
        v = sorted(self.values_ms)
        n = len(v)

        def pct(p):
            x = (n - 1) * p / 100.0
            lo, hi = int(math.floor(x)), int(math.ceil(x))
            return v[lo] + (v[hi] - v[lo]) * (x - lo)

        return {prefix + "avg_ms": sum(v) / n, prefix + "p50_ms": pct(50), prefix + "p95_ms": pct(95),
                prefix + "p99_ms": pct(99), prefix + "max_ms": v[-1]}


def greedy_decode_profiled(model: ShapedMoeModel, input_ids: torch.Tensor, attention_mask, max_new_tokens: int,
                           env, metrics: Optional[Metrics], measure_ttft: bool, use_graph: bool = True,
                           per_step_sync: bool = False) -> torch.Tensor:
    """Prefill, then `max_new_tokens - 1` decode steps, greedy; returns
    [B, prompt + max_new_tokens] ids.  Same arguments and the same wall-clock
    bookkeeping as the reference's loop (utils/eval_core.py:18464-18607):
    `metrics.wall_prefill_ms`, `wall_ttft_ms`, `wall_decode_ms`, and one sample
    per step in `metrics.decode_step_stats` when `per_step_sync` asks for the
    reference's per-step synchronisation.  `attention_mask` must be all ones
    (prompts of equal length), as the launchers produce with `--prompt-len`."""
    if attention_mask is not None and not bool(attention_mask.all()):
        raise NotImplementedError("padded prompts are not built; pass prompts of equal length")
    dev = model.device
    input_ids = input_ids.to(dev)
    torch.cuda.reset_peak_memory_stats(dev)
    SparseContext.current_phase = "prefill"
    SparseContext.begin_runtime_call(0)
    t0 = time.perf_counter()
    logits = model.prefill(input_ids)
    next_token = torch.argmax(logits, dim=-1)
    model.cur_ids.copy_(next_token)
    torch.cuda.synchronize(dev)
    prefill_ms = (time.perf_counter() - t0) * 1e3
    generated = [next_token.clone()]
    SparseContext.current_phase = "decode"
    t1 = time.perf_counter()
    for step in range(max_new_tokens - 1):
        SparseContext.begin_runtime_call(step + 1)
        ts = time.perf_counter()
        ids = model.decode_step(use_graph=use_graph)
        generated.append(ids.clone())
        if per_step_sync:
            torch.cuda.synchronize(dev)
            if metrics is not None and metrics.decode_step_stats is not None:
                metrics.decode_step_stats.add_ms((time.perf_counter() - ts) * 1e3)
    torch.cuda.synchronize(dev)
    decode_ms = (time.perf_counter() - t1) * 1e3
    model.check_status()
    if metrics is not None:
        metrics.wall_prefill_ms = prefill_ms
        metrics.wall_decode_ms = decode_ms
        if measure_ttft:
            metrics.wall_ttft_ms = prefill_ms
        metrics.peak_allocated_mb = torch.cuda.max_memory_allocated(dev) / (1024 ** 2)
        metrics.peak_reserved_mb = torch.cuda.max_memory_reserved(dev) / (1024 ** 2)
        metrics.finalize_events()
    SparseContext.current_phase = "none"
    return torch.cat([input_ids, torch.stack(generated, dim=1)], dim=1)
