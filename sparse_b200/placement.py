"""Expert placement: which rank executes expert e for tokens that sit on rank s.

Restates the reference's placement inputs (utils/eval_core.py:556-917,
4569-4792, 6736-6769) as one object with one question: `dest_table(layer,
stage)` -> int [ep][E], row s = destination rank of every expert for source
rank s.  On one NVSwitch box every peer costs the same, so the topology tiers
of the reference reduce to "self 0, any peer 1" unless the file carries its
own cost matrix.

Accepted inputs (the on-disk schemas of the reference):
  round_robin                 owner = e % ep                         (:4573-4576)
  weighted_random_balanced    seeded, quota-balanced shuffle         (:556-579)
  scp   flat map              {"<layer*E+e>": rank}, missing -> e%ep (:4683-4685)
  scp_ep plain                {"placement": {layer: {expert: rank}}} (:796-814)
  scp_ep replicated v1/v2/v3  "replicas"{layer}{expert} -> [ranks], optional
                              "replica_choice_cost_matrix"[src][dst], optional
                              "rank_to_node", optional explicit
                              "dest_rank_table[_prefill|_decode]"    (:582-717, 817-917)
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence, Set

import numpy as np

REPLICATED_FORMATS = ("replicated_scp_ep_v1", "replicated_scp_ep_v2", "replicated_scp_ep_v3")
MODES = ("round_robin", "scp", "scp_ep", "weighted_random_balanced")


def round_robin(num_experts: int, ep: int) -> List[int]:
    return [e % ep for e in range(num_experts)]


def weighted_random_balanced(num_experts: int, ep: int, layer_idx: int,
                             rank_weights: Optional[Sequence[float]] = None,
                             seed: int = 1) -> List[int]:
    """Quota per rank proportional to its weight (largest remainders get the
    leftover experts), then a shuffle seeded by (seed, layer, E, ep)."""
    w = np.asarray(rank_weights if rank_weights is not None else [1.0] * ep, dtype=np.float64)
    w = w / w.sum()
    raw = w * float(num_experts)
    quota = np.floor(raw).astype(np.int64)
    left = int(num_experts - int(quota.sum()))
    if left > 0:
        by_frac = np.argsort(-(raw - quota))
        for i in range(left):
            quota[by_frac[i % len(by_frac)]] += 1
    pool: List[int] = []
    for r in range(ep):
        pool += [r] * int(quota[r])
    rng = np.random.default_rng(int(seed) + int(layer_idx) * 10007 + int(num_experts) * 97 + int(ep))
    rng.shuffle(pool)
    return [int(r) for r in pool]


def _row_from(obj, num_experts: int) -> List[int]:
    if isinstance(obj, dict):
        return [int(obj[str(e)]) for e in range(num_experts)]
    return [int(v) for v in list(obj)]


class Placement:
    """Placement of every layer's experts over `ep` ranks."""

    def __init__(self, mode: str, num_layers: int, num_experts: int, ep: int,
                 obj: Optional[dict] = None, rank_to_node: Optional[Sequence[int]] = None,
                 apply_prefill: bool = True, apply_decode: bool = False,
                 wrb_seed: int = 1, wrb_weights: Optional[Sequence[float]] = None):
        if mode not in MODES:
            raise ValueError("placement_mode must be one of %s, got %r" % (MODES, mode))
        if mode in ("scp", "scp_ep") and obj is None:
            raise ValueError("placement_mode=%s needs a placement file" % mode)
        if obj is not None and not isinstance(obj, dict):
            raise ValueError("SCP-EP placement must be a JSON object")
        self.mode, self.num_layers, self.num_experts, self.ep = mode, num_layers, num_experts, ep
        self.obj = obj or {}
        self.apply_prefill, self.apply_decode = apply_prefill, apply_decode
        self.wrb_seed, self.wrb_weights = wrb_seed, wrb_weights
        self.rank_to_node = [int(x) for x in rank_to_node] if rank_to_node is not None else None
        self._cache: Dict[tuple, List[List[int]]] = {}

    @classmethod
    def from_file(cls, mode: str, path: str, num_layers: int, num_experts: int, ep: int, **kw) -> "Placement":
        obj = None
        if mode in ("scp", "scp_ep"):
            with open(path) as fh:
                obj = json.load(fh)
        return cls(mode, num_layers, num_experts, ep, obj=obj, **kw)

    # -- helpers over the replicated formats ---------------------------------------
    @property
    def replicated(self) -> bool:
        return str(self.obj.get("format", "")) in REPLICATED_FORMATS

    def cost_matrix(self) -> List[List[float]]:
        raw = self.obj.get("replica_choice_cost_matrix")
        ep = self.ep
        if raw is not None:
            m = [[float(v) for v in row] for row in raw]
            if len(m) != ep or any(len(r) != ep for r in m):
                raise ValueError("replica_choice_cost_matrix must be [%d,%d], got %dx%d" % (
                    ep, ep, len(m), len(m[0]) if m else 0))
            return m
        nodes = [0] * ep
        if self.rank_to_node is not None and len(self.rank_to_node) == ep:
            nodes = list(self.rank_to_node)
        else:
            rn = self.obj.get("rank_to_node", {})
            if isinstance(rn, dict):
                nodes = [int(rn.get(str(r), rn.get(r, r))) for r in range(ep)]
        same = float(os.environ.get("SPARSE_TOPOLOGY_SAME_NODE_COST", "1.0") or 1.0)
        cross = float(os.environ.get("SPARSE_TOPOLOGY_CROSS_NODE_COST", "8.0") or 8.0)
        return [[0.0 if s == r else (same if nodes[s] == nodes[r] else cross) for r in range(ep)]
                for s in range(ep)]

    def replicas(self, layer: int) -> List[List[int]]:
        """Ranks allowed to execute each expert of `layer`."""
        if not self.replicated:
            return [[r] for r in self._single_owner(layer)]
        lay = self.obj.get("replicas", {})
        lk = str(int(layer))
        if lk not in lay:
            raise KeyError("replicated SCP-EP replicas missing layer %s" % lk)
        out = []
        for e in range(self.num_experts):
            if str(e) not in lay[lk]:
                raise KeyError("replicated SCP-EP replicas missing layer %s expert %d" % (lk, e))
            ranks = sorted(set(int(r) for r in lay[lk][str(e)]))
            if not ranks:
                raise ValueError("replicated SCP-EP expert has no replicas at layer %s expert %d" % (lk, e))
            for r in ranks:
                if r < 0 or r >= self.ep:
                    raise ValueError("replicated SCP-EP replica rank out of range at layer %s expert %d: %d" % (lk, e, r))
            out.append(ranks)
        return out

    def _stage_table(self, stage: str):
        st = (stage or "").strip().lower()
        if st in ("prefill", "decode") and self.obj.get("dest_rank_table_" + st) is not None:
            return self.obj["dest_rank_table_" + st]
        return self.obj.get("dest_rank_table")

    def _table_row(self, layer: int, source_node: int, stage: str) -> Optional[List[int]]:
        table = self._stage_table(stage)
        if table is None:
            return None
        lk, nk = str(int(layer)), str(int(source_node))
        if isinstance(table, dict):
            if lk not in table:
                raise KeyError("replicated SCP-EP dest_rank_table missing layer %s" % lk)
            if not isinstance(table[lk], dict) or nk not in table[lk]:
                raise KeyError("replicated SCP-EP dest_rank_table missing layer %s source_node %s" % (lk, nk))
            row = table[lk][nk]
        else:
            row = table[int(layer)][int(source_node)]
        out = _row_from(row, self.num_experts)
        if len(out) != self.num_experts:
            raise ValueError("dest_rank_table layer %d source_node %d length %d != %d" % (
                layer, source_node, len(out), self.num_experts))
        for e, r in enumerate(out):
            if r < 0 or r >= self.ep:
                raise ValueError("dest_rank_table rank out of range layer %d node %d expert %d: %d" % (
                    layer, source_node, e, r))
        return out

    def _source_node(self, rank: int) -> int:
        if self.rank_to_node is not None and 0 <= rank < len(self.rank_to_node):
            return int(self.rank_to_node[rank])
        return int(rank)

    def _single_owner(self, layer: int) -> List[int]:
        e_n, ep = self.num_experts, self.ep
        if self.mode == "round_robin":
            return round_robin(e_n, ep)
        if self.mode == "weighted_random_balanced":
            return weighted_random_balanced(e_n, ep, layer, self.wrb_weights, self.wrb_seed)
        if self.mode == "scp":
            out = []
            for e in range(e_n):
                v = self.obj.get(str(layer * e_n + e))
                out.append(int(v) if v is not None else e % ep)
            for e, r in enumerate(out):
                if r < 0 or r >= ep:
                    raise ValueError("SCP owner rank out of range at layer %d expert %d: %d" % (layer, e, r))
            return out
        plc = self.obj.get("placement", self.obj)
        if not isinstance(plc, dict):
            raise ValueError("SCP-EP placement JSON must contain a placement object")
        lk = str(int(layer))
        if lk not in plc:
            raise KeyError("SCP-EP placement missing layer %s" % lk)
        if not isinstance(plc[lk], dict):
            raise ValueError("SCP-EP placement layer %s must be an expert->rank object" % lk)
        out = []
        for e in range(e_n):
            if str(e) not in plc[lk]:
                raise KeyError("SCP-EP placement missing layer %s expert %d" % (lk, e))
            r = int(plc[lk][str(e)])
            if r < 0 or r >= ep:
                raise ValueError("SCP-EP owner rank out of range at layer %s expert %d: %d" % (lk, e, r))
            out.append(r)
        return out

    def assignment(self, layer: int, source_rank: int, stage: str = "") -> List[int]:
        """Destination rank of every expert for tokens on `source_rank`."""
        if self.mode in ("scp", "scp_ep"):
            st = (stage or "").strip().lower()
            if (st == "prefill" and not self.apply_prefill) or (st == "decode" and not self.apply_decode):
                return round_robin(self.num_experts, self.ep)
        if not self.replicated:
            return self._single_owner(layer)
        row = self._table_row(layer, self._source_node(source_rank), stage)
        if row is not None:
            return row
        cost = self.cost_matrix()
        out = []
        for e, ranks in enumerate(self.replicas(layer)):
            rr = e % self.ep
            out.append(min(ranks, key=lambda r: (cost[source_rank][r], 0 if r == rr else 1, r)))
        return out

    def dest_table(self, layer: int, stage: str = "") -> List[List[int]]:
        key = (int(layer), (stage or "").lower())
        if key not in self._cache:
            self._cache[key] = [self.assignment(layer, s, stage) for s in range(self.ep)]
        return self._cache[key]

    def receive_experts(self, layer: int, rank: int, stage: str = "") -> Set[int]:
        """Experts some source rank may send to `rank`; the weights it must be
        able to execute.  A rank also keeps its round-robin experts whenever one
        stage still routes round-robin (utils/eval_core.py:4743-4773)."""
        got = set()
        for st in ({stage} if stage else {"prefill", "decode"}):
            for row in self.dest_table(layer, st):
                got.update(e for e, d in enumerate(row) if d == rank)
        return got


def balanced_replicated_placement(expert_load: Sequence[Sequence[float]], ep: int,
                                  max_replicas: int = 0) -> dict:
    """A small greedy stand-in for the reference's offline solver, for synthetic
    workloads: experts are placed on the least-loaded rank in order of
    decreasing load; an expert heavier than the mean rank load is replicated on
    as many ranks as needed to bring its share under the mean, and every source
    rank is told to use replica (source mod replicas).  Writes the
    `replicated_scp_ep_v3` schema with explicit destination tables."""
    layers = len(expert_load)
    replicas, table = {}, {}
    for layer in range(layers):
        load = np.asarray(expert_load[layer], dtype=np.float64)
        e_n = load.shape[0]
        mean = load.sum() / ep if load.sum() > 0 else 1.0
        order = np.argsort(-load, kind="stable")
        rank_load = np.zeros(ep)
        reps: List[List[int]] = [[] for _ in range(e_n)]
        for e in order:
            want = int(min(ep, max(1, np.ceil(load[e] / mean)))) if load[e] > 0 else 1
            if max_replicas:
                want = min(want, max_replicas)
            targets = np.argsort(rank_load, kind="stable")[:want]
            for r in targets:
                reps[e].append(int(r))
                rank_load[r] += load[e] / want
        replicas[str(layer)] = {str(e): sorted(reps[e]) for e in range(e_n)}
        table[str(layer)] = {str(s): [sorted(reps[e])[s % len(reps[e])] for e in range(e_n)]
                             for s in range(ep)}
    return {"format": "replicated_scp_ep_v3", "replicas": replicas, "dest_rank_table": table,
            "rank_to_node": {str(r): r for r in range(ep)}, "source_nodes": list(range(ep))}
