"""Expert co-activation graph, balanced placement and per-token prefetch plans
(reference: src/inferutil/routing.py:47-263).

Nodes are ``layer * n_experts + expert``; an edge counts how often two experts fire for the same token in one
layer or in adjacent layers. ``ingest_telemetry`` consumes the server's ``x_telemetry`` dictionaries.
"""
from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass, field
from itertools import combinations
from typing import Dict, Iterable, List, Tuple


def _key(a: int, b: int) -> Tuple[int, int]:
    return (a, b) if a < b else (b, a)


@dataclass
class CoActGraph:
    edges: Dict[Tuple[int, int], int] = field(default_factory=lambda: defaultdict(int))
    node_freq: Dict[int, int] = field(default_factory=lambda: defaultdict(int))
    n_experts: int = 128
    n_layers: int = 94

    def node_id(self, layer: int, expert_id: int) -> int:
        return layer * self.n_experts + expert_id

    def add_token_step(self, layer: int, expert_ids: List[int]) -> None:
        ids = [self.node_id(layer, e) for e in expert_ids]
        for n in ids:
            self.node_freq[n] += 1
        for a, b in combinations(ids, 2):
            self.edges[_key(a, b)] += 1

    def add_cross_layer(self, layer: int, experts_l: List[int], experts_l1: List[int]) -> None:
        for e0 in experts_l:
            a = self.node_id(layer, e0)
            for e1 in experts_l1:
                self.edges[_key(a, self.node_id(layer + 1, e1))] += 1

    def total_edge_weight(self) -> int:
        return sum(self.edges.values())

    def cross_gpu_weight(self, placement: Dict[int, int]) -> int:
        return sum(w for (a, b), w in self.edges.items() if placement.get(a, -1) != placement.get(b, -2))


def ingest_telemetry(graph: CoActGraph, telemetry_events: Iterable[dict]) -> None:
    for ev in telemetry_events:
        per_layer: Dict[int, List[int]] = defaultdict(list)
        for e in ev.get("experts", []):
            per_layer[e["layer"]].append(e["expert_id"])
        order = sorted(per_layer)
        for layer in order:
            graph.add_token_step(layer, per_layer[layer])
        for a, b in zip(order, order[1:]):
            graph.add_cross_layer(a, per_layer[a], per_layer[b])


def greedy_partition(graph: CoActGraph, n_gpus: int = 8, n_experts: int = 128, n_layers: int = 94) -> Dict[int, int]:
    """Per layer: hottest experts first, each to the GPU (with a free slot) it shares most edge weight with."""
    cap = n_experts // n_gpus
    adj: Dict[int, Dict[int, int]] = defaultdict(dict)
    for (a, b), w in graph.edges.items():
        adj[a][b] = w
        adj[b][a] = w
    placement: Dict[int, int] = {}
    for layer in range(n_layers):
        nodes = [graph.node_id(layer, e) for e in range(n_experts)]
        nodes.sort(key=lambda n: -graph.node_freq.get(n, 0))
        load = [0] * n_gpus
        here: Dict[int, int] = {}
        for node in nodes:
            score = [0] * n_gpus
            for other, w in adj.get(node, {}).items():
                g = here.get(other)
                if g is not None:
                    score[g] += w
            free = [g for g in range(n_gpus) if load[g] < cap] or list(range(n_gpus))
            best = max(free, key=lambda g: (score[g], -g))
            here[node] = best
            load[best] += 1
        placement.update(here)
    return placement


def round_robin_placement(n_gpus: int = 8, n_experts: int = 128, n_layers: int = 94) -> Dict[int, int]:
    return {layer * n_experts + e: e % n_gpus for layer in range(n_layers) for e in range(n_experts)}


@dataclass
class TokenDAG:
    """Layer-ordered expert activations of one token; the plan pairs each layer with the next layer's experts."""
    activations: Dict[int, List[int]] = field(default_factory=dict)

    def add_layer(self, layer: int, expert_ids: List[int]) -> None:
        self.activations[layer] = list(expert_ids)

    def topo_layers(self) -> List[int]:
        return sorted(self.activations)

    def prefetch_schedule(self, placement: Dict[int, int], n_experts: int = 128) -> List[dict]:
        layers = self.topo_layers()
        plan = []
        for cur, nxt in zip(layers, layers[1:]):
            pairs = [(e, placement.get(nxt * n_experts + e, e % 8)) for e in self.activations.get(nxt, [])]
            gpus = {g for _, g in pairs}
            plan.append({"compute_layer": cur, "prefetch_layer": nxt, "prefetch_experts": pairs,
                         "cross_gpu": len(gpus) > 1, "n_gpus_touched": len(gpus)})
        return plan


def placement_stats(graph: CoActGraph, placement: Dict[int, int], label: str = "placement") -> dict:
    total, cross = graph.total_edge_weight(), graph.cross_gpu_weight(placement)
    frac = (cross / total) if total else 0.0
    return {"label": label, "total_edge_weight": total, "cross_gpu_weight": cross,
            "cross_gpu_fraction": round(frac, 4), "local_fraction": round(1 - frac, 4) if total else 1.0}
