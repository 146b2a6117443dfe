"""Confidence-adaptive top-k routing: when the router's softmax is concentrated, a token uses fewer than ``top_k``
experts (the smallest prefix of its top-k whose renormalised mass reaches ``mass``, at least ``k_min``), which cuts
the expert weight bytes of a B = 1 step. This module measures the head-room (``router_mass``) and the quality cost
(with ``quality.compare_ids``) on this engine's model.

Reference: experiments/adaptive_topk/vllm_adaptive_moe.py (a vLLM ``custom_routing_function``) and
tools/router_mass.py (mass of the top-4 / top-6 inside the top-8 over many positions, expected average k).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Sequence

import torch


@dataclass
class AdaptiveStats:
    calls: int = 0
    kept: int = 0
    slots: int = 0
    per_layer_kept: Dict[int, int] = field(default_factory=dict)
    per_layer_slots: Dict[int, int] = field(default_factory=dict)

    @property
    def mean_k(self) -> float:
        return self.kept / self.calls if self.calls else 0.0

    @property
    def expert_byte_saving(self) -> float:
        return 1.0 - self.kept / self.slots if self.slots else 0.0


def adaptive_route(h: torch.Tensor, router_w: torch.Tensor, top_k: int, renorm: bool, mass: float, k_min: int):
    """-> (idx [T, k], w [T, k], logits, kept [T]): slots after the kept prefix carry weight 0; the kept weights are
    renormalised over the kept prefix when ``renorm``."""
    logits = h.float() @ router_w.float().t()
    probs = torch.softmax(logits, dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)                         # descending
    share = torch.cumsum(w, -1) / w.sum(-1, keepdim=True)
    kept = (share < mass).sum(-1) + 1                                   # smallest prefix reaching the mass
    kept = kept.clamp(min=max(1, k_min), max=top_k)
    keep = torch.arange(top_k, device=h.device)[None, :] < kept[:, None]
    w = torch.where(keep, w, torch.zeros_like(w))
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return idx, w, logits, kept


def install(model, mass: float = 0.9, k_min: int = 4) -> AdaptiveStats:
    stats = AdaptiveStats()

    def fn(L, h, router_w, top_k, renorm):
        idx, w, logits, kept = adaptive_route(h, router_w, top_k, renorm, mass, k_min)
        n = int(kept.numel())
        stats.calls += n
        stats.kept += int(kept.sum())
        stats.slots += n * top_k
        stats.per_layer_kept[L] = stats.per_layer_kept.get(L, 0) + int(kept.sum())
        stats.per_layer_slots[L] = stats.per_layer_slots.get(L, 0) + n * top_k
        return idx, w, logits

    model.route_fn = fn
    return stats


def uninstall(model) -> None:
    model.route_fn = None


def router_mass(model, prompts: Sequence[Sequence[int]], ks=(4, 6), thresholds=(0.85, 0.9, 0.95)) -> dict:
    """Over all (position, layer) of the prompts: how often the top-k' of the selected top-k holds at least a
    threshold of the selected mass, the expected k of the adaptive policy per threshold, and the concentration by
    depth (early / middle / late third of the stack)."""
    cfg = model.cfg
    shares: List[torch.Tensor] = []
    layers: List[int] = []

    def fn(L, h, router_w, top_k, renorm):
        logits = h.float() @ router_w.float().t()
        probs = torch.softmax(logits, -1)
        w, idx = torch.topk(probs, top_k, -1)
        shares.append(torch.cumsum(w, -1) / w.sum(-1, keepdim=True))
        layers.append(L)
        if renorm:
            w = w / w.sum(-1, keepdim=True)
        return idx, w, logits

    prev = model.route_fn
    model.route_fn = fn
    try:
        for p in prompts:
            cache = model.new_cache(len(p) + 1)
            model.forward_hidden(torch.as_tensor(list(p), dtype=torch.long, device=model.w.embed.device), cache,
                                 record_routes=False)
    finally:
        model.route_fn = prev
    allsh = torch.cat(shares, 0)                                        # [N, top_k] cumulative share
    out = {"positions_x_layers": int(allsh.shape[0]), "fraction_above": {}, "expected_k": {}, "by_depth": {}}
    for k in ks:
        if k <= cfg.top_k:
            out["fraction_above"][k] = {str(t): float((allsh[:, k - 1] >= t).float().mean()) for t in thresholds}
    for t in thresholds:
        kept = ((allsh < t).sum(-1) + 1).clamp(max=cfg.top_k).float()
        out["expected_k"][str(t)] = float(kept.mean())
    third = max(1, cfg.n_layers // 3)
    for name, lo, hi in (("early", 0, third), ("middle", third, 2 * third), ("late", 2 * third, cfg.n_layers)):
        sel = [s for s, L in zip(shares, layers) if lo <= L < hi]
        if sel:
            half = max(1, cfg.top_k // 2)
            out["by_depth"][name] = float(torch.cat(sel, 0)[:, half - 1].mean())
    return out


def quality_gate(engine, prompts: Sequence[Sequence[int]], new_tokens: int = 32, mass: float = 0.9, k_min: int = 4,
                 min_prefix: float = 0.8) -> dict:
    """Greedy outputs with and without the adaptive router; passes when the mean common-prefix share stays above
    ``min_prefix``."""
    from .quality import compare_ids
    base = [engine.generate(list(p), new_tokens).tokens for p in prompts]
    stats = install(engine.model, mass, k_min)
    try:
        got = [engine.generate(list(p), new_tokens).tokens for p in prompts]
    finally:
        uninstall(engine.model)
    c = compare_ids(base, got)
    return {**c, "mean_k": stats.mean_k, "expert_byte_saving": stats.expert_byte_saving,
            "passed": c["mean_prefix_agreement"] >= min_prefix}
