"""Ranked "what to try next" predictions for a configuration (reference: src/inferutil/bench/levers.py:32-139):
halve the weight bytes, fp8 KV, ideal expert routing, a better tp/ep split, speculative decoding."""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import List, Optional

from ..hardware import Cluster
from ..latency import decode_latency
from ..model import MoEConfig
from .config import BenchConfig
from .spec_model import spec_speedup as _floor_aware_speedup

_EFFORT_RANK = {"S": 0, "M": 1, "L": 2}


@dataclass(frozen=True)
class Lever:
    name: str
    predicted_tok_s: float
    speedup: float
    effort: str          # S | M | L
    rationale: str


def _tok_s(cfg, cluster, *, plan, dtype_bytes, kv_dtype_bytes, seq_len, tp, ep, ideal_routing=False) -> float:
    return decode_latency(cfg, cluster, plan=plan, dtype_bytes=dtype_bytes, kv_dtype_bytes=kv_dtype_bytes,
                          seq_len=seq_len, tp=tp, ep=ep, ideal_routing=ideal_routing).tokens_per_s


def _spec_speedup(accept_rate: float, draft_len: int, n_drafters: int = 1, floor: float = 0.5) -> float:
    return _floor_aware_speedup(accept_rate, draft_len, n_drafters, floor)


def _floor_from_bottleneck(b, default: float = 0.5) -> float:
    """Floor fraction (what speculation amortises) ~ 1 - share of the weight stream."""
    if b is None:
        return default
    if b.dominant_term == "weight_bw":
        return max(0.0, 1.0 - b.share)
    if getattr(b, "second_term", None) == "weight_bw":
        return max(0.0, 1.0 - b.second_share)
    return 0.85


def recommend(cfg: MoEConfig, cluster: Cluster, config: BenchConfig, *, bottleneck=None, accept_rate: float = 0.7,
              draft_len: int = 4, n_drafters: int = 1, spec_floor: Optional[float] = None,
              min_speedup: float = 1.02) -> List[Lever]:
    kw = dict(plan=config.plan, dtype_bytes=config.dtype_bytes, kv_dtype_bytes=config.kv_dtype_bytes,
              seq_len=config.seq_len, tp=config.tp, ep=config.ep)
    base = _tok_s(cfg, cluster, **kw)
    dominant = getattr(bottleneck, "dominant_term", None)
    out: List[Lever] = []

    def consider(name, pred, effort, why, targets=()):
        if base <= 0 or pred <= 0 or pred / base < min_speedup:
            return
        if dominant in targets:
            why += "  [targets diagnosed bottleneck]"
        out.append(Lever(name, pred, pred / base, effort, why))

    if config.dtype_bytes > 0.5:
        half = config.dtype_bytes / 2.0
        consider("int4 experts", _tok_s(cfg, cluster, **{**kw, "dtype_bytes": half}), "S",
                 f"weights {config.dtype_bytes}B -> {half}B/param", ("weight_bw",))
    if config.kv_dtype_bytes > 1:
        consider("fp8/int8 KV", _tok_s(cfg, cluster, **{**kw, "kv_dtype_bytes": 1}), "S", "KV cache 2B -> 1B/elem",
                 ("kv_bw",))
    if config.plan in ("ep", "hybrid"):
        consider("ideal expert routing", _tok_s(cfg, cluster, ideal_routing=True, **kw), "M",
                 "eliminate busiest-GPU expert imbalance (routing/placement optimizer)", ("weight_bw", "comms"))
    divs = [d for d in range(1, cluster.n_gpus + 1) if cluster.n_gpus % d == 0]
    best, split = base, (config.tp, config.ep)
    for tp in divs:
        for ep in divs:
            pred = _tok_s(cfg, cluster, **{**kw, "tp": tp, "ep": ep})
            if pred > best:
                best, split = pred, (tp, ep)
    if split != (config.tp, config.ep):
        consider("relayout tp/ep", best, "S", f"tp={config.tp},ep={config.ep} -> tp={split[0]},ep={split[1]}",
                 ("weight_bw", "comms"))
    floor = _floor_from_bottleneck(bottleneck) if spec_floor is None else spec_floor
    consider("speculative decode", base * _spec_speedup(accept_rate, draft_len, n_drafters, floor), "L",
             f"est. accept~{accept_rate:.2f}, k={draft_len}, drafters={n_drafters}, floor F={floor:.2f}",
             ("kernel_gap", "comms"))
    return sorted(out, key=lambda lv: (-lv.speedup, _EFFORT_RANK.get(lv.effort, 9)))
