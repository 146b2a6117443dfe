"""Which term of the token time dominates a measured run (reference: src/inferutil/bench/attribution.py:31-109).
The actual per-token time is split into the analytical floor, apportioned by the measured (or byte-share) shape,
plus ``kernel_gap`` = time above the floor, counted once."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

_HINTS = {
    "weight_bw": "weights dominate HBM reads -> quantize harder (fp8->int4 experts)",
    "kv_bw": "KV cache dominates -> fp8/int8 KV, prefix reuse, shorter context",
    "comms": "collective/launch latency -> TP-heavier layout, CUDA graphs, fused all-to-all",
    "compute": "compute-bound (unusual at B=1) -> check dequant isn't on the math path",
    "kernel_gap": "running below the analytical floor -> CUDA graphs, fused dequant, kernel tuning",
}


def dominant_of_breakdown(weight_s: float, kv_s: float, comms_s: float, compute_s: float) -> str:
    terms = (("weight_bw", weight_s), ("kv_bw", kv_s), ("comms", comms_s), ("compute", compute_s))
    return max(terms, key=lambda kv: kv[1])[0]


def lever_hint(term: str) -> str:
    return _HINTS.get(term, term)


@dataclass(frozen=True)
class Bottleneck:
    dominant_term: str
    share: float
    second_term: str
    second_share: float
    confidence: float              # dominant / (dominant + second)
    headroom_to_floor: float
    regime: str
    ai_decode: Optional[float]
    ridge: Optional[float]
    note: str


def _shape(result) -> dict:
    mb = result.measured_breakdown
    if mb is not None:
        raw = {"weight_bw": mb.weight_s, "kv_bw": mb.kv_s, "comms": mb.comms_s, "compute": mb.compute_s}
        total = sum(raw.values())
        if total > 0:
            return {k: v / total for k, v in raw.items()}
    kv = (result.efficiency.kv_byte_share if result.efficiency else None) or 0.0
    return {"weight_bw": 1.0 - kv, "kv_bw": kv, "comms": 0.0, "compute": 0.0}


def diagnose(result) -> Bottleneck:
    floor_rate, rate = result.analytical_floor_tok_per_s or 0.0, result.decode_tok_per_s or 0.0
    floor_s = 1.0 / floor_rate if floor_rate else 0.0
    actual_s = 1.0 / rate if rate else floor_s
    gap = max(0.0, actual_s - floor_s)
    parts = {k: (actual_s - gap) * frac for k, frac in _shape(result).items()}
    parts["kernel_gap"] = gap
    (t1, v1), (t2, v2) = sorted(parts.items(), key=lambda kv: kv[1], reverse=True)[:2]
    total = sum(parts.values()) or 1.0
    e = result.efficiency
    return Bottleneck(t1, v1 / total, t2, v2 / total, v1 / ((v1 + v2) or 1.0),
                      max(0.0, 1.0 - (result.pct_of_floor or 0.0)), e.regime_decode if e else "unknown",
                      e.ai_decode if e else None, e.roofline_ridge if e else None, lever_hint(t1))
