"""Closed-form speculative-decoding estimates (reference: src/inferutil/speculative.py:43-149).

One drafter proposing ``k`` tokens with per-token acceptance ``alpha`` yields a geometric run; ``n`` independent
drafters verified as a tree accept a position when any of them matches.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional


@dataclass(frozen=True)
class SpecConfig:
    alpha: float
    k: int
    n_drafters: int
    drafter_cost_ratio: float = 0.05


def _geometric_run(p: float, k: int) -> float:
    """sum_{i=0}^{k-1} p^i : expected number of positions reached before the first miss, capped at k."""
    return float(k) if p >= 1.0 else (1.0 - p ** k) / (1.0 - p)


def expected_accepted_single(alpha: float, k: int) -> float:
    """Draft tokens accepted per round with one drafter (the bonus token is not counted)."""
    return float(k) if alpha >= 1.0 else alpha * _geometric_run(alpha, k)


def expected_accepted_multi(alpha: float, k: int, n: int) -> float:
    if n <= 0:
        return 0.0
    hit = 1.0 - (1.0 - alpha) ** n
    return _geometric_run(hit, k)


def rounds_per_target_token(cfg: SpecConfig) -> float:
    return 1.0 / max(expected_accepted_multi(cfg.alpha, cfg.k, cfg.n_drafters), 1e-9)


def wall_clock_speedup(cfg: SpecConfig, target_bw_s: float = 1.0) -> float:
    """Accepted tokens per unit of (one drafter pass + one bandwidth-bound verify pass)."""
    return expected_accepted_multi(cfg.alpha, cfg.k, cfg.n_drafters) / (1.0 + cfg.drafter_cost_ratio)


@dataclass
class SpecSweepRow:
    n_drafters: int
    alpha: float
    k: int
    e_acc: float
    speedup: float
    verify_tokens: int


def sweep(alphas: Optional[List[float]] = None, ks: Optional[List[int]] = None,
          n_drafters_list: Optional[List[int]] = None, drafter_cost_ratio: float = 0.05) -> List[SpecSweepRow]:
    rows = []
    for alpha in alphas or [0.5, 0.6, 0.7, 0.8]:
        for k in ks or [4, 8, 16]:
            for n in n_drafters_list or [1, 2, 4, 8]:
                c = SpecConfig(alpha, k, n, drafter_cost_ratio)
                rows.append(SpecSweepRow(n, alpha, k, round(expected_accepted_multi(alpha, k, n), 2),
                                         round(wall_clock_speedup(c), 2), n * k))
    return rows


def memory_feasibility(target_total_gb: float = 470.0, target_active_gb: float = 43.2, hbm_total_gb: float = 640.0,
                       draft_model_gb: float = 3.4, use_fp8_target: bool = True) -> dict:
    weights = target_total_gb * (0.5 if use_fp8_target else 1.0)
    headroom = hbm_total_gb - weights
    return {"target_weight_gb": round(weights, 1), "hbm_headroom_gb": round(headroom, 1),
            "draft_model_gb": draft_model_gb, "max_drafters": int(headroom // draft_model_gb),
            "use_fp8_target": use_fp8_target}
