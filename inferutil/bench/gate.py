"""Pass/fail thresholds and the regression gate (reference: src/inferutil/bench/gate.py:12-66): a candidate fails
only when its throughput mean dropped AND the 95 % confidence intervals are disjoint."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .stats import means_differ, stat_from_dict


@dataclass(frozen=True)
class Thresholds:
    min_decode_tok_per_s: Optional[float] = None
    max_ttft_s: Optional[float] = None
    min_pct_of_floor: Optional[float] = None
    min_quality_match: Optional[float] = None


@dataclass(frozen=True)
class GateResult:
    passed: bool
    failures: tuple


def evaluate(result, thresholds: Thresholds) -> GateResult:
    t, bad = thresholds, []
    if t.min_decode_tok_per_s is not None and result.decode_tok_per_s < t.min_decode_tok_per_s:
        bad.append(f"decode {result.decode_tok_per_s:.1f} < min {t.min_decode_tok_per_s:.1f} tok/s")
    if t.max_ttft_s is not None and result.ttft_s > t.max_ttft_s:
        bad.append(f"ttft {result.ttft_s * 1e3:.1f} > max {t.max_ttft_s * 1e3:.1f} ms")
    if t.min_pct_of_floor is not None and result.pct_of_floor < t.min_pct_of_floor:
        bad.append(f"pct_of_floor {result.pct_of_floor * 100:.1f} < min {t.min_pct_of_floor * 100:.1f} %")
    if t.min_quality_match is not None:
        q = result.quality
        if q is None:
            bad.append(f"quality not measured (run had no reference) — required min {t.min_quality_match:.3f}")
        elif q.match_rate < t.min_quality_match:
            bad.append(f"quality {q.match_rate:.3f} < min {t.min_quality_match:.3f}")
    return GateResult(not bad, tuple(bad))


def _throughput(result):
    return stat_from_dict((getattr(result, "latency", None) or {}).get("throughput_tok_s"))


def regression_gate(baseline_result, candidate_result) -> GateResult:
    b, c = _throughput(baseline_result), _throughput(candidate_result)
    have_ci = all(s is not None and s.mean is not None and s.ci95_lo is not None for s in (b, c))
    bad = []
    if not have_ci:
        if candidate_result.decode_tok_per_s < baseline_result.decode_tok_per_s:
            bad.append(f"throughput {candidate_result.decode_tok_per_s:.1f} < baseline "
                       f"{baseline_result.decode_tok_per_s:.1f} tok/s (no CI; n<2)")
    elif c.mean < b.mean and means_differ(b, c):
        bad.append(f"throughput regressed {c.mean:.1f} vs baseline {b.mean:.1f} tok/s (95% CIs disjoint)")
    return GateResult(not bad, tuple(bad))
