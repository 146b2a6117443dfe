"""Small-sample statistics for repeated runs (reference: src/inferutil/bench/stats.py:20-128)."""
from __future__ import annotations

from dataclasses import asdict, dataclass
from math import sqrt
from typing import List, Optional

# two-sided 95 % Student-t critical values for 1..30 degrees of freedom
_T95 = (12.706, 4.303, 3.182, 2.776, 2.571, 2.447, 2.365, 2.306, 2.262, 2.228, 2.201, 2.179, 2.160, 2.145, 2.131,
        2.120, 2.110, 2.101, 2.093, 2.086, 2.080, 2.074, 2.069, 2.064, 2.060, 2.056, 2.052, 2.048, 2.045, 2.042)


def t95(df: int) -> float:
    if df <= 0:
        return float("inf")
    return _T95[df - 1] if df <= len(_T95) else 1.96


def percentile(sorted_vals: List[float], p: float) -> Optional[float]:
    """Linear interpolation between order statistics, ``p`` in [0, 1]; ``None`` for no data."""
    n = len(sorted_vals)
    if n == 0:
        return None
    pos = (n - 1) * p
    lo = int(pos)
    hi = min(lo + 1, n - 1)
    return sorted_vals[lo] + (sorted_vals[hi] - sorted_vals[lo]) * (pos - lo)


@dataclass(frozen=True)
class Stat:
    n: int = 0
    mean: Optional[float] = None
    std: Optional[float] = None
    cv: Optional[float] = None
    p50: Optional[float] = None
    p90: Optional[float] = None
    p95: Optional[float] = None
    p99: Optional[float] = None
    min: Optional[float] = None
    max: Optional[float] = None
    ci95_lo: Optional[float] = None
    ci95_hi: Optional[float] = None
    samples: tuple = ()

    @property
    def ci95_half_width(self) -> Optional[float]:
        if self.ci95_lo is None or self.ci95_hi is None:
            return None
        return 0.5 * (self.ci95_hi - self.ci95_lo)


def summarize(values) -> Stat:
    xs = [float(v) for v in (values or []) if v is not None]
    n = len(xs)
    if n == 0:
        return Stat()
    srt = sorted(xs)
    mean = sum(xs) / n
    pct = {k: percentile(srt, q) for k, q in (("p50", .5), ("p90", .9), ("p95", .95), ("p99", .99))}
    if n == 1:
        return Stat(n=1, mean=mean, min=srt[0], max=srt[0], samples=tuple(xs), **pct)
    std = sqrt(sum((x - mean) ** 2 for x in xs) / (n - 1))
    half = t95(n - 1) * std / sqrt(n)
    return Stat(n=n, mean=mean, std=std, cv=(std / mean if mean else None), min=srt[0], max=srt[-1],
                ci95_lo=mean - half, ci95_hi=mean + half, samples=tuple(xs), **pct)


def stat_to_dict(s: Stat) -> dict:
    d = asdict(s)
    d["samples"] = list(s.samples)
    return d


def stat_from_dict(d: Optional[dict]) -> Optional[Stat]:
    if not d:
        return None
    d = dict(d)
    d["samples"] = tuple(d.get("samples") or ())
    return Stat(**d)


def means_differ(a: Stat, b: Stat) -> bool:
    """True when both 95 % confidence intervals exist and do not overlap."""
    if a.ci95_lo is None or b.ci95_lo is None:
        return False
    return a.ci95_hi < b.ci95_lo or b.ci95_hi < a.ci95_lo
