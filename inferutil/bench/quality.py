"""Greedy-output parity against a reference token sequence (reference: src/inferutil/bench/quality.py:19-36)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class QualityResult:
    match_rate: float
    n_compared: int
    first_divergence: int          # -1: identical over the compared prefix


def match_rate(candidate_ids, reference_ids) -> QualityResult:
    pairs = list(zip(candidate_ids, reference_ids))
    if not pairs:
        return QualityResult(1.0, 0, -1)
    same = [a == b for a, b in pairs]
    first = same.index(False) if False in same else -1
    return QualityResult(sum(same) / len(pairs), len(pairs), first)
