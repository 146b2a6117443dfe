"""Speculative-decoding accept statistics from a Prometheus ``/metrics`` scrape of a proxied vLLM server
(reference: server/spec_metrics.py:24-95). Counters are cumulative: the per-turn rate is the difference of two
scrapes; counter names drift between versions, so matching is by substring."""
from __future__ import annotations

import re
import urllib.request
from typing import Dict, Optional

_LINE = re.compile(r"^([a-zA-Z_:][\w:]*)(?:\{[^}]*\})?\s+([0-9.eE+-]+)$")


def _scalars(metrics_text: str) -> Dict[str, float]:
    """Metric name -> sum over label sets."""
    out: Dict[str, float] = {}
    for raw in (metrics_text or "").splitlines():
        m = _LINE.match(raw.strip())
        if m:
            try:
                out[m.group(1)] = out.get(m.group(1), 0.0) + float(m.group(2))
            except ValueError:
                continue
    return out


def _find(vals: Dict[str, float], *subs: str) -> Optional[float]:
    for name, v in vals.items():
        low = name.lower()
        if all(s in low for s in subs):
            return v
    return None


def parse_spec_counters(metrics_text: str) -> dict:
    vals = _scalars(metrics_text)
    accepted = _find(vals, "spec_decode", "accepted")
    if accepted is None:
        accepted = _find(vals, "accepted", "token")
    drafts = _find(vals, "spec_decode", "num_drafts")
    if drafts is None:
        drafts = _find(vals, "spec_decode", "draft")
    return {"accepted": accepted or 0.0, "drafts": drafts or 0.0}


def _stats(accepted: float, drafts: float) -> dict:
    if drafts <= 0:
        return {"accept_rate": 0.0, "tau": 1.0, "accepted": accepted, "drafts": drafts}
    rate = accepted / drafts
    return {"accept_rate": round(min(rate, 1.0), 4), "tau": round(1.0 + rate, 3), "accepted": accepted, "drafts": drafts}


def accept_stats(before_text: str, after_text: str) -> dict:
    b, a = parse_spec_counters(before_text), parse_spec_counters(after_text)
    return _stats(max(a["accepted"] - b["accepted"], 0.0), max(a["drafts"] - b["drafts"], 0.0))


def cumulative_accept(metrics_text: str) -> dict:
    c = parse_spec_counters(metrics_text)
    return _stats(c["accepted"], c["drafts"])


def fetch_metrics(vllm_url: str, timeout: float = 2.0) -> str:
    try:
        with urllib.request.urlopen(f"{vllm_url}/metrics", timeout=timeout) as r:
            return r.read().decode(errors="replace")
    except Exception:
        return ""
