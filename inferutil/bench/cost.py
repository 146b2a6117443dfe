"""Energy and rental cost per million tokens (reference: src/inferutil/bench/cost.py:20-45)."""
from __future__ import annotations

from typing import Optional


def energy_metrics(decode_tok_s: Optional[float], power_w: Optional[float], *, usd_per_kwh: float = 0.12) -> dict:
    if not decode_tok_s or not power_w:
        return dict.fromkeys(("joules_per_token", "tok_s_per_watt", "kwh_per_mtok", "usd_per_mtok_energy"))
    joules = power_w / decode_tok_s
    kwh = joules * 1e6 / 3.6e6
    return {"joules_per_token": joules, "tok_s_per_watt": decode_tok_s / power_w, "kwh_per_mtok": kwh,
            "usd_per_mtok_energy": kwh * usd_per_kwh}


def rental_usd_per_mtok(decode_tok_s: Optional[float], n_gpus: int, *, usd_per_gpu_hr: float = 3.0) -> Optional[float]:
    if not decode_tok_s:
        return None
    return 1e6 * (n_gpus * usd_per_gpu_hr / 3600.0) / decode_tok_s
