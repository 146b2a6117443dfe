"""Result record of one benchmark run and its derived figures (reference: src/inferutil/bench/metrics.py:13-188)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..hardware import Cluster
from ..latency import decode_latency
from ..model import MoEConfig
from .config import BenchConfig
from .efficiency import Efficiency, compute_efficiency, peak_flops_for_dtype
from .stats import stat_to_dict, summarize


@dataclass(frozen=True)
class TelemetrySummary:
    available: bool
    n_gpus: int
    temp_c_max: float
    sm_util_pct_mean: float
    mem_util_pct_mean: float
    power_w_mean: float            # mean of the summed power of all GPUs
    energy_j_per_token: float
    util_imbalance: float          # busiest GPU's mean utilisation / mean over GPUs
    per_gpu_mean_util: tuple


@dataclass(frozen=True)
class MeasuredBreakdown:
    weight_s: float
    kv_s: float
    comms_s: float
    compute_s: float


@dataclass(frozen=True)
class BenchResult:
    ttft_s: float
    prefill_tok_per_s: float
    decode_tok_per_s: float
    tpot_p50_s: float
    tpot_p95_s: float
    total_s: float
    n_decode_tokens: int
    bytes_per_token: int
    achieved_hbm_bw: float
    pct_of_peak_bw: float
    analytical_floor_tok_per_s: float
    pct_of_floor: float
    telemetry: TelemetrySummary
    n_repeats: int = 1
    decode_tok_per_s_std: float = 0.0
    measured_breakdown: Optional[MeasuredBreakdown] = None
    quality: Optional[object] = None
    efficiency: Optional[Efficiency] = None
    latency: Optional[dict] = None


def bytes_per_token(cfg: MoEConfig, seq_len: int, dtype_bytes: int, kv_dtype_bytes: int) -> int:
    return cfg.active_params * dtype_bytes + seq_len * cfg.kv_bytes_per_token(kv_dtype_bytes)


def percentile(sorted_vals: list, p: float) -> float:
    if not sorted_vals:
        return 0.0
    pos = (len(sorted_vals) - 1) * p
    lo = int(pos)
    hi = min(lo + 1, len(sorted_vals) - 1)
    return sorted_vals[lo] + (sorted_vals[hi] - sorted_vals[lo]) * (pos - lo)


def summarize_telemetry(samples, n_decode_tokens: int, decode_window_s: float) -> TelemetrySummary:
    if not samples:
        return TelemetrySummary(False, 0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, ())
    groups: dict = {}
    for s in samples:
        groups.setdefault(s.gpu_index, []).append(s)
    order = sorted(groups)

    def mean(xs):
        return sum(xs) / len(xs)

    util = tuple(mean([s.sm_util_pct for s in groups[g]]) for g in order)
    overall = mean(util)
    power = sum(mean([s.power_w for s in groups[g]]) for g in order)      # robust to uneven sample counts
    return TelemetrySummary(True, len(order), max(s.temp_c for s in samples), mean([s.sm_util_pct for s in samples]),
                            mean([s.mem_util_pct for s in samples]), power,
                            power * decode_window_s / n_decode_tokens if n_decode_tokens else 0.0,
                            max(util) / overall if overall else 0.0, util)


def aggregate_breakdown(step_breakdowns) -> Optional[MeasuredBreakdown]:
    rows = [b for b in (step_breakdowns or []) if b is not None]
    if not rows:
        return None
    n = len(rows)
    return MeasuredBreakdown(sum(b.weight_s for b in rows) / n, sum(b.kv_s for b in rows) / n,
                             sum(b.comms_s for b in rows) / n, sum(b.compute_s for b in rows) / n)


def _latency_panel(*, ttft_samples, e2e_samples, throughput_samples, tpot_step_seconds, ttft_s, decode_tok_per_s,
                   total_s) -> dict:
    """End-to-end, throughput and per-token latency as distributions (ms; tok/s)."""
    def ms(xs):
        return [1e3 * x for x in xs]
    return {"ttft_ms": stat_to_dict(summarize(ms(ttft_samples or [ttft_s]))),
            "e2e_ms": stat_to_dict(summarize(ms(e2e_samples or [total_s]))),
            "throughput_tok_s": stat_to_dict(summarize(list(throughput_samples or [decode_tok_per_s]))),
            "tpot_ms": stat_to_dict(summarize(ms(tpot_step_seconds or [])))}


def build_result(*, cfg: MoEConfig, cluster: Cluster, config: BenchConfig, ttft_s: float, prefill_tok_per_s: float,
                 decode_step_seconds: list, telemetry_summary: TelemetrySummary, decode_tok_per_s_samples=None,
                 step_breakdowns=None, quality=None, ttft_samples=None, e2e_samples=None) -> BenchResult:
    n = len(decode_step_seconds)
    decode_total = sum(decode_step_seconds)
    tpot = decode_total / n if n else float("inf")
    tok_s = 1.0 / tpot if tpot else float("inf")
    bpt = bytes_per_token(cfg, config.seq_len, config.dtype_bytes, config.kv_dtype_bytes)
    bw = bpt / tpot if tpot else 0.0
    floor = decode_latency(cfg, cluster, plan=config.plan, dtype_bytes=config.dtype_bytes,
                           kv_dtype_bytes=config.kv_dtype_bytes, seq_len=config.seq_len, tp=config.tp,
                           ep=config.ep).tokens_per_s
    n_rep, std = 1, 0.0
    if decode_tok_per_s_samples:
        n_rep = len(decode_tok_per_s_samples)
        tok_s = sum(decode_tok_per_s_samples) / n_rep
        std = (sum((x - tok_s) ** 2 for x in decode_tok_per_s_samples) / n_rep) ** 0.5
    total_s = ttft_s + decode_total
    peak = cluster.n_gpus * peak_flops_for_dtype(cluster.gpu.bf16_flops, cluster.gpu.fp8_flops, config.dtype_bytes)
    eff = compute_efficiency(active_params=cfg.active_params, weight_bytes=cfg.active_params * config.dtype_bytes,
                             bytes_per_token=bpt, kv_bytes=config.seq_len * cfg.kv_bytes_per_token(config.kv_dtype_bytes),
                             prompt_tokens=config.prompt_tokens, prefill_tok_s=prefill_tok_per_s, decode_tok_s=tok_s,
                             peak_flops=peak, peak_bw=cluster.aggregate_hbm_bw)
    srt = sorted(decode_step_seconds)
    return BenchResult(
        ttft_s=ttft_s, prefill_tok_per_s=prefill_tok_per_s, decode_tok_per_s=tok_s, tpot_p50_s=percentile(srt, 0.5),
        tpot_p95_s=percentile(srt, 0.95), total_s=total_s, n_decode_tokens=config.decode_tokens, bytes_per_token=bpt,
        achieved_hbm_bw=bw, pct_of_peak_bw=bw / cluster.aggregate_hbm_bw, analytical_floor_tok_per_s=floor,
        pct_of_floor=tok_s / floor if floor else 0.0, telemetry=telemetry_summary, n_repeats=n_rep,
        decode_tok_per_s_std=std, measured_breakdown=aggregate_breakdown(step_breakdowns), quality=quality,
        efficiency=eff,
        latency=_latency_panel(ttft_samples=ttft_samples, e2e_samples=e2e_samples,
                               throughput_samples=decode_tok_per_s_samples, tpot_step_seconds=decode_step_seconds,
                               ttft_s=ttft_s, decode_tok_per_s=tok_s, total_s=total_s))
