"""Plain-text reports over stored runs and sweeps (reference: src/inferutil/bench/report.py:19-256)."""
from __future__ import annotations

from typing import List, Optional

from .attribution import diagnose
from .cost import energy_metrics, rental_usd_per_mtok
from .stats import stat_from_dict
from .store import RunRecord


def _pct(x) -> str:
    return "—" if x is None else f"{100.0 * x:.1f}%"


def _num(x, fmt="{:.2f}") -> str:
    return "—" if x is None else fmt.format(x)


def is_significant(mean_a: float, std_a: float, mean_b: float, std_b: float) -> bool:
    """Difference of means larger than the sum of the two standard deviations."""
    return abs(mean_a - mean_b) > (std_a + std_b)


def _stat_line(label: str, d: Optional[dict], unit: str) -> str:
    s = stat_from_dict(d)
    if s is None or s.mean is None:
        return f"  {label:<14} —"
    ci = f"  ±{s.ci95_half_width:.3g} (95% CI, n={s.n})" if s.ci95_half_width is not None else f"  (n={s.n})"
    return f"  {label:<14} mean {s.mean:.3f} {unit}  p50 {_num(s.p50, '{:.3f}')}  p95 {_num(s.p95, '{:.3f}')}{ci}"


def format_result(record: RunRecord) -> str:
    r, c = record.result, record.config
    n_gpus = record.env.get("n_gpus", 8)
    out = [f"run {record.runid}  config '{c.name}': plan={c.plan} tp={c.tp} ep={c.ep} "
           f"weights={c.dtype_bytes}B kv={c.kv_dtype_bytes}B prompt={c.prompt_tokens} decode={c.decode_tokens} "
           f"repeats={r.n_repeats}", "", "latency"]
    lat = r.latency or {}
    out += [_stat_line("TTFT", lat.get("ttft_ms"), "ms"), _stat_line("TPOT", lat.get("tpot_ms"), "ms"),
            _stat_line("end-to-end", lat.get("e2e_ms"), "ms"), _stat_line("throughput", lat.get("throughput_tok_s"), "tok/s"),
            f"  decode {r.decode_tok_per_s:.1f} tok/s (std {r.decode_tok_per_s_std:.2f})   TPOT p50 "
            f"{1e3 * r.tpot_p50_s:.3f} ms  p95 {1e3 * r.tpot_p95_s:.3f} ms   prefill {r.prefill_tok_per_s:.0f} tok/s",
            "", "roofline",
            f"  bytes/token {r.bytes_per_token / 1e9:.2f} GB   achieved {r.achieved_hbm_bw / 1e12:.2f} TB/s "
            f"({_pct(r.pct_of_peak_bw)} of peak)   floor {r.analytical_floor_tok_per_s:.1f} tok/s "
            f"({_pct(r.pct_of_floor)} of floor)"]
    e = r.efficiency
    if e is not None:
        out += ["", "efficiency",
                f"  MBU decode {_pct(e.mbu_decode)}   MFU decode {_pct(e.mfu_decode)}   MFU prefill {_pct(e.mfu_prefill)}",
                f"  intensity decode {_num(e.ai_decode)} FLOP/B  prefill {_num(e.ai_prefill, '{:.0f}')} FLOP/B  ridge "
                f"{_num(e.roofline_ridge, '{:.0f}')}  -> decode {e.regime_decode}, prefill {e.regime_prefill}; "
                f"KV share of bytes {_pct(e.kv_byte_share)}"]
    power = r.telemetry.power_w_mean if r.telemetry.available else None
    en = energy_metrics(r.decode_tok_per_s, power)
    out += ["", "cost",
            f"  rental ${_num(rental_usd_per_mtok(r.decode_tok_per_s, n_gpus))}/Mtok   energy "
            f"{_num(en['joules_per_token'])} J/token  {_num(en['kwh_per_mtok'], '{:.3f}')} kWh/Mtok"]
    b = diagnose(r)
    out += ["", "bottleneck",
            f"  {b.dominant_term} {_pct(b.share)} (then {b.second_term} {_pct(b.second_share)}; confidence "
            f"{b.confidence:.2f}; headroom to floor {_pct(b.headroom_to_floor)})", f"  {b.note}"]
    mb = r.measured_breakdown
    if mb is not None:
        out += ["", "measured breakdown (ms/token)",
                f"  weight {1e3 * mb.weight_s:.3f}  kv {1e3 * mb.kv_s:.3f}  comms {1e3 * mb.comms_s:.3f}  compute "
                f"{1e3 * mb.compute_s:.3f}"]
    if r.quality is not None:
        out += ["", f"quality: match rate {r.quality.match_rate:.3f} over {r.quality.n_compared} tokens "
                    f"(first divergence {r.quality.first_divergence})"]
    t = r.telemetry
    out += ["", "telemetry: " + (f"{t.n_gpus} GPUs  max {t.temp_c_max:.0f} C  SM util {t.sm_util_pct_mean:.0f}%  "
                                 f"power {t.power_w_mean:.0f} W  imbalance {t.util_imbalance:.2f}" if t.available
                                 else "unavailable")]
    return "\n".join(out)


def format_sweep(points, *, n_gpus: int = 8, usd_per_gpu_hr: float = 3.0, title: str = "sweep") -> str:
    out = [title, f"  {'label':<24}{'seq':>7}{'tok/s':>10}{'TPOT ms':>10}{'MBU':>8}{'KV%':>7}{'$/Mtok':>9}  dominant"]
    for p in points:
        usd = rental_usd_per_mtok(p.decode_tok_s, n_gpus, usd_per_gpu_hr=usd_per_gpu_hr)
        out.append(f"  {p.label:<24}{p.seq_len:>7}{p.decode_tok_s:>10.1f}{p.tpot_ms:>10.3f}{_pct(p.mbu_decode):>8}"
                   f"{_pct(p.kv_byte_share):>7}{_num(usd):>9}  {p.dominant_term}")
    return "\n".join(out)


def format_spec_sweep(rows, feasibility: dict, *, base_tok_s=None) -> str:
    out = ["speculative decoding sweep (independent drafters, tree verify)",
           f"  {'alpha':>6}{'k':>4}{'N':>4}{'E[acc]':>9}{'speedup':>9}{'verify toks':>13}" + ("  tok/s" if base_tok_s else "")]
    for r in rows:
        tail = f"  {base_tok_s * r.speedup:.0f}" if base_tok_s else ""
        out.append(f"  {r.alpha:>6.2f}{r.k:>4}{r.n_drafters:>4}{r.e_acc:>9.2f}{r.speedup:>9.2f}{r.verify_tokens:>13}{tail}")
    out.append(f"  memory: target {feasibility['target_weight_gb']} GB, headroom {feasibility['hbm_headroom_gb']} GB, "
               f"up to {feasibility['max_drafters']} drafters of {feasibility['draft_model_gb']} GB")
    return "\n".join(out)


def format_spec_floor(rows, feasibility: dict, *, accept: float, floor: float, base_tok_s=None) -> str:
    out = [f"floor-aware speculative model: accept {accept:.2f}, floor fraction F {floor:.2f}",
           f"  {'k':>4}{'N':>4}{'emitted':>10}{'verify cost':>13}{'speedup':>9}" + ("  tok/s" if base_tok_s else "")]
    for r in rows:
        tail = f"  {base_tok_s * r.speedup:.0f}" if base_tok_s else ""
        out.append(f"  {r.draft_len:>4}{r.n_drafters:>4}{r.emitted:>10.2f}{r.verify_cost:>13.2f}{r.speedup:>9.2f}{tail}")
    out.append(f"  memory: headroom {feasibility['hbm_headroom_gb']} GB -> up to {feasibility['max_drafters']} drafters")
    return "\n".join(out)


def _lever_lines(levers) -> List[str]:
    if not levers:
        return ["  (no lever predicted above the minimum speed-up)"]
    return [f"  {lv.speedup:>5.2f}x  {lv.predicted_tok_s:>8.1f} tok/s  [{lv.effort}] {lv.name}: {lv.rationale}" for lv in levers]


def format_plan(record: RunRecord, bottleneck, levers, best_point=None) -> str:
    out = [f"plan for '{record.config.name}' (baseline {record.result.decode_tok_per_s:.1f} tok/s)",
           f"  bottleneck: {bottleneck.dominant_term} ({_pct(bottleneck.share)}) — {bottleneck.note}", "levers"]
    out += _lever_lines(levers)
    if best_point is not None:
        out.append(f"best layout in sweep: {best_point.label} at {best_point.decode_tok_s:.1f} tok/s")
    return "\n".join(out)


def format_diagnosis(record: RunRecord, levers=None) -> str:
    b = diagnose(record.result)
    out = [f"diagnosis of run {record.runid} ('{record.config.name}')",
           f"  dominant {b.dominant_term} {_pct(b.share)}; second {b.second_term} {_pct(b.second_share)}; confidence "
           f"{b.confidence:.2f}", f"  regime {b.regime}  intensity {_num(b.ai_decode)}  ridge {_num(b.ridge, '{:.0f}')}  "
           f"headroom to floor {_pct(b.headroom_to_floor)}", f"  {b.note}"]
    if levers is not None:
        out += ["next levers"] + _lever_lines(levers)
    return "\n".join(out)


def _delta(a: float, b: float) -> str:
    return "—" if not a else f"{100.0 * (b - a) / a:+.1f}%"


def format_compare(a: RunRecord, b: RunRecord) -> str:
    ra, rb = a.result, b.result
    rows = [("decode tok/s", ra.decode_tok_per_s, rb.decode_tok_per_s), ("TTFT ms", 1e3 * ra.ttft_s, 1e3 * rb.ttft_s),
            ("TPOT p50 ms", 1e3 * ra.tpot_p50_s, 1e3 * rb.tpot_p50_s), ("TPOT p95 ms", 1e3 * ra.tpot_p95_s, 1e3 * rb.tpot_p95_s),
            ("% of floor", 100 * ra.pct_of_floor, 100 * rb.pct_of_floor), ("% of peak BW", 100 * ra.pct_of_peak_bw, 100 * rb.pct_of_peak_bw)]
    out = [f"compare {a.runid} -> {b.runid}", f"  {'metric':<14}{'A':>12}{'B':>12}{'delta':>9}"]
    out += [f"  {name:<14}{x:>12.3f}{y:>12.3f}{_delta(x, y):>9}" for name, x, y in rows]
    sig = is_significant(ra.decode_tok_per_s, ra.decode_tok_per_s_std, rb.decode_tok_per_s, rb.decode_tok_per_s_std)
    out.append("  throughput difference is " + ("significant" if sig else "within noise"))
    return "\n".join(out)
