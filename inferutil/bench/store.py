"""Run records on disk and tabular exports (reference: src/inferutil/bench/store.py:12-172).
Layout: ``<results>/<config name>/<runid>.json`` (+ ``.manifest.json`` beside it)."""
from __future__ import annotations

import csv
import json
import os
import warnings
from dataclasses import asdict, dataclass
from typing import Optional

from .config import BenchConfig
from .efficiency import Efficiency
from .metrics import BenchResult, MeasuredBreakdown, TelemetrySummary
from .quality import QualityResult


@dataclass(frozen=True)
class RunRecord:
    runid: str
    config: BenchConfig
    env: dict
    result: BenchResult


def _record_to_dict(r: RunRecord) -> dict:
    return {"runid": r.runid, "config": asdict(r.config), "env": r.env, "result": asdict(r.result)}


def _record_from_dict(d: dict) -> RunRecord:
    body = dict(d["result"])
    tele = dict(body.pop("telemetry"))
    tele["per_gpu_mean_util"] = tuple(tele["per_gpu_mean_util"])

    def opt(key, cls):
        raw = body.pop(key, None)
        return cls(**raw) if raw else None

    result = BenchResult(telemetry=TelemetrySummary(**tele), measured_breakdown=opt("measured_breakdown", MeasuredBreakdown),
                         quality=opt("quality", QualityResult), efficiency=opt("efficiency", Efficiency), **body)
    return RunRecord(d["runid"], BenchConfig(**d["config"]), d["env"], result)


def write_run(record: RunRecord, results_dir: str) -> str:
    folder = os.path.join(results_dir, record.config.name)
    os.makedirs(folder, exist_ok=True)
    path = os.path.join(folder, f"{record.runid}.json")
    with open(path, "w", encoding="utf-8") as f:
        json.dump(_record_to_dict(record), f, indent=2)
    return path


def load_run(path: str) -> RunRecord:
    with open(path, encoding="utf-8") as f:
        return _record_from_dict(json.load(f))


def load_all(name: str, results_dir: str) -> list:
    folder = os.path.join(results_dir, name)
    if not os.path.isdir(folder):
        return []
    names = sorted(n for n in os.listdir(folder) if n.endswith(".json") and not n.endswith(".manifest.json"))
    runs = []
    for n in names:
        try:
            runs.append(load_run(os.path.join(folder, n)))
        except (OSError, ValueError, KeyError, TypeError, AttributeError) as e:
            # one truncated or foreign file must not hide the other runs of the experiment
            warnings.warn(f"skipping unreadable run file {os.path.join(folder, n)}: {type(e).__name__}: {e}")
    return runs


def load_latest(name: str, results_dir: str):
    runs = load_all(name, results_dir)
    return runs[-1] if runs else None


EM_DASH = "—"      # shown for unmeasured values, never a made-up zero

CSV_COLUMNS = ["runid", "name", "plan", "dtype_bytes", "kv_dtype_bytes", "tp", "ep", "prompt_tokens", "decode_tokens",
               "seq_len", "n_repeats", "decode_tok_per_s", "decode_tok_per_s_std", "ttft_ms_p50", "tpot_p50_ms",
               "tpot_p95_ms", "e2e_ms_p50", "mbu_decode", "mfu_prefill", "mfu_decode", "ai_decode", "roofline_ridge",
               "regime_decode", "kv_byte_share", "pct_of_peak_bw", "pct_of_floor", "energy_j_per_token",
               "util_imbalance"]


def _stat(latency: Optional[dict], key: str, field: str):
    entry = (latency or {}).get(key)
    return entry.get(field) if entry else None


def record_row(record: RunRecord) -> dict:
    r, c = record.result, record.config
    e, t = r.efficiency, r.telemetry
    row = {k: getattr(c, k) for k in ("plan", "dtype_bytes", "kv_dtype_bytes", "tp", "ep", "prompt_tokens",
                                      "decode_tokens", "seq_len")}
    row.update(runid=record.runid, name=c.name, n_repeats=r.n_repeats, decode_tok_per_s=r.decode_tok_per_s,
               decode_tok_per_s_std=r.decode_tok_per_s_std, ttft_ms_p50=_stat(r.latency, "ttft_ms", "p50"),
               tpot_p50_ms=1e3 * r.tpot_p50_s, tpot_p95_ms=1e3 * r.tpot_p95_s,
               e2e_ms_p50=_stat(r.latency, "e2e_ms", "p50"), pct_of_peak_bw=r.pct_of_peak_bw,
               pct_of_floor=r.pct_of_floor,
               energy_j_per_token=t.energy_j_per_token if t.available else None,
               util_imbalance=t.util_imbalance if t.available else None)
    for k in ("mbu_decode", "mfu_prefill", "mfu_decode", "ai_decode", "roofline_ridge", "regime_decode",
              "kv_byte_share"):
        row[k] = getattr(e, k) if e else None
    return row


def export_csv(records: list, path: str) -> str:
    with open(path, "w", newline="", encoding="utf-8") as f:
        w = csv.DictWriter(f, fieldnames=CSV_COLUMNS)
        w.writeheader()
        for rec in records:
            row = record_row(rec)
            w.writerow({k: EM_DASH if row.get(k) is None else row[k] for k in CSV_COLUMNS})
    return path


def export_jsonl(records: list, path: str) -> str:
    with open(path, "w", encoding="utf-8") as f:
        f.writelines(json.dumps(_record_to_dict(rec)) + "\n" for rec in records)
    return path


def _md_cell(v) -> str:
    if v is None:
        return EM_DASH
    return f"{v:.4g}" if isinstance(v, float) else str(v)


def export_markdown(records: list, path: str) -> str:
    lines = ["| " + " | ".join(CSV_COLUMNS) + " |", "| " + " | ".join("---" for _ in CSV_COLUMNS) + " |"]
    for rec in records:
        row = record_row(rec)
        lines.append("| " + " | ".join(_md_cell(row.get(c)) for c in CSV_COLUMNS) + " |")
    with open(path, "w", encoding="utf-8") as f:
        f.write("\n".join(lines) + "\n")
    return path


def result_to_x_summary(record: RunRecord) -> dict:
    """The server's ``x_summary`` vocabulary for a stored run."""
    r = record.result
    return {"ttft_ms": round(1e3 * r.ttft_s, 3), "decode_tok_per_s": r.decode_tok_per_s,
            "prefill_tokens": record.config.prompt_tokens, "completion_tokens": r.n_decode_tokens}
