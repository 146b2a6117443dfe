"""report.html from benchmark lines: tok/s and bandwidth use against context, the per-phase breakdown of the
persistent kernel, TTFT and the latency table. Input: a file of JSON lines as printed by ``bench.py`` (one per
context length / GPU count); output: one self-contained HTML page with inline SVG charts (no external assets).
Reference: tools/gen_report.py (builds the same page from the text log of its context sweep).
"""
from __future__ import annotations

import html
import json
import sys
from typing import Dict, List

ACTIVE_PARAMS = 22.0e9


def load_lines(path: str) -> List[dict]:
    rows = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line.startswith("{"):
                try:
                    rows.append(json.loads(line))
                except json.JSONDecodeError:
                    pass
    return [r for r in rows if "value" in r]


def derive(r: dict, hbm_gbs: float, weight_bytes_per_gpu: float, peak_flops: float) -> dict:
    """Adds modelled figures to a measured line: bandwidth use (weight bytes per GPU / step time / copy peak) and
    decode MFU (2 x active parameters per token)."""
    ms = float(r.get("ms_per_step") or 1000.0 / r["value"])
    n = int(r.get("n_gpus", 1))
    cfg = r.get("config", {})
    out = dict(r)
    out["ctx"] = int(cfg.get("prompt", cfg.get("seq_len", 0)) or 0)
    out["mbu"] = weight_bytes_per_gpu / (ms * 1e-3) / (hbm_gbs * 1e9)
    out["mfu"] = 2 * ACTIVE_PARAMS / (ms * 1e-3) / (peak_flops * n)
    return out


def _svg_line(points, w=520, h=220, label="") -> str:
    if not points:
        return ""
    xs, ys = [p[0] for p in points], [p[1] for p in points]
    x0, x1, y1 = min(xs), max(xs) or 1, max(ys) * 1.1 or 1
    sx = lambda x: 50 + (w - 70) * ((x - x0) / (x1 - x0) if x1 > x0 else 0.5)
    sy = lambda y: h - 30 - (h - 50) * (y / y1)
    path = " ".join(f"{'M' if i == 0 else 'L'}{sx(x):.1f},{sy(y):.1f}" for i, (x, y) in enumerate(points))
    dots = "".join(f'<circle cx="{sx(x):.1f}" cy="{sy(y):.1f}" r="3"><title>{x}: {y:.3g}</title></circle>' for x, y in points)
    ticks = "".join(f'<text x="{sx(x):.1f}" y="{h - 12}" font-size="10" text-anchor="middle">{x}</text>' for x in xs)
    return (f'<svg width="{w}" height="{h}" role="img"><text x="8" y="14" font-size="12">{html.escape(label)}</text>'
            f'<line x1="50" y1="{h - 30}" x2="{w - 20}" y2="{h - 30}" stroke="#999"/>'
            f'<line x1="50" y1="20" x2="50" y2="{h - 30}" stroke="#999"/>'
            f'<text x="46" y="{sy(max(ys)):.1f}" font-size="10" text-anchor="end">{max(ys):.3g}</text>'
            f'<path d="{path}" fill="none" stroke="#1f6feb" stroke-width="2"/><g fill="#1f6feb">{dots}</g>{ticks}</svg>')


def _table(rows: List[Dict], cols: List[str]) -> str:
    head = "".join(f"<th>{html.escape(c)}</th>" for c in cols)
    body = ""
    for r in rows:
        body += "<tr>" + "".join(
            f"<td>{html.escape(f'{r.get(c):.3f}' if isinstance(r.get(c), float) else str(r.get(c, '')))}</td>" for c in cols) + "</tr>"
    return f"<table><tr>{head}</tr>{body}</table>"


def build(rows: List[dict], hbm_gbs: float = 6561.6, weight_bytes_per_gpu: float = 2.9e9, peak_flops: float = 3.3e15,
          title: str = "B = 1 decode report") -> str:
    d = sorted((derive(r, hbm_gbs, weight_bytes_per_gpu, peak_flops) for r in rows), key=lambda r: (r.get("n_gpus", 1), r["ctx"]))
    charts = ""
    for n in sorted({r.get("n_gpus", 1) for r in d}):
        sel = [r for r in d if r.get("n_gpus", 1) == n]
        charts += _svg_line([(r["ctx"], r["value"]) for r in sel], label=f"tok/s vs context, {n} GPU(s)")
        charts += _svg_line([(r["ctx"], 100 * r["mbu"]) for r in sel], label=f"% of measured copy bandwidth, {n} GPU(s)")
    phases = [dict(gpus=r.get("n_gpus", 1), ctx=r["ctx"], **r["phase_us"]) for r in d if isinstance(r.get("phase_us"), dict)]
    lat = [{"gpus": r.get("n_gpus", 1), "ctx": r["ctx"], "tok_s": float(r["value"]), "ms_per_step": float(r.get("ms_per_step", 0)),
            "tpot_p50_ms": r.get("tpot_p50_ms", ""), "tpot_p95_ms": r.get("tpot_p95_ms", ""), "ttft_ms": r.get("ttft_ms", ""),
            "e2e_tok_s": (r.get("e2e") or {}).get("value", ""), "mbu": r["mbu"], "mfu_decode_modelled": r["mfu"]} for r in d]
    page = f"""<!doctype html><html><head><meta charset="utf-8"><title>{html.escape(title)}</title>
<style>body{{font:14px system-ui;margin:24px;max-width:1100px}}table{{border-collapse:collapse;margin:12px 0}}
td,th{{border:1px solid #ccc;padding:4px 8px;text-align:right}}th{{background:#f3f3f3}}svg{{margin:8px 16px 8px 0}}</style></head>
<body><h1>{html.escape(title)}</h1>
<p>Measured: tok/s, TPOT, TTFT, per-phase times (device clocks). Modelled from the model shape and the measured step time:
bandwidth use and decode MFU.</p>{charts}
<h2>Latency table</h2>{_table(lat, list(lat[0].keys()) if lat else [])}
<h2>Per-phase breakdown of the persistent kernel (microseconds per layer; head and token update per token)</h2>
{_table(phases, list(phases[0].keys())) if phases else '<p>no per-phase data in the input (run the bench with IHB_MEGA_PROF=1)</p>'}
</body></html>"""
    return page


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        print("usage: python -m inferencehackathon_b200.experiments.html_report <bench_lines.jsonl> [report.html]")
        return 2
    rows = load_lines(argv[0])
    out = argv[1] if len(argv) > 1 else "report.html"
    with open(out, "w") as f:
        f.write(build(rows))
    print(f"{len(rows)} runs -> {out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
