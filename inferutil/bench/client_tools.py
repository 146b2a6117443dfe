"""Stand-alone client-side tools over the OpenAI-compatible SSE endpoint (standard library only, no package imports
at run time besides this file's own helpers):

    python -m inferutil.bench.client_tools measure  --base http://127.0.0.1:8000 --ctx 2048 --decode 128 --repeats 5
    python -m inferutil.bench.client_tools roofline --ctx 4096 --weight-bytes 1 --kv-bytes 2 [--tpot-ms 2.3] [--gpu b200]
    python -m inferutil.bench.client_tools next     --base ... --ctx 32768 --label tp8-fp8 --out results.jsonl

``measure`` streams the same request several times and reports TTFT / TPOT / decode tok/s from the client's wall clock
as distributions (mean, percentiles, Student-t 95 % interval). ``roofline`` turns a TPOT into MFU / MBU, the regime
and the dominant time term. ``next`` measures, analyses and appends one JSON line with the levers to try next.
Reference: bench/measure.py:61-131, bench/roofline.py:18-89, bench/sweep.py:14-62 (8 x H100 constants there; the GPU is
a parameter here).
"""
from __future__ import annotations

import argparse
import json
import sys
import time
import urllib.request
from math import sqrt
from typing import Dict, List, Optional

_T95 = [12.706, 4.303, 3.182, 2.776, 2.571, 2.447, 2.365, 2.306, 2.262, 2.228, 2.201, 2.179, 2.160, 2.145, 2.131,
        2.120, 2.110, 2.101, 2.093, 2.086, 2.080, 2.074, 2.069, 2.064, 2.060, 2.056, 2.052, 2.048, 2.045, 2.042]

# per-GPU peaks: HBM bytes/s, dense bf16 FLOP/s, dense fp8 FLOP/s
GPUS = {"h100": (3.35e12, 989.4e12, 1978.9e12), "b200": (7.7e12, 2.25e15, 4.5e15), "b200-measured": (6.56e12, 1.65e15, 3.3e15)}
ACTIVE_PARAMS = 21.57e9            # Qwen3-235B-A22B per-token active parameters (attention + router + 8 experts + head)
KV_ELEMS_PER_TOKEN = 94 * 4 * 128 * 2


def t95(df: int) -> float:
    if df <= 0:
        return float("inf")
    return _T95[df - 1] if df <= 30 else 1.96


def percentile(sorted_vals: List[float], p: float) -> Optional[float]:
    if not sorted_vals:
        return None
    k = (len(sorted_vals) - 1) * p
    lo = int(k)
    hi = min(lo + 1, len(sorted_vals) - 1)
    return sorted_vals[lo] + (sorted_vals[hi] - sorted_vals[lo]) * (k - lo)


def summarize(xs) -> Dict:
    xs = [x for x in xs if x is not None]
    n = len(xs)
    if n == 0:
        return {"n": 0}
    mean = sum(xs) / n
    sv = sorted(xs)
    out = {"n": n, "mean": mean, "min": sv[0], "max": sv[-1]}
    for name, p in (("p50", .5), ("p90", .9), ("p95", .95), ("p99", .99)):
        out[name] = percentile(sv, p)
    if n > 1:
        std = sqrt(sum((x - mean) ** 2 for x in xs) / (n - 1))
        half = t95(n - 1) * std / sqrt(n)
        out.update(std=std, ci95_lo=mean - half, ci95_hi=mean + half)
    return out


def stream_once(base: str, prompt: str, decode: int, engine: Optional[str] = None, model: str = "qwen3-235b-a22b",
                temperature: float = 0.0, timeout: float = 600.0) -> Dict:
    body = {"model": model, "messages": [{"role": "user", "content": prompt}], "max_tokens": decode,
            "temperature": temperature, "stream": True}
    if engine:
        body["engine"] = engine
    req = urllib.request.Request(base.rstrip("/") + "/v1/chat/completions", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    t0 = time.perf_counter()
    stamps: List[float] = []
    summary = None
    error = None
    with urllib.request.urlopen(req, timeout=timeout) as r:
        for raw in r:
            line = raw.decode().strip()
            if not line.startswith("data:"):
                continue
            payload = line[5:].strip()
            if payload == "[DONE]":
                break
            obj = json.loads(payload)
            if "error" in obj:
                error = obj["error"]
                break
            ch = obj.get("choices")
            if ch and ch[0].get("delta", {}).get("content"):
                stamps.append(time.perf_counter())
            if "x_summary" in obj:
                summary = obj["x_summary"]
    gaps = [(b - a) * 1e3 for a, b in zip(stamps, stamps[1:])]
    n = len(stamps)
    return {"ttft_ms": (stamps[0] - t0) * 1e3 if stamps else 0.0, "tpot_ms": sum(gaps) / len(gaps) if gaps else 0.0,
            "decode_tok_s": (n - 1) / (stamps[-1] - stamps[0]) if n > 1 and stamps[-1] > stamps[0] else 0.0,
            "tokens": n, "inter_ms": gaps, "server_summary": summary, "error": error}


def measure(base: str, ctx: int, decode: int, repeats: int = 5, warmup: int = 1, engine=None, model="qwen3-235b-a22b",
            temperature: float = 0.0) -> Dict:
    prompt = ("Summarize the following. " + "context " * max(0, ctx)).strip()
    for _ in range(warmup):
        stream_once(base, "warm up", 8, engine, model)
    runs = [stream_once(base, prompt, decode, engine, model, temperature) for _ in range(max(1, repeats))]
    return {"ttft_ms": summarize([r["ttft_ms"] for r in runs]),
            "tpot_ms": summarize([g for r in runs for g in r["inter_ms"]]),
            "decode_tok_s": summarize([r["decode_tok_s"] for r in runs]),
            "tokens": runs[-1]["tokens"], "repeats": len(runs), "server_summary": runs[-1]["server_summary"],
            "errors": [r["error"] for r in runs if r["error"]]}


HINTS = {"weight_bw": "weights dominate: narrower expert weights, speculative decoding",
         "kv_bw": "KV dominates: fp8 KV, prefix reuse, shorter context",
         "kernel_gap": "below the floor: fewer launches (persistent kernel / graphs), fused epilogues, kernel tuning"}
NEXT_LEVER = {"weight_bw": ["weight dtype bf16 -> fp8 (-> fp4) on experts", "speculative decoding n-gram -> draft head", "longer drafts"],
              "kv_bw": ["KV dtype bf16 -> fp8", "prefix reuse / shorter context", "KV compression"],
              "comms": ["layout ep8 -> tp2ep4 -> tp8 (fewer collectives)", "fused GEMV + all-reduce kernels", "in-kernel dispatch/combine"],
              "kernel_gap": ["persistent decode kernel / CUDA graphs", "fused dequant + epilogues", "profile the top kernel"],
              "compute": ["unusual at one token: check that dequantisation is off the math path"]}


def analyze(ctx: int, tpot_ms: float, weight_bytes: float = 1.0, kv_bytes: float = 1.0, gpu: str = "b200",
            n_gpus: int = 8) -> Dict:
    bw, bf16, fp8 = GPUS[gpu]
    agg = bw * n_gpus
    w = ACTIVE_PARAMS * weight_bytes
    kv = KV_ELEMS_PER_TOKEN * ctx * kv_bytes
    total = w + kv
    peak = (bf16 if weight_bytes >= 2 else fp8) * n_gpus
    tok_s = 1e3 / tpot_ms
    read_ms = total / agg * 1e3
    terms = {"weight_bw": w / agg * 1e3, "kv_bw": kv / agg * 1e3, "kernel_gap": max(0.0, tpot_ms - read_ms)}
    dom = max(terms, key=terms.get)
    ai = 2.0 * ACTIVE_PARAMS / total
    return {"weight_GB": w / 1e9, "kv_GB": kv / 1e9, "total_GB": total / 1e9, "roofline_tok_s": agg / total,
            "ideal_TPOT_ms": read_ms, "achieved_frac": tok_s / (agg / total), "mfu": 2.0 * ACTIVE_PARAMS * tok_s / peak,
            "mbu": total * tok_s / agg, "arithmetic_intensity": ai, "roofline_ridge": peak / agg,
            "regime": "memory-bound" if ai < peak / agg else "compute-bound", "overhead_ms": terms["kernel_gap"],
            "dominant_term": dom, "recommendation": HINTS[dom], "gpu": gpu, "n_gpus": n_gpus}


def _fmt(s: Dict) -> str:
    if s.get("n", 0) < 2:
        return f"{s.get('mean', 0):.2f}"
    return f"{s['mean']:.2f} (p50 {s['p50']:.2f} / p95 {s['p95']:.2f}, 95% CI {s['ci95_lo']:.2f}-{s['ci95_hi']:.2f}, n={s['n']})"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="inferutil.bench.client_tools")
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("measure", "next"):
        p = sub.add_parser(name)
        p.add_argument("--base", default="http://127.0.0.1:8000")
        p.add_argument("--ctx", type=int, default=2048)
        p.add_argument("--decode", type=int, default=128)
        p.add_argument("--engine", default=None)
        p.add_argument("--model", default="qwen3-235b-a22b")
        p.add_argument("--warmup", type=int, default=1)
        p.add_argument("--repeats", type=int, default=5)
        p.add_argument("--temperature", type=float, default=0.0)
        if name == "next":
            p.add_argument("--label", default="run")
            p.add_argument("--out", default="results.jsonl")
            p.add_argument("--weight-bytes", type=float, default=1.0)
            p.add_argument("--kv-bytes", type=float, default=2.0)
            p.add_argument("--gpu", default="b200", choices=sorted(GPUS))
            p.add_argument("--n-gpus", type=int, default=8)
    p = sub.add_parser("roofline")
    p.add_argument("--ctx", type=int, default=32768)
    p.add_argument("--weight-bytes", type=float, default=1.0, help="1 = fp8, 0.5 = fp4/int4, 2 = bf16")
    p.add_argument("--kv-bytes", type=float, default=2.0)
    p.add_argument("--tpot-ms", type=float, default=None)
    p.add_argument("--gpu", default="b200", choices=sorted(GPUS))
    p.add_argument("--n-gpus", type=int, default=8)
    a = ap.parse_args(argv)
    if a.cmd == "roofline":
        ideal = analyze(a.ctx, 1.0, a.weight_bytes, a.kv_bytes, a.gpu, a.n_gpus)
        print(f"ctx={a.ctx}  weights={ideal['weight_GB']:.1f}GB  KV={ideal['kv_GB']:.2f}GB  total={ideal['total_GB']:.1f}GB/token")
        print(f"roofline = {ideal['roofline_tok_s']:.0f} tok/s  (ideal TPOT {ideal['ideal_TPOT_ms']:.2f} ms) on {a.n_gpus} x {a.gpu}")
        if a.tpot_ms:
            for k, v in analyze(a.ctx, a.tpot_ms, a.weight_bytes, a.kv_bytes, a.gpu, a.n_gpus).items():
                print(f"  {k}: {v}")
        return 0
    m = measure(a.base, a.ctx, a.decode, a.repeats, a.warmup, a.engine, a.model, a.temperature)
    if a.cmd == "measure":
        print(json.dumps(m, indent=2))
        print(f"\nTTFT {_fmt(m['ttft_ms'])} ms | TPOT {m['tpot_ms'].get('mean', 0):.2f} ms ({_fmt(m['tpot_ms'])}) | "
              f"decode {_fmt(m['decode_tok_s'])} tok/s | {m['tokens']} tokens, {m['repeats']} repeats")
        return 0
    tpot = m["tpot_ms"].get("mean") or 1e9
    an = analyze(a.ctx, tpot, a.weight_bytes, a.kv_bytes, a.gpu, a.n_gpus)
    rec = {"label": a.label, "ctx": a.ctx, "tpot_ms": tpot, "ttft_ms": m["ttft_ms"].get("mean"),
           "decode_tok_s": m["decode_tok_s"].get("mean"), **an, "next_levers": NEXT_LEVER.get(an["dominant_term"], [])}
    with open(a.out, "a") as f:
        f.write(json.dumps(rec) + "\n")
    print(f"[{a.label}] TPOT {tpot:.2f} ms  {rec['decode_tok_s'] or 0:.0f} tok/s  {an['achieved_frac'] * 100:.0f}% of roofline")
    print(f"  dominant: {an['dominant_term']}\n  try next: {rec['next_levers']}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
