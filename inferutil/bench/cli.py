"""``python -m inferutil.bench <command>`` (reference: src/inferutil/bench/cli.py:36-390): run, report, gate,
diagnose, plan, calibrate, sweep, spec, export, compare. ``run --engine b200`` drives the real engine through the
same seam as the analytical ``mock``."""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from dataclasses import asdict, replace

from ..hardware import GPUS, Cluster, TB
from ..model import QWEN3_235B, QWEN3_30B
from ..speculative import memory_feasibility
from .attribution import diagnose
from .config import BenchConfig
from .engine import MockEngine
from .gate import Thresholds, evaluate, regression_gate
from .levers import recommend
from .manifest import build_manifest
from .report import (format_compare, format_diagnosis, format_plan, format_result, format_spec_floor, format_sweep)
from .runner import run_benchmark
from .spec_model import spec_sweep
from .store import (RunRecord, export_csv, export_jsonl, export_markdown, load_all, load_latest, load_run, write_run)
from .sweep import config_sweep, depth_sweep, full_grid, layout_grid, realized_efficiency
from .telemetry import NullTelemetry, NvmlTelemetry

DEFAULT_RESULTS_DIR = os.environ.get("INFERUTIL_RESULTS", "results")
MODELS = {"qwen3-235b-a22b": QWEN3_235B, "qwen3-30b-a3b": QWEN3_30B}


def _build_config(args) -> BenchConfig:
    return BenchConfig(name=getattr(args, "name", "plan"), plan=args.plan, dtype_bytes=args.dtype,
                       kv_dtype_bytes=args.kv_dtype, tp=args.tp, ep=args.ep, prompt_tokens=args.prompt,
                       decode_tokens=args.decode, repeats=getattr(args, "repeats", 5))


def _unique_runid(results_dir: str, name: str) -> str:
    stamp = time.strftime("%Y%m%d-%H%M%S")
    folder = os.path.join(results_dir, name)
    runid, n = stamp, 1
    while os.path.exists(os.path.join(folder, runid + ".json")):
        n += 1
        runid = f"{stamp}-{n}"
    return runid


def _measured_cluster(cluster: Cluster, peak_bw_gbs) -> Cluster:
    """Replace the nominal per-GPU bandwidth with a measured one (GB/s) when given."""
    if not peak_bw_gbs:
        return cluster
    return Cluster(replace(cluster.gpu, hbm_bw=peak_bw_gbs * 1e9), cluster.n_gpus)


def _cluster(args) -> Cluster:
    return _measured_cluster(Cluster(GPUS[args.gpu], args.n_gpus), getattr(args, "peak_bw_gbs", None))


def _cluster_from_env(rec: RunRecord) -> Cluster:
    gpu = GPUS.get(rec.env.get("gpu", ""), GPUS["H100-SXM-80GB"])
    return _measured_cluster(Cluster(gpu, rec.env.get("n_gpus", 8)), rec.env.get("peak_bw_gbs"))


def _cmd_run(args) -> None:
    cluster, config = _cluster(args), _build_config(args)
    cfg = MODELS[args.model]
    if args.engine == "mock":
        engine = MockEngine(cfg, cluster, efficiency=args.efficiency, jitter=args.jitter, seed=config.seed)
    else:
        from inferencehackathon_b200.runtime.bench_adapter import B200Engine   # imported only when asked for
        engine = B200Engine.from_cli(args)
    tele = NvmlTelemetry() if args.telemetry else NullTelemetry()
    result = run_benchmark(engine, config, cfg, cluster, telemetry=tele if tele.available else NullTelemetry())
    runid = _unique_runid(args.results_dir, config.name)
    env = {"gpu": cluster.gpu.name, "n_gpus": cluster.n_gpus, "engine": args.engine, "model": cfg.name,
           "peak_bw_gbs": args.peak_bw_gbs}
    record = RunRecord(runid, config, env, result)
    path = write_run(record, args.results_dir)
    manifest = build_manifest(cfg, cluster, config, peak_bw_measured=(args.peak_bw_gbs * 1e9 if args.peak_bw_gbs else None),
                              cli=" ".join(sys.argv), runid=runid)
    with open(path[:-5] + ".manifest.json", "w", encoding="utf-8") as f:
        json.dump(manifest, f, indent=2)
    print(json.dumps({"runid": runid, "path": path, "result": asdict(result)}) if args.json else format_result(record))


def _resolve(args) -> RunRecord:
    if args.runid == "latest":
        rec = load_latest(args.name, args.results_dir)
        if rec is None:
            raise SystemExit(f"no runs stored for '{args.name}' under {args.results_dir}")
        return rec
    path = args.runid if os.path.exists(args.runid) else os.path.join(args.results_dir, args.name, args.runid + ".json")
    if not os.path.exists(path):
        raise SystemExit(f"run not found: {path}")
    return load_run(path)


def _cmd_report(args) -> None:
    rec = _resolve(args)
    print(json.dumps(asdict(rec.result)) if args.json else format_result(rec))


def _cmd_gate(args) -> None:
    rec = _resolve(args)
    res = evaluate(rec.result, Thresholds(args.min_tok_s, args.max_ttft_s, args.min_pct_floor, args.min_quality))
    fails = list(res.failures)
    if args.baseline:
        base = load_run(args.baseline) if os.path.exists(args.baseline) else \
            load_run(os.path.join(args.results_dir, args.name, args.baseline + ".json"))
        fails += list(regression_gate(base.result, rec.result).failures)
    if fails:
        print("GATE FAIL")
        for f in fails:
            print("  - " + f)
        raise SystemExit(1)
    print("GATE PASS")


def _cmd_diagnose(args) -> None:
    rec = _resolve(args)
    b = diagnose(rec.result)
    cfg = MODELS.get(str(rec.env.get("model", "")).lower(), QWEN3_235B)
    levers = recommend(cfg, _cluster_from_env(rec), rec.config, bottleneck=b, min_speedup=args.min_speedup)
    print(format_diagnosis(rec, levers))


def _analytic_record(args, cluster, config) -> RunRecord:
    engine = MockEngine(QWEN3_235B, cluster, efficiency=args.efficiency)
    result = run_benchmark(engine, replace(config, repeats=1, warmup_steps=0), QWEN3_235B, cluster)
    return RunRecord("analytical", config, {"gpu": cluster.gpu.name, "n_gpus": cluster.n_gpus}, result)


def _cmd_plan(args) -> None:
    cluster, config = _cluster(args), _build_config(args)
    rec = _analytic_record(args, cluster, config)
    b = diagnose(rec.result)
    levers = recommend(QWEN3_235B, cluster, config, bottleneck=b)
    pts = config_sweep(QWEN3_235B, cluster, layout_grid(config, cluster.n_gpus), efficiency=args.efficiency)
    print(format_plan(rec, b, levers, pts[0] if pts else None))


def _cmd_calibrate(args) -> None:
    cluster, config = _cluster(args), _build_config(args)
    e, floor = realized_efficiency(QWEN3_235B, cluster, config, args.measured_tok_s)
    print(f"analytical floor {floor:.1f} tok/s; measured {args.measured_tok_s:.1f} tok/s -> realized efficiency "
          f"{e:.3f}" if e is not None else "floor is zero")
    print(f"re-run sweeps/plan with --efficiency {e:.3f}" if e is not None else "")


def _cmd_sweep(args) -> None:
    cluster, config = _cluster(args), _build_config(args)
    if args.full:
        pts = config_sweep(QWEN3_235B, cluster, full_grid(config, cluster.n_gpus), efficiency=args.efficiency)
        title = "quantisation x layout sweep"
    elif args.layout:
        pts = config_sweep(QWEN3_235B, cluster, layout_grid(config, cluster.n_gpus), efficiency=args.efficiency)
        title = "layout sweep"
    else:
        depths = [int(x) for x in args.depths.split(",")] if args.depths else [1024, 2048, 4096, 8192, 16384, 32768]
        pts = depth_sweep(QWEN3_235B, cluster, config, depths, efficiency=args.efficiency)
        title = "context-depth sweep"
    print(format_sweep(pts, n_gpus=cluster.n_gpus, usd_per_gpu_hr=args.gpu_hr, title=title))


def _cmd_spec(args) -> None:
    rows = spec_sweep(args.accept, args.floor, ks=tuple(args.ks), ns=tuple(args.drafters))
    feas = memory_feasibility(draft_model_gb=args.draft_gb, use_fp8_target=not args.bf16_target)
    print(format_spec_floor(rows, feas, accept=args.accept, floor=args.floor, base_tok_s=args.base_tok_s))


def _cmd_export(args) -> None:
    recs = load_all(args.name, args.results_dir)
    fn = {"csv": export_csv, "jsonl": export_jsonl, "md": export_markdown}[args.format]
    print(fn(recs, args.out))


def _cmd_compare(args) -> None:
    def get(x):
        return load_run(x) if os.path.exists(x) else load_run(os.path.join(args.results_dir, args.name, x + ".json"))
    print(format_compare(get(args.a), get(args.b)))


def _common(p, dtype_type=float, dtype_default=1.0, name=False):
    if name:
        p.add_argument("--name", default="default")
    p.add_argument("--gpu", default="H100-SXM-80GB", choices=list(GPUS))
    p.add_argument("--n-gpus", type=int, default=8)
    p.add_argument("--plan", default="hybrid", choices=["tp", "ep", "hybrid"])
    p.add_argument("--dtype", type=dtype_type, default=dtype_default, help="2=bf16, 1=fp8, 0.5=int4")
    p.add_argument("--kv-dtype", type=int, default=2, choices=[1, 2])
    p.add_argument("--tp", type=int, default=2)
    p.add_argument("--ep", type=int, default=8)
    p.add_argument("--prompt", type=int, default=512)
    p.add_argument("--decode", type=int, default=128)
    p.add_argument("--peak-bw-gbs", type=float, default=None, help="measured per-GPU HBM bandwidth in GB/s")


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(prog="inferutil.bench")
    ap.add_argument("--results-dir", default=DEFAULT_RESULTS_DIR)
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("run", help="run a benchmark and store it")
    _common(r, int, 2, name=True)
    r.add_argument("--repeats", type=int, default=5)
    r.add_argument("--efficiency", type=float, default=1.0)
    r.add_argument("--jitter", type=float, default=0.0)
    r.add_argument("--engine", default="mock", choices=["mock", "b200"])
    r.add_argument("--model", default="qwen3-235b-a22b", choices=list(MODELS))
    r.add_argument("--engine-model", default="tiny", help="preset of the real engine (b200 engine only)")
    r.add_argument("--engine-weights", default="fp32")
    r.add_argument("--engine-device", default="cpu")
    r.add_argument("--telemetry", action="store_true")
    r.add_argument("--json", action="store_true")
    r.set_defaults(fn=_cmd_run)
    for name, fn, helptext in (("report", _cmd_report, "print a stored run (default: latest)"),
                               ("gate", _cmd_gate, "pass/fail a stored run against thresholds"),
                               ("diagnose", _cmd_diagnose, "name the dominant bottleneck and next levers")):
        p = sub.add_parser(name, help=helptext)
        p.add_argument("--name", default="default")
        p.add_argument("runid", nargs="?", default="latest")
        p.set_defaults(fn=fn)
        if name == "report":
            p.add_argument("--json", action="store_true")
        if name == "gate":
            p.add_argument("--min-tok-s", type=float, default=None)
            p.add_argument("--max-ttft-s", type=float, default=None)
            p.add_argument("--min-pct-floor", type=float, default=None)
            p.add_argument("--min-quality", type=float, default=None)
            p.add_argument("--baseline", default=None, help="run id or path to regress against")
        if name == "diagnose":
            p.add_argument("--min-speedup", type=float, default=1.02)
    pl = sub.add_parser("plan", help="analytical plan: bottleneck, levers, best layout")
    _common(pl)
    pl.add_argument("--efficiency", type=float, default=1.0)
    pl.set_defaults(fn=_cmd_plan)
    ca = sub.add_parser("calibrate", help="realized efficiency from a measured tok/s")
    _common(ca)
    ca.add_argument("--measured-tok-s", type=float, required=True)
    ca.set_defaults(fn=_cmd_calibrate)
    sw = sub.add_parser("sweep", help="context-depth / layout / full sweeps")
    _common(sw)
    sw.add_argument("--depths", default=None, help="comma-separated context lengths")
    sw.add_argument("--layout", action="store_true")
    sw.add_argument("--full", action="store_true")
    sw.add_argument("--gpu-hr", type=float, default=3.0)
    sw.add_argument("--efficiency", type=float, default=1.0)
    sw.set_defaults(fn=_cmd_sweep)
    sp = sub.add_parser("spec", help="floor-aware speculative decoding sweep")
    sp.add_argument("--accept", type=float, default=0.7)
    sp.add_argument("--floor", type=float, default=0.86)
    sp.add_argument("--ks", type=int, nargs="+", default=[2, 4, 8])
    sp.add_argument("--drafters", type=int, nargs="+", default=[1, 2, 4])
    sp.add_argument("--draft-gb", type=float, default=3.4)
    sp.add_argument("--bf16-target", action="store_true")
    sp.add_argument("--base-tok-s", type=float, default=None)
    sp.set_defaults(fn=_cmd_spec)
    ex = sub.add_parser("export", help="export stored runs to csv / jsonl / md")
    ex.add_argument("--name", default="default")
    ex.add_argument("--format", choices=["csv", "jsonl", "md"], default="csv")
    ex.add_argument("--out", required=True)
    ex.set_defaults(fn=_cmd_export)
    cp = sub.add_parser("compare", help="diff two stored runs")
    cp.add_argument("--name", default="default")
    cp.add_argument("a")
    cp.add_argument("b")
    cp.set_defaults(fn=_cmd_compare)
    args = ap.parse_args(argv)
    args.fn(args)


if __name__ == "__main__":
    main()
