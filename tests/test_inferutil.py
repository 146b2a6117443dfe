"""Analytical model and benchmark harness (CPU only). Mirrors the reference's unit-test strategy: model accounting,
MockEngine == analytical floor, statistics, store/export round trips, gates, levers, sweeps, optimiser, CLI."""
import json
import os

import pytest

import inferutil as iu
from inferutil import bench as B
from inferutil.bench.cli import main as bench_main
from inferutil.optimize import MEASURED_BASELINE, apply_spec, optimize, plain_decode_ceiling, sensitivity_grid

H100 = iu.Cluster(iu.H100_SXM, 8)
CFG = iu.QWEN3_235B


def test_param_accounting():
    assert 234e9 < CFG.total_params < 236e9 and 21e9 < CFG.active_params < 23e9
    assert CFG.kv_bytes_per_token(2) == 2 * 94 * 512 * 2
    assert 30e9 < iu.QWEN3_30B.total_params < 31e9


def test_emax_and_latency_plans():
    assert iu.expected_max_experts_per_gpu(8, 1) == 8.0
    assert abs(iu.expected_max_experts_per_gpu(8, 8) - 2.597) < 1e-3
    floor = iu.decode_latency(CFG, H100, plan="floor", dtype_bytes=1, seq_len=2048)
    tp = iu.decode_latency(CFG, H100, plan="tp", dtype_bytes=1, seq_len=2048)
    ep = iu.decode_latency(CFG, H100, plan="ep", dtype_bytes=1, seq_len=2048)
    ideal = iu.decode_latency(CFG, H100, plan="ep", dtype_bytes=1, seq_len=2048, ideal_routing=True)
    assert floor.total_s < tp.total_s < ep.total_s and ideal.total_s < ep.total_s and ep.imbalance > 2.5
    assert tp.comms_s == pytest.approx(188 * 5e-6)
    b200 = iu.decode_latency(CFG, iu.Cluster(iu.B200_SXM, 8), plan="tp", dtype_bytes=1, seq_len=2048)
    assert b200.tokens_per_s > tp.tokens_per_s
    with pytest.raises(ValueError):
        iu.decode_latency(CFG, H100, plan="nope")


def test_mock_engine_reproduces_the_floor():
    cfgb = B.BenchConfig("t", "hybrid", 1, 2, 2, 8, prompt_tokens=64, decode_tokens=16, repeats=2, warmup_steps=2)
    eng = B.MockEngine(CFG, H100)
    assert isinstance(eng, B.Engine)
    res = B.run_benchmark(eng, cfgb, CFG, H100, telemetry=B.FakeTelemetrySource([
        B.GpuSample(g, 0.0, 60.0, 50.0 + g, 40.0, 300.0, 1500.0, 2000.0, 1 << 30) for g in range(2)]))
    assert res.pct_of_floor == pytest.approx(1.0, rel=1e-9)
    assert res.telemetry.available and res.telemetry.n_gpus == 2 and res.telemetry.power_w_mean == pytest.approx(600.0)
    slow = B.run_benchmark(B.MockEngine(CFG, H100, efficiency=0.5, jitter=0.1, seed=3, expose_routes=True), cfgb, CFG, H100)
    assert 0.4 < slow.pct_of_floor < 0.6 and slow.tpot_p95_s >= slow.tpot_p50_s
    step = B.MockEngine(CFG, H100, expose_routes=True)
    step.reset(plan="tp", dtype_bytes=1, kv_dtype_bytes=2, tp=8, ep=1, seq_len=128)
    s = step.decode_step()
    assert len(s.routes) == 8 and all(0 <= r.gpu < 8 for r in s.routes)
    with pytest.raises(ValueError):
        B.run_benchmark(eng, B.BenchConfig("x", "tp", 1, 2, 8, 1, decode_tokens=1), CFG, H100)


def test_stats_and_quality():
    s = B.summarize([1.0, 2.0, 3.0, 4.0])
    assert s.mean == 2.5 and s.ci95_lo < 2.5 < s.ci95_hi and s.p50 == 2.5
    assert B.summarize([]).n == 0 and B.summarize([5]).std is None
    a, b = B.summarize([10, 10.1, 9.9]), B.summarize([20, 20.1, 19.9])
    assert B.means_differ(a, b) and not B.means_differ(a, a)
    q = B.match_rate([1, 2, 3, 4], [1, 2, 9, 4])
    assert q.match_rate == 0.75 and q.first_divergence == 2


def test_store_roundtrip_exports_and_gates(tmp_path):
    cfgb = B.BenchConfig("rt", "tp", 2, 2, 8, 1, prompt_tokens=32, decode_tokens=8, repeats=3, warmup_steps=1)
    res = B.run_benchmark(B.MockEngine(CFG, H100, jitter=0.05, seed=1), cfgb, CFG, H100, reference_ids=[0] * 7)
    rec = B.RunRecord("r1", cfgb, {"gpu": "H100-SXM-80GB", "n_gpus": 8}, res)
    path = B.write_run(rec, str(tmp_path))
    back = B.load_run(path)
    assert back.result.decode_tok_per_s == res.decode_tok_per_s and back.config == cfgb
    assert B.load_latest("rt", str(tmp_path)).runid == "r1"
    row = B.record_row(back)
    assert row["energy_j_per_token"] is None and row["regime_decode"] == "memory-bound"
    for fn, ext in ((B.export_csv, "csv"), (B.export_jsonl, "jsonl"), (B.export_markdown, "md")):
        assert os.path.getsize(fn([back], str(tmp_path / f"o.{ext}"))) > 0
    assert set(B.result_to_x_summary(back)) == {"ttft_ms", "decode_tok_per_s", "prefill_tokens", "completion_tokens"}
    assert B.evaluate(res, B.Thresholds(min_decode_tok_per_s=1.0)).passed
    assert not B.evaluate(res, B.Thresholds(min_decode_tok_per_s=1e9, min_quality_match=0.99)).passed
    slow = B.run_benchmark(B.MockEngine(CFG, H100, efficiency=0.5, jitter=0.01, seed=2), cfgb, CFG, H100)
    assert not B.regression_gate(res, slow).passed and B.regression_gate(slow, res).passed
    man = B.build_manifest(CFG, H100, cfgb, runid="r1")
    assert man["bench"]["config_id"] == B.config_id(cfgb) and len(B.model_hash(CFG)) == 12


def test_diagnose_levers_sweeps_and_spec_model():
    cfgb = B.BenchConfig("d", "hybrid", 1, 2, 2, 8, prompt_tokens=512, decode_tokens=16, repeats=1, warmup_steps=0)
    res = B.run_benchmark(B.MockEngine(CFG, H100, efficiency=0.4), cfgb, CFG, H100)
    b = B.diagnose(res)
    assert b.dominant_term == "kernel_gap" and 0.5 <= b.confidence <= 1.0
    levers = B.recommend(CFG, H100, cfgb, bottleneck=b)
    assert levers and all(lv.speedup >= 1.02 for lv in levers) and levers == sorted(levers, key=lambda l: -l.speedup)
    pts = B.depth_sweep(CFG, H100, cfgb, [1024, 32768])
    assert pts[0].decode_tok_s > pts[1].decode_tok_s and pts[1].kv_byte_share > pts[0].kv_byte_share
    assert len(B.layout_grid(cfgb, 8)) == 16 and len(B.quant_grid(cfgb)) == 6 and len(B.full_grid(cfgb, 8)) == 96
    ranked = B.config_sweep(CFG, H100, B.layout_grid(cfgb, 8))
    assert ranked[0].decode_tok_s >= ranked[-1].decode_tok_s
    e, floor = B.realized_efficiency(CFG, H100, cfgb, 80.0)
    assert 0 < e < 1 and floor > 80
    assert B.expected_emitted(0.7, 4) == pytest.approx((1 - 0.7 ** 5) / 0.3)
    assert B.verify_cost(4, 1, 1.0) == pytest.approx(1.0) and B.verify_cost(8, 4, 0.0) > B.verify_cost(2, 1, 0.0)
    rows = B.spec_sweep(0.7, 0.86)
    assert rows[0].speedup == max(r.speedup for r in rows)
    assert B.prefill_latency(CFG, H100, dtype_bytes=1, kv_dtype_bytes=2, prompt_tokens=2048) > \
        B.prefill_latency(CFG, H100, dtype_bytes=1, kv_dtype_bytes=2, prompt_tokens=128)
    assert B.rental_usd_per_mtok(100.0, 8) == pytest.approx(8 * 3.0 / 3600 / 100 * 1e6)
    assert B.energy_metrics(None, None)["joules_per_token"] is None


def test_optimiser_is_monotone():
    final, steps = optimize()
    assert final.tok_s > MEASURED_BASELINE.tok_s and all(s.after_tok_s >= s.before_tok_s for s in steps if s.kept)
    assert all(s.status != "MISSING" or "UNMEASURED" in s.note for s in steps)
    lossy, _ = optimize(allow_lossy=True)
    assert lossy.tok_s >= final.tok_s
    sp = apply_spec(final)
    assert sp.spec_tok_s > sp.plain_tok_s and 0 <= sp.floor_fraction <= 1
    c = plain_decode_ceiling()
    assert c["hard_floor_fp8_weight"] > c["optimistic_overlap"] > c["conservative_nvls2us"]
    assert sensitivity_grid()[0]["min_overlap_for_1000"] is not None


def test_routing_graph_and_speculative_math():
    g = iu.CoActGraph(n_experts=16, n_layers=2)
    iu.ingest_telemetry(g, [{"token_index": 0, "experts": [{"layer": 0, "expert_id": e, "gpu": 0} for e in (0, 1, 2, 3)]
                             + [{"layer": 1, "expert_id": e, "gpu": 0} for e in (4, 5)]}] * 5)
    assert g.total_edge_weight() == 5 * (6 + 1 + 8)
    gp = iu.greedy_partition(g, n_gpus=4, n_experts=16, n_layers=2)
    rr = iu.round_robin_placement(4, 16, 2)
    assert iu.placement_stats(g, gp)["cross_gpu_weight"] <= iu.placement_stats(g, rr)["cross_gpu_weight"]
    assert sorted(list(gp.values()).count(x) for x in range(4)) == [8, 8, 8, 8]
    dag = iu.TokenDAG()
    dag.add_layer(0, [0, 1]); dag.add_layer(1, [4, 5])
    plan = dag.prefetch_schedule(gp, 16)
    assert plan[0]["prefetch_layer"] == 1 and len(plan[0]["prefetch_experts"]) == 2
    assert iu.expected_accepted_multi(0.7, 4, 2) > iu.expected_accepted_multi(0.7, 4, 1)
    assert iu.expected_accepted_single(1.0, 4) == 4.0 and iu.memory_feasibility()["max_drafters"] > 0


def test_cli_smoke(tmp_path, capsys):
    d = str(tmp_path)
    bench_main(["--results-dir", d, "run", "--name", "c", "--repeats", "2", "--decode", "8", "--prompt", "16"])
    bench_main(["--results-dir", d, "run", "--name", "c", "--repeats", "2", "--decode", "8", "--prompt", "16", "--json"])
    bench_main(["--results-dir", d, "report", "--name", "c"])
    bench_main(["--results-dir", d, "gate", "--name", "c", "--min-pct-floor", "0.9"])
    bench_main(["--results-dir", d, "diagnose", "--name", "c"])
    runs = sorted(f[:-5] for f in os.listdir(os.path.join(d, "c")) if f.endswith(".json") and "manifest" not in f)
    assert len(runs) == 2
    bench_main(["--results-dir", d, "compare", "--name", "c", runs[0], runs[1]])
    bench_main(["--results-dir", d, "export", "--name", "c", "--format", "csv", "--out", os.path.join(d, "o.csv")])
    for cmd in (["plan"], ["sweep"], ["sweep", "--layout"], ["spec"], ["calibrate", "--measured-tok-s", "90"]):
        bench_main(cmd)
    with pytest.raises(SystemExit):
        bench_main(["--results-dir", d, "gate", "--name", "c", "--min-tok-s", "1e9"])
    from inferutil.cli import main as top
    top(["--gpu", "B200-SXM-180GB", "--n-gpus", "8"])
    out = capsys.readouterr().out
    assert "GATE PASS" in out and "takeaways" in out and not B.NvmlTelemetry().available in (None,)


def test_real_engine_through_the_seam(tmp_path):
    from inferencehackathon_b200.runtime.bench_adapter import B200Engine
    from inferencehackathon_b200.runtime.engine import InferenceEngine
    eng = B200Engine(InferenceEngine.build("tiny", weights="fp32", max_seq=128))
    assert isinstance(eng, B.Engine)
    cfgb = B.BenchConfig("real", "tp", 4, 4, 1, 1, prompt_tokens=16, decode_tokens=6, repeats=2, warmup_steps=1)
    res = B.run_benchmark(eng, cfgb, eng.cfg, eng.cluster, collect_ids=True)
    assert res.decode_tok_per_s > 0 and res.measured_breakdown is not None and len(res.generated_token_ids) == 5
    again = B.run_benchmark(eng, cfgb, eng.cfg, eng.cluster, reference_ids=res.generated_token_ids)
    assert again.quality.match_rate == 1.0
    bench_main(["--results-dir", str(tmp_path), "run", "--name", "real", "--engine", "b200", "--repeats", "1",
                "--prompt", "8", "--decode", "4", "--dtype", "2"])


def test_client_tools_measure_and_roofline_against_the_mock_server():
    """Stand-alone SSE client: TTFT / TPOT distributions from the wall clock; roofline attribution."""
    import threading
    import uvicorn
    from inferutil.bench import client_tools as ct
    from inferencehackathon_b200.serve.app import create_app
    from inferencehackathon_b200.serve.backends import MockBackend
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    server = uvicorn.Server(uvicorn.Config(create_app(MockBackend()), host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    import time
    for _ in range(100):
        if server.started:
            break
        time.sleep(0.05)
    try:
        m = ct.measure(f"http://127.0.0.1:{port}", ctx=8, decode=6, repeats=2, warmup=0, engine="conifer")
        assert m["tokens"] >= 2 and m["ttft_ms"]["n"] == 2 and m["tpot_ms"]["mean"] > 0
        assert m["server_summary"] and "decode_tok_per_s" in m["server_summary"]
    finally:
        server.should_exit = True
        th.join(timeout=5)
    a = ct.analyze(4096, 3.0, 1.0, 2.0, "b200", 8)
    assert a["regime"] == "memory-bound" and a["dominant_term"] == "kernel_gap" and 0 < a["mbu"] < 1
    assert ct.analyze(4096, a["ideal_TPOT_ms"], 1.0, 2.0)["dominant_term"] == "weight_bw"
    s5 = ct.summarize([1.0, 2.0, 3.0, 4.0, 5.0])
    assert s5["p50"] == 3.0 and s5["ci95_lo"] < 3.0 < s5["ci95_hi"] and ct.t95(4) == 2.776
    assert ct.main(["roofline", "--ctx", "1024", "--tpot-ms", "2.5"]) == 0


def test_b200_measured_baseline_is_consistent():
    from inferutil import optimize as O
    b = O.B200_MEASURED
    total = b.overhead_ms + b.comms_ms + b.weight_ms + b.kv_ms
    assert abs(1000.0 / total - O.B200_MEASURED_TOK_S) < 1.0
    final, steps = O.optimize(b)
    assert (final.overhead_ms + final.comms_ms + final.weight_ms + final.kv_ms) <= total


def test_kv_row_split_trades_kv_bytes_for_two_exchanges_per_layer():
    import dataclasses
    from inferutil.hardware import GPUS, Cluster
    from inferutil.latency import decode_latency
    from inferutil.model import QWEN3_235B
    g = dataclasses.replace(GPUS["B200-SXM-180GB"], collective_latency_s=1.4e-6)
    c = Cluster(g, 8)
    kw = dict(plan="tp", dtype_bytes=1, kv_dtype_bytes=2)
    rep = decode_latency(QWEN3_235B, c, seq_len=32768, **kw)
    spl = decode_latency(QWEN3_235B, c, seq_len=32768, kv_seq_split=True, **kw)
    assert spl.kv_read_s == rep.kv_read_s / 2                      # 4 KV heads on 8 ranks: two ranks per head
    assert spl.comms_s == rep.comms_s * 2 and spl.total_s > rep.total_s          # does not pay at 32 K tokens ...
    long_rep = decode_latency(QWEN3_235B, c, seq_len=131072, **kw)
    long_spl = decode_latency(QWEN3_235B, c, seq_len=131072, kv_seq_split=True, **kw)
    assert long_spl.total_s < long_rep.total_s                     # ... but does at 128 K
    # no effect where every rank already owns whole KV heads
    c4 = Cluster(g, 4)
    assert decode_latency(QWEN3_235B, c4, seq_len=32768, kv_seq_split=True, **kw).total_s == \
        decode_latency(QWEN3_235B, c4, seq_len=32768, **kw).total_s


from hypothesis import given, settings, strategies as st   # noqa: E402


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 3), st.sampled_from([8, 16]), st.sampled_from([2, 4, 8]), st.integers(0, 2 ** 31 - 1))
def test_co_activation_partition_places_every_expert_once_with_even_counts(n_layers, n_experts, n_gpus, seed):
    """For any co-activation history: every (layer, expert) gets one GPU in range, every GPU holds exactly
    n_experts / n_gpus experts of a layer, and the edge weight between GPUs plus the weight kept inside GPUs is the
    graph's total (nothing counted twice)."""
    import random
    from inferutil.routing import CoActGraph, greedy_partition, placement_stats, round_robin_placement
    rng = random.Random(seed)
    g = CoActGraph(n_experts=n_experts, n_layers=n_layers)
    for _ in range(60):
        for layer in range(n_layers):
            g.add_token_step(layer, rng.sample(range(n_experts), 4))
    pl = greedy_partition(g, n_gpus=n_gpus, n_experts=n_experts, n_layers=n_layers)
    assert sorted(pl) == list(range(n_layers * n_experts)) and all(0 <= v < n_gpus for v in pl.values())
    for layer in range(n_layers):
        per_gpu = [0] * n_gpus
        for e in range(n_experts):
            per_gpu[pl[g.node_id(layer, e)]] += 1
        assert per_gpu == [n_experts // n_gpus] * n_gpus
    cross = g.cross_gpu_weight(pl)
    assert 0 <= cross <= g.total_edge_weight()
    rr = round_robin_placement(n_gpus, n_experts, n_layers)
    st_g, st_r = placement_stats(g, pl, "greedy"), placement_stats(g, rr, "rr")
    assert st_g["label"] == "greedy" and st_r["label"] == "rr"


def test_an_unreadable_run_file_does_not_hide_the_other_runs(tmp_path):
    import warnings
    cfgb = B.BenchConfig("rt", "tp", 2, 2, 8, 1, prompt_tokens=32, decode_tokens=8, repeats=2, warmup_steps=1)
    res = B.run_benchmark(B.MockEngine(CFG, H100, jitter=0.0, seed=1), cfgb, CFG, H100)
    for rid in ("a1", "c3"):
        B.write_run(B.RunRecord(rid, cfgb, {"gpu": "H100-SXM-80GB", "n_gpus": 8}, res), str(tmp_path))
    folder = tmp_path / "rt"
    (folder / "b2.json").write_text('{"runid": "b2", "config": {"name"')       # a write that was cut short
    (folder / "b4.json").write_text('[1, 2, 3]')                               # not a run record at all
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        runs = B.load_all("rt", str(tmp_path))
    assert [r.runid for r in runs] == ["a1", "c3"] and len(seen) == 2
    assert B.load_latest("rt", str(tmp_path)).runid == "c3"
