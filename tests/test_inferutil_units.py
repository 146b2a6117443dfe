"""Granular unit tests of the analytical model and the bench harness (pure CPU), one behaviour per test, in the
spirit of the reference's tests/ directory (tests/test_model.py, test_bench_engine.py, test_stats.py, test_store.py,
test_gate.py, test_sweep.py, test_prefill.py, test_efficiency.py, test_cost.py, test_manifest.py)."""
import dataclasses
import json
import math

import pytest

from inferutil.bench import config as C
from inferutil.bench import cost, efficiency as E, gate, prefill as P, stats as S, sweep as W
from inferutil.bench.attribution import dominant_of_breakdown, lever_hint
from inferutil.hardware import B200_SXM, GPUS, H100_SXM, Cluster
from inferutil.latency import decode_latency, expected_max_experts_per_gpu
from inferutil.model import QWEN3_235B


def _cfg(**kw):
    base = dict(name="t", plan="tp", dtype_bytes=1, kv_dtype_bytes=2, tp=8, ep=1)
    base.update(kw)
    return C.BenchConfig(**base)


# ---- stats --------------------------------------------------------------------------------------------------------
def test_t95_table_edges():
    assert S.t95(0) == float("inf") and S.t95(1) == pytest.approx(12.706) and S.t95(30) == pytest.approx(2.042)
    assert S.t95(31) == pytest.approx(1.96) and S.t95(1000) == pytest.approx(1.96)


def test_percentile_interpolates_and_handles_empty():
    assert S.percentile([], 0.5) is None
    assert S.percentile([3.0], 0.95) == 3.0
    assert S.percentile([1.0, 2.0, 3.0, 4.0], 0.5) == pytest.approx(2.5)
    assert S.percentile([1.0, 2.0, 3.0, 4.0], 1.0) == 4.0 and S.percentile([1.0, 2.0], 0.0) == 1.0


def test_summarize_mean_std_ci_and_roundtrip():
    s = S.summarize([10.0, 12.0, 14.0])
    assert s.n == 3 and s.mean == pytest.approx(12.0) and s.std == pytest.approx(2.0)
    assert s.ci95_half_width == pytest.approx(S.t95(2) * 2.0 / math.sqrt(3))
    assert S.stat_from_dict(S.stat_to_dict(s)) == s and S.stat_from_dict(None) is None
    one = S.summarize([5.0])
    assert one.n == 1 and one.mean == 5.0 and one.ci95_half_width is None
    assert S.summarize([]).n == 0


def test_means_differ_needs_disjoint_intervals():
    a, b = S.summarize([10.0, 10.1, 9.9, 10.0]), S.summarize([12.0, 12.1, 11.9, 12.0])
    assert S.means_differ(a, b) and not S.means_differ(a, S.summarize([10.05, 9.95, 10.1, 9.9]))
    assert not S.means_differ(S.summarize([1.0]), b)               # no interval from one sample


# ---- config -------------------------------------------------------------------------------------------------------
def test_config_id_depends_on_every_field_and_is_stable():
    a = _cfg()
    assert C.config_id(a) == C.config_id(_cfg()) and len(C.config_id(a)) == 12
    for change in (dict(plan="ep"), dict(dtype_bytes=2), dict(tp=4), dict(prompt_tokens=513), dict(seed=1), dict(repeats=6)):
        assert C.config_id(_cfg(**change)) != C.config_id(a), change
    assert a.seq_len == 512 + 128
    with pytest.raises(dataclasses.FrozenInstanceError):
        a.tp = 2


# ---- efficiency ---------------------------------------------------------------------------------------------------------
def test_flops_mfu_mbu_and_none_propagation():
    assert E.flops_per_token(10) == 20.0
    assert E.flops_per_token(10, seq_len=4, n_layers=2, d_model=8, include_attention=True) == 20.0 + 2 * 2 * 4 * 8
    assert E.mfu(100.0, 10, 4000.0) == pytest.approx(0.5) and E.mfu(None, 10, 1.0) is None and E.mfu(1.0, 10, 0.0) is None
    assert E.mbu(100.0, 5.0, 1000.0) == pytest.approx(0.5) and E.mbu(100.0, None, 1.0) is None
    assert E.achieved_tflops(1e6, 10 ** 6) == pytest.approx(2.0)


def test_roofline_regime():
    ridge = E.roofline_ridge(B200_SXM.fp8_flops, B200_SXM.hbm_bw)
    ai = E.arithmetic_intensity_decode(QWEN3_235B.active_params, QWEN3_235B.active_params * 1.0)
    assert ai == pytest.approx(2.0) and E.classify_regime(ai, ridge) == "memory-bound"
    big = E.arithmetic_intensity_prefill(QWEN3_235B.active_params, QWEN3_235B.active_params * 1.0, 4096)
    assert E.classify_regime(big, ridge) == "compute-bound" and E.classify_regime(None, ridge) == "unknown"
    assert E.peak_flops_for_dtype(1.0, 2.0, 2) == 1.0 and E.peak_flops_for_dtype(1.0, 2.0, 1) == 2.0


# ---- cost ---------------------------------------------------------------------------------------------------------------
def test_energy_and_rental_cost():
    m = cost.energy_metrics(200.0, 8000.0, usd_per_kwh=0.10)
    assert m["joules_per_token"] == pytest.approx(40.0) and m["tok_s_per_watt"] == pytest.approx(0.025)
    assert m["kwh_per_mtok"] == pytest.approx(40.0 * 1e6 / 3.6e6) and m["usd_per_mtok_energy"] == pytest.approx(m["kwh_per_mtok"] * 0.10)
    assert all(v is None for v in cost.energy_metrics(None, 100.0).values())
    assert cost.rental_usd_per_mtok(100.0, 8, usd_per_gpu_hr=3.0) == pytest.approx(1e6 * (24.0 / 3600.0) / 100.0)
    assert cost.rental_usd_per_mtok(0.0, 8) is None


# ---- prefill model --------------------------------------------------------------------------------------------------------
def test_distinct_experts_limits():
    assert P.expected_distinct_experts(128, 8, 1) == pytest.approx(8.0)
    assert P.expected_distinct_experts(128, 8, 10 ** 5) == pytest.approx(128.0)
    assert P.expected_distinct_experts(128, 8, 0) == 0.0 and P.expected_distinct_experts(0, 8, 5) == 0.0
    vals = [P.expected_distinct_experts(128, 8, p) for p in (1, 2, 4, 8, 16)]
    assert vals == sorted(vals)


def test_prefill_bytes_between_active_and_total_and_latency_regimes():
    lo = P.prefill_weight_bytes(QWEN3_235B, 1, 1)
    hi = P.prefill_weight_bytes(QWEN3_235B, 1, 10 ** 6)
    # one token touches top-k experts per layer: the active parameters plus the embedding table (counted as resident)
    assert QWEN3_235B.active_params <= lo <= QWEN3_235B.active_params + QWEN3_235B.vocab * QWEN3_235B.hidden * 1.01
    assert hi == pytest.approx(QWEN3_235B.total_params, rel=1e-6)
    cl = Cluster(B200_SXM, 8)
    assert P.prefill_latency(QWEN3_235B, cl, dtype_bytes=1, kv_dtype_bytes=2, prompt_tokens=0) == 0.0
    short = P.prefill_latency(QWEN3_235B, cl, dtype_bytes=1, kv_dtype_bytes=2, prompt_tokens=16)
    long = P.prefill_latency(QWEN3_235B, cl, dtype_bytes=1, kv_dtype_bytes=2, prompt_tokens=32768)
    assert short < long
    # a long prompt is compute bound: doubling it roughly doubles the time
    longer = P.prefill_latency(QWEN3_235B, cl, dtype_bytes=1, kv_dtype_bytes=2, prompt_tokens=65536)
    assert longer / long == pytest.approx(2.0, rel=0.05)


# ---- sweeps -----------------------------------------------------------------------------------------------------------------
def test_grids_enumerate_variants_with_distinct_ids():
    base = _cfg()
    q = W.quant_grid(base)
    assert len(q) == 6 and {c.dtype_bytes for c in q} == {2, 1, 0.5} and {c.kv_dtype_bytes for c in q} == {2, 1}
    lay = W.layout_grid(base, 8)
    assert len(lay) == 16 and {(c.tp, c.ep) for c in lay} == {(t, e) for t in (1, 2, 4, 8) for e in (1, 2, 4, 8)}
    full = W.full_grid(base, 4)
    assert len(full) == 3 * 2 * 3 * 3 and len({c.name for c in full}) == len(full)
    assert len({C.config_id(c) for c in full}) == len(full)


def test_depth_sweep_slows_with_context_and_efficiency_scales():
    cl = Cluster(B200_SXM, 8)
    pts = W.depth_sweep(QWEN3_235B, cl, _cfg(), [1024, 8192, 32768])
    tok = [p.decode_tok_s for p in pts]
    assert tok == sorted(tok, reverse=True) and [p.seq_len for p in pts] == [1024, 8192, 32768]
    assert pts[-1].kv_byte_share > pts[0].kv_byte_share
    ratio, floor = W.realized_efficiency(QWEN3_235B, cl, _cfg(), measured_tok_s=100.0)
    assert ratio == pytest.approx(100.0 / floor) and floor > 100.0


# ---- latency model ----------------------------------------------------------------------------------------------------------------
def test_balls_in_bins_and_plan_ordering():
    assert expected_max_experts_per_gpu(8, 1) == 8.0
    m = expected_max_experts_per_gpu(8, 8)
    assert 2.3 < m < 2.8                                            # the EP busiest-rank figure
    cl = Cluster(H100_SXM, 8)
    floor = decode_latency(QWEN3_235B, cl, plan="floor", dtype_bytes=1, seq_len=512)
    tp = decode_latency(QWEN3_235B, cl, plan="tp", dtype_bytes=1, seq_len=512)
    ep = decode_latency(QWEN3_235B, cl, plan="ep", dtype_bytes=1, seq_len=512)
    ideal = decode_latency(QWEN3_235B, cl, plan="ep", dtype_bytes=1, seq_len=512, ideal_routing=True)
    assert floor.total_s < tp.total_s < ep.total_s and ideal.weight_read_s < ep.weight_read_s
    assert tp.comms_s == pytest.approx(2 * 94 * 5e-6) and ep.comms_s == pytest.approx(3 * 94 * 5e-6)
    assert ep.imbalance == pytest.approx(m / 1.0) and ideal.imbalance == pytest.approx(1.0)
    with pytest.raises(ValueError):
        decode_latency(QWEN3_235B, cl, plan="pp")


def test_kv_shards_cap_at_kv_heads():
    cl = Cluster(B200_SXM, 8)
    a = decode_latency(QWEN3_235B, cl, plan="tp", dtype_bytes=1, seq_len=32768, tp=8)
    b = decode_latency(QWEN3_235B, cl, plan="hybrid", dtype_bytes=1, seq_len=32768, tp=4, ep=8)
    c = decode_latency(QWEN3_235B, cl, plan="hybrid", dtype_bytes=1, seq_len=32768, tp=2, ep=8)
    assert a.kv_read_s == pytest.approx(b.kv_read_s)                # min(tp, 4 kv heads) = 4 both
    assert c.kv_read_s == pytest.approx(2 * b.kv_read_s)


# ---- attribution ---------------------------------------------------------------------------------------------------------------------
def test_dominant_term_and_hint():
    assert dominant_of_breakdown(3.0, 1.0, 2.0, 0.1) in ("weight", "weight_bw")
    assert dominant_of_breakdown(0.1, 0.1, 2.0, 0.1) == "comms"
    assert isinstance(lever_hint("comms"), str) and lever_hint("comms")


def test_gpu_registry_and_cluster_aggregates():
    assert set(GPUS) >= {"H100-SXM-80GB", "H200-SXM-141GB", "B200-SXM-180GB"}
    cl = Cluster(B200_SXM, 8)
    assert cl.total_hbm == 8 * B200_SXM.hbm_bytes and cl.aggregate_hbm_bw == pytest.approx(8 * 7.7e12)
    assert H100_SXM.collective_latency_s == pytest.approx(5e-6)


# ---- gate ------------------------------------------------------------------------------------------------------------------------------
class _R:
    def __init__(self, tok=100.0, ttft=0.5, pct=0.4, quality=None, latency=None):
        self.decode_tok_per_s, self.ttft_s, self.pct_of_floor, self.quality, self.latency = tok, ttft, pct, quality, latency


class _Q:
    def __init__(self, m):
        self.match_rate = m


def test_threshold_gate_lists_every_failure():
    ok = gate.evaluate(_R(), gate.Thresholds(min_decode_tok_per_s=90.0, max_ttft_s=1.0, min_pct_of_floor=0.3))
    assert ok.passed and ok.failures == ()
    bad = gate.evaluate(_R(), gate.Thresholds(min_decode_tok_per_s=150.0, max_ttft_s=0.1, min_pct_of_floor=0.9))
    assert not bad.passed and len(bad.failures) == 3
    assert gate.evaluate(_R(), gate.Thresholds()).passed                      # no thresholds: nothing to fail


def test_quality_gate_needs_a_reference():
    t = gate.Thresholds(min_quality_match=0.95)
    assert not gate.evaluate(_R(quality=None), t).passed                      # not measured is a failure, not a pass
    assert gate.evaluate(_R(quality=_Q(0.99)), t).passed and not gate.evaluate(_R(quality=_Q(0.5)), t).passed


def test_regression_gate_uses_confidence_intervals_when_present():
    def lat(vals):
        return {"throughput_tok_s": S.stat_to_dict(S.summarize(vals))}
    base = _R(tok=100.0, latency=lat([100.0, 100.5, 99.5, 100.2]))
    same = _R(tok=99.8, latency=lat([99.8, 100.4, 99.3, 100.1]))
    worse = _R(tok=90.0, latency=lat([90.0, 90.4, 89.6, 90.1]))
    assert gate.regression_gate(base, same).passed                            # lower mean but overlapping intervals
    assert not gate.regression_gate(base, worse).passed
    assert gate.regression_gate(worse, base).passed                           # an improvement never fails
    # without intervals (single repeat) the point estimates decide
    assert not gate.regression_gate(_R(tok=100.0), _R(tok=99.0)).passed and gate.regression_gate(_R(tok=100.0), _R(tok=101.0)).passed


# ---- telemetry ---------------------------------------------------------------------------------------------------------------------------
def test_telemetry_summary_sums_power_over_gpus_and_reports_imbalance():
    from inferutil.bench.metrics import aggregate_breakdown, summarize_telemetry
    from inferutil.bench.telemetry import FakeTelemetrySource, GpuSample, NullTelemetry
    from inferutil.bench.engine import StepBreakdown
    samples = [GpuSample(0, 0.0, 60.0, 80.0, 40.0, 500.0, 1900.0, 3900.0, 10 ** 9),
               GpuSample(0, 0.1, 62.0, 90.0, 50.0, 520.0, 1900.0, 3900.0, 10 ** 9),
               GpuSample(1, 0.0, 70.0, 40.0, 20.0, 300.0, 1900.0, 3900.0, 10 ** 9)]
    src = FakeTelemetrySource(samples)
    src.start()
    t = summarize_telemetry(src.stop(), n_decode_tokens=100, decode_window_s=2.0)
    assert t.available and t.n_gpus == 2 and t.temp_c_max == 70.0
    assert t.power_w_mean == pytest.approx(510.0 + 300.0)                      # per-GPU means, then summed
    assert t.energy_j_per_token == pytest.approx(810.0 * 2.0 / 100)
    assert t.per_gpu_mean_util == (85.0, 40.0) and t.util_imbalance == pytest.approx(85.0 / 62.5)
    assert NullTelemetry().stop() == [] and not summarize_telemetry([], 10, 1.0).available
    b = aggregate_breakdown([StepBreakdown(1.0, 2.0, 3.0, 4.0), None, StepBreakdown(3.0, 2.0, 1.0, 0.0)])
    assert (b.weight_s, b.kv_s, b.comms_s, b.compute_s) == (2.0, 2.0, 2.0, 2.0) and aggregate_breakdown([None]) is None


# ---- mock engine ---------------------------------------------------------------------------------------------------------------------------
def test_mock_engine_is_seeded_and_scales_with_efficiency():
    from inferutil.bench.engine import Engine, MockEngine
    cl = Cluster(H100_SXM, 8)
    kw = dict(plan="tp", dtype_bytes=1, kv_dtype_bytes=2, tp=8, ep=1, seq_len=640)
    a, b = MockEngine(QWEN3_235B, cl, jitter=0.1, seed=3), MockEngine(QWEN3_235B, cl, jitter=0.1, seed=3)
    a.reset(**kw); b.reset(**kw)
    assert [a.decode_step().seconds for _ in range(5)] == [b.decode_step().seconds for _ in range(5)]
    half = MockEngine(QWEN3_235B, cl, efficiency=0.5)
    full = MockEngine(QWEN3_235B, cl)
    half.reset(**kw); full.reset(**kw)
    assert half.decode_step().seconds == pytest.approx(2 * full.decode_step().seconds)
    assert isinstance(full, Engine)                                            # runtime-checkable protocol
    routed = MockEngine(QWEN3_235B, cl, expose_routes=True)
    routed.reset(**kw)
    step = routed.decode_step()
    assert len(step.routes) == QWEN3_235B.top_k and all(0 <= r.gpu < 8 for r in step.routes)
    bd = step.breakdown
    assert bd.weight_s + bd.kv_s + bd.comms_s + bd.compute_s == pytest.approx(step.seconds)


def test_manifest_names_commit_model_and_host():
    from inferutil.bench.manifest import build_manifest, model_hash
    m = build_manifest(QWEN3_235B, Cluster(B200_SXM, 8), _cfg())
    text = json.dumps(m)
    assert model_hash(QWEN3_235B) in text and len(model_hash(QWEN3_235B)) >= 8
    assert model_hash(QWEN3_235B) != model_hash(dataclasses.replace(QWEN3_235B, n_layers=93))
    assert {"schema", "runid", "host", "code", "model", "hardware", "bench"} <= set(m)
    assert "commit" in json.dumps(m["code"]) and m["hardware"] and m["bench"]
