"""Experiments on the engine's own model (CPU) and the closed-form studies."""
import json
import math

import pytest
import torch

from inferencehackathon_b200.experiments import adaptive_topk, html_report, quality, route_study, self_spec, stale_tp
from inferencehackathon_b200.experiments.stale_tp import EXACT, LOCAL, REAL, REAL_FALLBACK, STALE, StaleConfig, StaleScheduler
from inferencehackathon_b200.runtime.engine import InferenceEngine
from inferutil import studies


def _engine(model="tiny"):
    return InferenceEngine.build(model, device="cpu", backend="torch", max_seq=96)


def _prompts(eng, n=3, length=10):
    g = torch.Generator().manual_seed(1)
    return [torch.randint(0, eng.cfg.model.vocab, (length,), generator=g).tolist() for _ in range(n)]


# ---- stale tensor parallelism ---------------------------------------------------------------------------------------
def test_scheduler_layer_mode_refreshes_every_kth_layer():
    s = StaleScheduler(StaleConfig(K=2, mode="layer", period=8, collectives_per_layer=2))
    actions = []
    for _ in range(8):
        a, idx, cached = s.decide(1)
        actions.append(a)
        s.record(a, idx, object() if a in (REAL, REAL_FALLBACK) else None)
    # layers 0 and 2 are real (both slots), layers 1 and 3 reuse the cached value of their slot
    assert actions == [REAL, REAL, STALE, STALE, REAL, REAL, STALE, STALE]
    assert s._step == 1 and s._call == 0 and not s._by_slot          # wrapped: within-token caches are dropped


def test_scheduler_temporal_mode_and_policies():
    s = StaleScheduler(StaleConfig(K=3, mode="temporal", period=4))
    per_step = []
    for step in range(4):
        acts = []
        for _ in range(4):
            a, idx, c = s.decide(1)
            acts.append(a)
            s.record(a, idx, ("v", step, idx) if a in (REAL, REAL_FALLBACK) else None)
        per_step.append(set(acts))
    assert per_step == [{REAL}, {STALE}, {STALE}, {REAL}]
    loc = StaleScheduler(StaleConfig(K=2, mode="layer", policy="local", period=4))
    seq = []
    for _ in range(4):
        a, idx, _ = loc.decide(1)
        seq.append(a)
        loc.record(a, idx)
    assert seq == [REAL, REAL, LOCAL, LOCAL]
    ex = StaleScheduler(StaleConfig(K=1))
    assert ex.decide(1)[0] == EXACT
    pre = StaleScheduler(StaleConfig(K=2, decode_only=True))
    assert pre.decide(7)[0] == EXACT                                  # multi-token passes stay exact


def test_stale_probe_is_exact_at_k1_and_degrades_gracefully():
    eng = _engine()
    rows = stale_tp.probe(eng, _prompts(eng), new_tokens=8, Ks=(1, 2), modes=("layer",))
    by_k = {r["K"]: r for r in rows}
    assert by_k[1]["exact_match_rate"] == 1.0 and by_k[1]["stale_fraction"] == 0.0
    assert 0.0 < by_k[2]["stale_fraction"] <= 0.5
    assert 0.0 <= by_k[2]["mean_prefix_agreement"] <= 1.0
    assert not isinstance(eng.model.comm, stale_tp.StaleCollectives)   # uninstalled


# ---- adaptive top-k ------------------------------------------------------------------------------------------------------
def test_adaptive_route_keeps_the_smallest_prefix_reaching_the_mass():
    torch.manual_seed(0)
    h = torch.randn(5, 16)
    rw = torch.randn(12, 16)
    idx, w, logits, kept = adaptive_topk.adaptive_route(h, rw, 4, True, 0.9, 2)
    p = torch.softmax(logits, -1)
    tw, ti = torch.topk(p, 4, -1)
    assert torch.equal(idx, ti)
    for t in range(5):
        share = torch.cumsum(tw[t], 0) / tw[t].sum()
        want = max(2, int((share < 0.9).sum()) + 1)
        assert int(kept[t]) == min(4, want)
        assert torch.all(w[t, int(kept[t]):] == 0)
        assert abs(float(w[t].sum()) - 1.0) < 1e-6
    # mass 1.0 keeps everything: identical to the plain router
    idx2, w2, _, kept2 = adaptive_topk.adaptive_route(h, rw, 4, True, 1.01, 1)
    assert torch.all(kept2 == 4) and torch.allclose(w2, tw / tw.sum(-1, keepdim=True))


def test_adaptive_gate_and_router_mass_on_the_model():
    eng = _engine()
    prompts = _prompts(eng)
    gate = adaptive_topk.quality_gate(eng, prompts, new_tokens=6, mass=2.0, k_min=1)     # unreachable mass: exact
    assert gate["exact_match_rate"] == 1.0 and gate["expert_byte_saving"] == 0.0
    gate = adaptive_topk.quality_gate(eng, prompts, new_tokens=6, mass=0.5, k_min=1)
    assert 0.0 < gate["expert_byte_saving"] < 1.0 and gate["mean_k"] < eng.cfg.model.top_k
    assert eng.model.route_fn is None
    rm = adaptive_topk.router_mass(eng.model, prompts, ks=(1, 2), thresholds=(0.5, 0.9))
    assert rm["positions_x_layers"] == 3 * 10 * eng.cfg.model.n_layers
    assert 1.0 <= rm["expected_k"]["0.5"] <= rm["expected_k"]["0.9"] <= eng.cfg.model.top_k


# ---- route study, self speculation, quality, report ---------------------------------------------------------------------------------
def test_route_study_numbers_are_consistent():
    eng = _engine()
    m = eng.cfg.model
    routes, hid = route_study.collect_routes(eng, _prompts(eng, 2), new_tokens=6)
    assert len(routes) == 12 and all(len(t) == m.n_layers and all(len(e) == m.top_k for e in t) for t in routes)
    rep = route_study.analyze(routes, hid, [lw.router for lw in eng.weights.layers], m.n_experts, m.top_k, n_gpus=2,
                              hot_k=m.n_experts, replicate=1)
    assert rep["static_hot"] == pytest.approx(1.0)                     # every expert is "hot" when hot_k = all
    assert rep["combined"] >= rep["persistence"]
    assert 0.0 <= rep["direct_proxy"] <= 1.0 and 0.0 <= rep["layer_to_layer"] <= 1.0
    assert rep["imbalance"]["round_robin"] >= 1.0
    assert rep["coverage"][4] <= rep["coverage"].get(8, 1.0) <= 1.0
    pl = route_study.placement_report(routes, m.n_experts, n_gpus=2)
    assert set(pl) == {"round_robin", "affinity"}
    assert eng.model.route_fn is None


def test_self_speculation_curve():
    eng = _engine("small")
    rows = self_spec.agreement_curve(eng.model, _prompts(eng, 2, 8))
    assert rows and all(0.0 <= r["top1_agreement"] <= r["in_top4"] <= 1.0 for r in rows)
    assert [r["depth"] for r in rows] == sorted(r["depth"] for r in rows)
    assert all(r["draft_cost_steps"] == pytest.approx(2 * r["depth"] / eng.cfg.model.n_layers) for r in rows)


def test_quality_compare_and_fp8_validation():
    assert quality.prefix_agreement([1, 2, 3, 4], [1, 2, 9, 4]) == 0.5
    c = quality.compare_ids([[1, 2, 3], [4, 5]], [[1, 2, 3], [4, 6]])
    assert c["exact_match_rate"] == 0.5 and c["mean_prefix_agreement"] == pytest.approx(0.75)
    base = {"outputs": [{"prompt": "p", "text": "a b c d"}]}
    cand = {"outputs": [{"prompt": "p", "text": "a b c x"}]}
    r = quality.compare(base, cand, min_agreement=0.7)
    assert r["mean_agreement"] == 0.75 and r["passed"] and r["exact_match_rate"] == 0.0
    rows = quality.validate_fp8(hidden=256, inter=128, vocab=512)
    assert len(rows) == 5 and all(r["ok"] and r["cosine"] > 0.995 for r in rows)


def test_html_report(tmp_path):
    lines = [{"metric": "decode_tok_per_s", "value": 100.0 + i, "ms_per_step": 1000.0 / (100.0 + i), "n_gpus": 8,
              "config": {"prompt": 512 * (i + 1)}, "ttft_ms": 500.0, "e2e": {"value": 99.0},
              "phase_us": {"qkv": 8.0, "attention": 12.0}} for i in range(3)]
    src = tmp_path / "lines.jsonl"
    src.write_text("noise\n" + "\n".join(json.dumps(l) for l in lines))
    out = tmp_path / "report.html"
    assert html_report.main([str(src), str(out)]) == 0
    page = out.read_text()
    assert page.count("<svg") == 2 and "attention" in page and "1536" in page and "<table>" in page


# ---- closed-form studies -------------------------------------------------------------------------------------------------------------
def test_backout_floor_recovers_the_floor_share():
    F = 0.8
    meas = []
    for k, tau in ((2, 1.7), (5, 2.8), (8, 3.3)):
        v = studies.floor_verify_cost(F, studies.expert_union(k))
        meas.append((k, tau, tau / v))
    r = studies.backout_floor(meas)
    assert r["F"] == pytest.approx(F, abs=1e-9)
    assert all(f == pytest.approx(F, abs=1e-9) for f in r["pairwise_F"])
    assert r["verdict"]["route_aware_pays"] in (True, False)


def test_union_reconcile_ladder_and_tree():
    assert studies.expert_union(1) == pytest.approx(8.0)
    assert studies.expert_union(1000) == pytest.approx(128.0, abs=1e-6)
    assert studies.expert_union(8, overlap=0.5) == pytest.approx(studies.expert_union(4))
    rows = studies.comms_reconcile(11.67, 188, 1.56, 0.19, [5, 16, 35, 60])
    assert [r["consistent"] for r in rows] == [True, True, False, False]
    lad = studies.ladder()
    assert lad[0]["tok_s"] == pytest.approx(1000.0 / 3.74) and all(b["tok_s"] > a["tok_s"] for a, b in zip(lad, lad[1:]))
    hi = studies.tree_optimizer(0.9, 0.7)[0]
    lo = studies.tree_optimizer(0.0, 0.7)[0]
    assert hi["positions"] > lo["positions"]                       # a floor-bound step favours large trees
    assert studies.spec_predict(0.5, 0.7, 2, 4, layout="ep")["verify_cost"] <= studies.spec_predict(0.5, 0.7, 2, 4)["verify_cost"]
    assert studies.spec_predict(0.5, 0.7, 2, 4, draft_ms_per_step=0.6)["speedup"] < studies.spec_predict(0.5, 0.7, 2, 4)["speedup"]


def test_layout_studies_and_monte_carlo():
    rows = studies.tp_degree()
    assert [r["gpus"] for r in rows] == [1, 2, 4, 8] and rows[0]["fits"] is False and rows[-1]["fits"] is True
    assert rows[-1]["tok_s"] > rows[1]["tok_s"]
    st = studies.stale_tp_ceiling()
    assert st["speedup"] > 1.0
    vc = studies.verify_cost_check()
    assert vc[0]["ratio"] == pytest.approx(1.0) and vc[-1]["ratio"] > 1.3
    m = studies.mbu_ceiling(0.42, {"router": 6.0, "attention": 12.0}, kernel_mbu=0.6)
    assert m["fused_ms"] < m["unfused_ms"] and m["whole_engine_mbu_unfused"] < 0.6
    mc = studies.validate_routing_model(trials=400)
    for r in mc["union"]:
        assert r["simulated"] == pytest.approx(r["formula"], rel=0.05)
    assert mc["busiest_rank"]["simulated"] == pytest.approx(mc["busiest_rank"]["formula"], rel=0.1)
    assert mc["verify_imbalance"][-1]["busiest_over_mean"] < mc["verify_imbalance"][0]["busiest_over_mean"]
    b = studies.latency_budget(turns=2, prefix_cache=False, plan="tp", tp=8, ep=1, dtype_bytes=1, collective_us=10.0,
                               efficiency=0.5, host_ms=0.0)
    assert b["turns"][1]["ttft_ms"] > b["turns"][0]["ttft_ms"]
    a = studies.spec_analyze(100, 180, 300, 200, 5, floor_hint=0.8)
    assert a["tau"] == 2.5 and a["V"] == pytest.approx(2.5 / 1.8) and a["implied_union"] > 8
    assert len(studies.predict_matrix()) == 2 * 3 * 4 and studies.main(["verify-cost"]) == 0


def test_window_group_table_covers_every_pair_once():
    """Host-free bookkeeping of the grouped expert GEMM (pure tensor ops, so it can be checked on the CPU)."""
    from inferencehackathon_b200.runtime.gpu_window import GpuWindow
    g = torch.Generator().manual_seed(4)
    for n_experts, pairs, nt in ((16, 96, 16), (8, 40, 32), (128, 1024, 64), (4, 3, 16)):
        flat_e = torch.randint(0, n_experts, (pairs,), generator=g)
        order, groups, n_groups, gmax = GpuWindow._group_table(flat_e, n_experts, nt)
        ng = int(n_groups[0])
        assert ng <= gmax and groups.shape == (gmax, 4)
        covered = torch.zeros(pairs, dtype=torch.int32)
        sorted_e = flat_e[order]
        for e, tok0, ntok, _ in groups[:ng].tolist():
            assert 0 < ntok <= nt
            assert torch.all(sorted_e[tok0: tok0 + ntok] == e)       # a group holds rows of ONE expert
            covered[tok0: tok0 + ntok] += 1
        assert torch.all(covered == 1)                                # every (token, slot) pair exactly once
        assert torch.all(groups[ng:, 2] == 0)                         # unused entries are empty
        assert torch.equal(torch.sort(order).values, torch.arange(pairs))


def test_scaling_fit_separates_the_byte_part_from_the_fixed_part():
    # exact data from t = 1.5 * x + 3.0 is recovered
    bw, by = 6.5616e12, 21.7e9
    pts = [(n, 1.5 * by / n / bw * 1e3 + 3.0) for n in (1, 2, 4, 8)]
    r = studies.scaling_fit(pts, by, bw)
    assert r["bandwidth_efficiency"] == pytest.approx(1 / 1.5) and r["fixed_ms"] == pytest.approx(3.0)
    assert r["max_fit_error_ms"] < 1e-9 and r["fixed_us_per_layer"] == pytest.approx(3000.0 / 94)
    # the measured points: the part that GPUs do not shrink is most of the token at 8 GPUs
    m = studies.scaling_fit()
    assert 2.5 < m["fixed_ms"] < 3.6 and m["rows"][-1]["fixed_share"] > 0.75 and m["max_fit_error_ms"] < 0.7
    assert m["rows"][-1]["tok_s_if_fixed_halves"] > 1.5 * m["rows"][-1]["tok_s"]
    assert studies.main(["scaling-fit"]) == 0 and studies.main(["scaling-fit", "1:8.0", "2:5.0", "4:3.5"]) == 0


from hypothesis import given, settings, strategies as st   # noqa: E402


@settings(max_examples=80, deadline=None)
@given(st.integers(1, 300), st.sampled_from([1, 4, 16, 128]), st.sampled_from([16, 32, 64]), st.integers(0, 2 ** 31 - 1))
def test_expert_group_table_oracle_tiles_every_pair_exactly_once(pairs, n_experts, nt, seed):
    """The oracle of the device group-table kernel, for any routing: the groups are contiguous runs of the pairs sorted by
    expert, each within one expert and at most ``nt`` rows long, together they cover every pair once, the entries past
    ``n_groups`` are empty, and the shape-only bound G is never exceeded."""
    import torch
    from inferencehackathon_b200.runtime.gpu_window import GpuWindow
    g = torch.Generator().manual_seed(seed)
    skew = torch.rand(n_experts, generator=g) ** 3 + 1e-3                  # a few hot experts, many cold ones
    flat_e = torch.multinomial(skew, pairs, replacement=True, generator=g)
    order, groups, n_groups, gmax = GpuWindow._group_table(flat_e, n_experts, nt)
    n = int(n_groups[0])
    assert groups.shape == (gmax, 4) and n <= gmax
    sorted_e = flat_e[order]
    assert torch.equal(sorted_e, torch.sort(flat_e).values) and sorted(order.tolist()) == list(range(pairs))
    covered = 0
    for e, first, rows, _ in groups[:n].tolist():
        assert 1 <= rows <= nt and first == covered                         # consecutive, no gap, no overlap
        assert bool((sorted_e[first:first + rows] == e).all())
        covered += rows
    assert covered == pairs
    assert int(groups[n:, 2].sum()) == 0
