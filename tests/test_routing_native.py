"""Expert-routing control plane (C++): placement optimiser, predictors, prefetch scheduler, accuracy / traces.

Invariants follow the reference's routing test modules (engine/src/routing/{optimizer,predictor,scheduler,stats}.rs).
"""
import json
import subprocess
import sys

import numpy as np
import pytest

from inferencehackathon_b200.routing import native as rt


def test_placement_separates_hot_experts_and_beats_round_robin():
    counts = np.ones((2, 16), np.uint32) * 10
    counts[0, 0] = counts[0, 8] = 500          # round-robin would put both on GPU 0 (8 GPUs)
    pm, doc = rt.optimize_placement(counts, 8)
    assert pm.gpu_for(0, 0) != pm.gpu_for(0, 8)
    st = doc["stats"]
    assert st["optimized_mean_imbalance"] < st["round_robin_mean_imbalance"]
    assert st["n_layers"] == 2 and st["n_experts"] == 16 and st["n_gpus"] == 8
    assert pm.is_replicated(0, 0) and pm.is_replicated(0, 8) and not pm.is_replicated(1, 3)
    prim, rep = pm.gpus_for(0, 0)
    assert rep is not None and rep != prim
    assert st["total_replicated_expert_layers"] == pm.n_replicated_experts() == 2
    assert set(doc) == {"placement", "replicas", "stats"} and doc["placement"]["1"]["3"] == pm.gpu_for(1, 3)
    assert "1" not in doc["replicas"]


def test_placement_uniform_counts_is_balanced_and_json_roundtrip():
    pm, doc = rt.optimize_placement(np.full((3, 128), 7, np.uint32), 8)
    assert doc["stats"]["optimized_mean_imbalance"] == pytest.approx(1.0)
    assert pm.n_replicated_experts() == 0
    for l in range(3):
        assert np.bincount(pm.primary[l], minlength=8).tolist() == [16] * 8
    back = rt.PlacementMap.from_json(json.loads(json.dumps(doc)))
    assert np.array_equal(back.primary, pm.primary) and np.array_equal(back.replica, pm.replica) and back.n_gpus == 8


def test_placement_zero_counts():
    pm, doc = rt.optimize_placement(np.zeros((1, 8), np.uint32), 4)
    assert doc["stats"]["optimized_mean_imbalance"] == 1.0 and pm.n_replicated_experts() == 0


def test_placement_cli(tmp_path):
    src = tmp_path / "routing_stats.json"
    rng = np.random.default_rng(0)
    src.write_text(json.dumps({"routing": {"activation_counts": rng.integers(0, 1000, (4, 32)).tolist()}}))
    dst = tmp_path / "optimized_placement.json"
    r = subprocess.run([sys.executable, "-m", "inferencehackathon_b200.routing.optimize_placement", str(src), str(dst),
                        "--n-gpus", "8"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    doc = json.loads(dst.read_text())
    assert len(doc["placement"]) == 4 and len(doc["placement"]["0"]) == 32
    assert "imbalance" in r.stdout


def test_round_robin_and_contiguous_maps():
    pm = rt.PlacementMap.round_robin(2, 4, 16)
    assert pm.gpu_for(1, 5) == 1 and pm.gpus_for(0, 7) == (3, None)
    pm.set(0, 7, 0)
    pm.set_replica(0, 7, 2)
    assert pm.gpus_for(0, 7) == (0, 2) and pm.n_replicated_experts() == 1
    cg = rt.PlacementMap.contiguous(1, 8, 128)
    assert cg.gpu_for(0, 0) == 0 and cg.gpu_for(0, 16) == 1 and cg.gpu_for(0, 127) == 7


def _proxy(n_layers=4, hidden=16, n_experts=8):
    p = rt.RoutePredictor(n_layers, hidden, n_experts)
    for l in range(n_layers):
        w = np.zeros((n_experts, hidden), np.float32)
        for e in range(n_experts):
            w[e, (e + l) % hidden] = 1.0
        p.set_router(l, w)
    return p


def test_direct_proxy_uses_next_layer_router():
    p = _proxy()
    h = np.zeros(16, np.float32)
    h[3] = 5.0                                  # layer 1 router: expert e looks at dim e + 1 -> expert 2
    h[6] = 2.0                                  # -> expert 5
    pred = p.predict(0, h, top_k=2)
    assert pred.layer == 1 and pred.experts == [2, 5] and pred.scores == [5.0, 2.0] and pred.source == "DirectProxy"
    assert p.predict(3, h).experts == []        # no layer after the last one


def test_learned_linear_starts_as_proxy_and_learns():
    p = _proxy()
    p.init_linear_from_proxy()
    rng = np.random.default_rng(0)
    h = rng.standard_normal(16).astype(np.float32)
    assert p.predict(0, h, top_k=3, kind=rt.LINEAR).experts == p.predict(0, h, top_k=3, kind=rt.PROXY).experts
    # teach layer 0 that expert 7 always fires
    hb = rng.standard_normal((32, 16)).astype(np.float32)
    tgt = np.zeros((32, 8), np.float32)
    tgt[:, 7] = 10.0 * np.abs(hb[:, 0])
    hb[:, 0] = np.abs(hb[:, 0])
    for _ in range(300):
        p.linear_update(0, hb, tgt, lr=0.05)
    probe = np.zeros(16, np.float32)
    probe[0] = 1.0
    assert p.predict(0, probe, top_k=1, kind=rt.LINEAR).experts == [7]


def test_markov_transition_learns_cooccurrence():
    p = rt.RoutePredictor(3, 4, 8)
    p.enable_markov()
    for _ in range(50):
        p.markov_observe(0, [1, 2], [5, 6])
    pred = p.predict(0, None, current_experts=[1], top_k=2, kind=rt.MARKOV)
    assert sorted(pred.experts) == [5, 6] and pred.layer == 1 and pred.source == "MarkovTransition"
    assert p.predict(2, None, current_experts=[1], kind=rt.MARKOV).experts == []


def test_ensemble_fuses_normalised_scores():
    p = _proxy()
    p.enable_markov()
    for _ in range(100):
        p.markov_observe(0, [0], [7])
    h = np.zeros(16, np.float32)
    h[3] = 1.0                                   # proxy says expert 2
    p.weights = [1.0, 0.0, 0.0]
    assert p.predict(0, h, [0], top_k=1, kind=rt.ENSEMBLE).experts == [2]
    p.weights = [0.0, 0.0, 1.0]
    assert p.predict(0, h, [0], top_k=1, kind=rt.ENSEMBLE).experts == [7]
    p.weights = [1.0, 0.0, 1.0]
    assert sorted(p.predict(0, h, [0], top_k=2, kind=rt.ENSEMBLE).experts) == [2, 7]


def test_prefetch_scheduler_actions_and_hit_rate():
    pm = rt.PlacementMap.round_robin(4, 4, 8)
    pm.set_replica(1, 5, 3)
    seen = []
    s = rt.PrefetchScheduler(pm, sink=seen.append)
    n = s.on_prediction(rt.ExpertPrediction(1, [5, 2], [1.0, 0.5], "DirectProxy"))
    assert n == 6 and len(seen) == 6
    kinds = [(a.kind, a.expert_id, a.gpu_id) for a in seen]
    assert kinds == [("WarmExpert", 5, 1), ("EarlyDispatch", 5, 1), ("WarmExpert", 5, 3), ("EarlyDispatch", 5, 3),
                     ("WarmExpert", 2, 2), ("EarlyDispatch", 2, 2)]
    assert [a.layer for a in seen] == [1] * 6
    s.on_layer_complete(0, [5, 2])               # not the pending layer: ignored
    assert s.total_hits() == 0
    s.on_layer_complete(1, [5, 7])
    assert s.total_hits() == 1 and s.total_prefetched() == 2 and s.hit_rate() == pytest.approx(0.5)
    assert len(s.drain()) == 6 and s.drain() == []


def test_prefetch_scheduler_null_sink():
    s = rt.PrefetchScheduler(rt.PlacementMap.round_robin(2, 2, 4), record=False)
    s.on_prediction(rt.ExpertPrediction(1, [0, 1], [1, 1], "Ensemble"))
    assert s.drain() == [] and s.hit_rate() == 0.0


def test_accuracy_tracker():
    t = rt.AccuracyTracker(4, 8)
    t.record(rt.ExpertPrediction(1, list(range(8)), [1.0] * 8, "DirectProxy"), 1, list(range(8)))
    assert t.hit_rate(1) == pytest.approx(1.0) and t.expected_hits(1) == pytest.approx(8.0)
    t.record(rt.ExpertPrediction(2, [0, 1, 2, 3, 4, 5, 6, 7], [1.0] * 8, "DirectProxy"), 2, [0, 1, 2, 3, 20, 21, 22, 23])
    assert t.hit_rate(2) == pytest.approx(0.5)
    assert t.mean_hit_rate() == pytest.approx(0.75)
    s = t.layer_summaries()
    assert s[1].n_tokens == 1 and s[0].n_tokens == 0 and s[2].expected_hits == pytest.approx(4.0)
    t.record(rt.ExpertPrediction(9, [0], [1.0], "DirectProxy"), 9, [0])        # out of range: ignored
    t.reset()
    assert t.mean_hit_rate() == 0.0


def test_trace_collector_bounded_and_drain():
    tc = rt.TraceCollector(4, 3, max_traces=5)
    for i in range(7):
        ok = tc.push(i % 2, np.full(4, i, np.float32), np.full(3, 10 + i, np.float32))
        assert ok == (i < 5)
    assert tc.n_traces() == 5 and tc.is_full()
    h, l, n = tc.drain_layer(0)
    assert n == 3 and h[:, 0].tolist() == [0, 2, 4] and l[:, 0].tolist() == [10, 12, 14]
    assert tc.n_traces() == 2
    h, l, n = tc.drain_layer(1)
    assert n == 2 and h[:, 0].tolist() == [1, 3]
    tc.push(3, np.zeros(4), np.zeros(3))
    tc.clear()
    assert tc.n_traces() == 0


def test_live_pipeline_scores_predictions_against_real_routing():
    """Routing records in, Markov predictions + prefetch actions out: high hit rate on structured routing, the chance
    rate on random routing, actions for the GPUs that hold the predicted experts."""
    import random
    from inferencehackathon_b200.routing.pipeline import RoutingPipeline
    L, E, k = 6, 32, 4

    def run(structured, sink=None):
        rng = random.Random(0)
        p = RoutingPipeline(L, E, k, n_gpus=4, warmup_tokens=8, sink=sink)
        for _ in range(150):
            cur = rng.sample(range(E), k)
            tok = {}
            for layer in range(L):
                tok[layer] = cur
                cur = ([(e + 1) % E if rng.random() < 0.9 else rng.randrange(E) for e in cur] if structured
                       else rng.sample(range(E), k))
            p.on_token(tok)
        return p

    good, rand = run(True), run(False)
    gs, rs = good.stats(), rand.stats()
    assert gs["tokens"] == 150 and gs["records"] == 150 * L
    assert gs["prefetch_hit_rate"] > 0.6 and gs["mean_layer_hit_rate"] > 0.6
    assert rs["prefetch_hit_rate"] < 0.3                                   # chance is k / E = 0.125
    acts = good.scheduler.drain()
    assert acts and all(a.gpu_id == good.placement.gpu_for(a.layer, a.expert_id) for a in acts[:50])
    assert {a.kind for a in acts} == {"WarmExpert", "EarlyDispatch"}
    seen = []
    run(True, sink=seen.append)
    assert len(seen) > 100 and seen[0].layer >= 1                          # predictions are for the NEXT layer
    # nothing is predicted during warm-up or for the layer after the last one
    p = RoutingPipeline(L, E, k, warmup_tokens=2)
    assert p.on_layer(0, [1, 2, 3, 4]) is None
    for _ in range(3):
        for layer in range(L):
            out = p.on_layer(layer, [layer, layer + 1, layer + 2, layer + 3])
    assert out is None


from hypothesis import given, settings, strategies as st   # noqa: E402


@settings(max_examples=60, deadline=None)
@given(st.integers(1, 4), st.sampled_from([8, 16, 32]), st.sampled_from([2, 4, 8]), st.integers(0, 2 ** 31 - 1))
def test_placement_optimiser_invariants(n_layers, n_experts, n_gpus, seed):
    """For any activation counts: every expert has exactly one primary GPU in range, a replica (if any) sits on another
    GPU, the greedy placement never loads the busiest GPU more than round robin does (with replicas taking half of a
    hot expert's traffic), and the JSON document round-trips."""
    rng = np.random.default_rng(seed)
    counts = (rng.pareto(1.2, size=(n_layers, n_experts)) * 50).astype(np.uint32)
    pm, doc = rt.optimize_placement(counts, n_gpus)
    prim, rep = np.asarray(pm.primary).reshape(n_layers, n_experts), np.asarray(pm.replica).reshape(n_layers, n_experts)
    assert prim.min() >= 0 and prim.max() < n_gpus
    has = rep >= 0
    assert (rep[has] < n_gpus).all() and (rep[has] != prim[has]).all()
    for layer in range(n_layers):
        load = np.zeros(n_gpus)
        rr = np.zeros(n_gpus)
        for e in range(n_experts):
            c = float(counts[layer, e])
            if rep[layer, e] >= 0:
                load[prim[layer, e]] += c / 2
                load[rep[layer, e]] += c / 2
            else:
                load[prim[layer, e]] += c
            rr[e % n_gpus] += c
        assert load.max() <= rr.max() + 1e-6
        assert abs(load.sum() - rr.sum()) < 1e-6 * max(1.0, rr.sum())
    back = rt.PlacementMap.from_json(doc, n_gpus)
    assert np.array_equal(np.asarray(back.primary), np.asarray(pm.primary))
    assert np.array_equal(np.asarray(back.replica), np.asarray(pm.replica))
    assert doc["stats"]["optimized_mean_imbalance"] <= doc["stats"]["round_robin_mean_imbalance"] + 1e-9


@settings(max_examples=50, deadline=None)
@given(st.integers(2, 5), st.sampled_from([8, 16]), st.integers(1, 4), st.integers(0, 2 ** 31 - 1))
def test_scheduler_and_predictor_invariants_on_arbitrary_routing(n_layers, n_experts, k, seed):
    """Any routing stream, including out-of-range ids, repeated layers and layers out of order: counters stay consistent
    (hits <= prefetched, rates in [0, 1]), a Markov prediction names distinct experts in range (its Laplace prior lets
    it name experts it has not seen yet), once a transition dominates it is predicted, actions only name GPUs that hold
    the expert, and nothing reads or writes outside a table (this test also runs under ASan in ops/sanitize_ctrl.py)."""
    rng = np.random.default_rng(seed)
    pm = rt.PlacementMap.round_robin(n_layers, 4, n_experts)
    sched = rt.PrefetchScheduler(pm)
    pred = rt.RoutePredictor(n_layers, 1, n_experts)
    pred.enable_markov()
    acc = rt.AccuracyTracker(n_layers, k)
    seen_after = {}
    prev = None
    for _ in range(60):
        layer = int(rng.integers(-1, n_layers + 1))                          # sometimes out of range
        experts = [int(e) for e in rng.integers(-2, n_experts + 2, size=k)]    # sometimes out of range
        if prev is not None and prev[0] == layer - 1 and 0 <= prev[0] < n_layers - 1:
            pred.markov_observe(prev[0], prev[1], experts)
            for a in prev[1]:
                if 0 <= a < n_experts:
                    seen_after.setdefault((prev[0], a), set()).update(e for e in experts if 0 <= e < n_experts)
        sched.on_layer_complete(layer, experts)
        if 0 <= layer < n_layers - 1:
            p = pred.predict(layer, None, current_experts=experts, top_k=k, kind=rt.MARKOV)
            assert len(set(p.experts)) == len(p.experts) <= k and p.layer == layer + 1
            assert all(0 <= e < n_experts for e in p.experts)
            if p.experts:
                sched.on_prediction(p)
                acc.record(p, layer + 1, experts)
        prev = (layer, experts)
    assert 0 <= sched.total_hits() <= sched.total_prefetched()
    assert 0.0 <= sched.hit_rate() <= 1.0 and 0.0 <= acc.mean_hit_rate() <= 1.0
    for a in sched.drain():
        assert 0 <= a.layer < n_layers and a.gpu_id in [g for g in pm.gpus_for(a.layer, a.expert_id) if g is not None]
    # a transition observed many times wins over the prior
    for _ in range(40):
        pred.markov_observe(0, [1], [n_experts - 1])
    assert pred.predict(0, None, current_experts=[1], top_k=1, kind=rt.MARKOV).experts == [n_experts - 1]
    assert acc.hit_rate(-1) == 0.0 and acc.hit_rate(n_layers + 3) == 0.0


_doc_values = st.recursive(st.none() | st.booleans() | st.integers(-3, 40) | st.text(alphabet="0123456789x-", max_size=3),
                           lambda c: st.lists(c, max_size=3) | st.dictionaries(st.sampled_from(["0", "1", "3", "x", "placement", "replicas", "stats", "n_gpus"]), c, max_size=4),
                           max_leaves=14)


@settings(max_examples=200, deadline=None)
@given(_doc_values)
def test_placement_document_reader_accepts_or_refuses_cleanly(doc):
    """Any JSON-like document: the reader returns a complete map (missing entries round robin) or raises ValueError."""
    try:
        pm = rt.PlacementMap.from_json(doc if isinstance(doc, dict) else {"placement": doc})
    except ValueError:
        return
    prim, rep = np.asarray(pm.primary), np.asarray(pm.replica)
    assert prim.shape == rep.shape and prim.ndim == 2 and prim.size > 0 and prim.min() >= 0 and rep.min() >= -1
    back = rt.PlacementMap.from_json(pm.to_json(), pm.n_gpus)
    assert np.array_equal(np.asarray(back.primary), prim) and np.array_equal(np.asarray(back.replica), rep)
