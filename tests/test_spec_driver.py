"""Speculative drivers: n-gram drafter, multi-drafter engine, EAGLE-3-style engine (chain + tree), telemetry, and
the real-engine runner. The central invariant (engine/src/spec tests of the reference): greedy speculative
decoding emits exactly the tokens plain greedy decoding emits."""
import json

import numpy as np
import pytest
import torch

from inferencehackathon_b200.runtime.engine import InferenceEngine
from inferencehackathon_b200.spec import driver as D
from inferencehackathon_b200.spec import ngram
from inferencehackathon_b200.spec.eagle_head import EagleHead, EagleHeadConfig, default_aux_layers


# ---- n-gram drafter ------------------------------------------------------------------------------------------------------
def test_ngram_proposes_continuation_of_latest_match():
    d = ngram.NGramDrafter(n=2)
    ctx = [1, 2, 3, 4, 9, 1, 2, 7, 8, 1, 2]
    assert d.propose(ctx, 3) == [7, 8, 1]            # the most recent earlier "1 2" is followed by 7 8 1
    assert d.propose(ctx + [7], 2) == [8, 1]
    assert ngram.NGramDrafter(n=3).propose([5, 6, 7], 4) == []


def test_ngram_backs_off_to_shorter_ngrams_and_handles_rollback():
    d = ngram.NGramDrafter(n=3, min_n=1)
    assert d.propose([4, 5, 6, 9, 9, 6], 2) == [9, 9]   # only the unigram "6" matches
    assert d.propose([4, 5, 6, 9], 2) == []             # shorter context after a rollback: index rebuilt
    assert d.propose([4, 5, 6, 9, 4, 5], 2) == [6, 9]


def test_ngram_tau_extremes():
    rep = ngram.repeated_block_stream(32, 8, vocab=1000)
    r = ngram.ngram_tau(rep, k=8, n=2, prompt_len=64)
    assert r.tau > 8.5                                   # everything after the first block is predictable
    rnd = np.random.default_rng(0).integers(0, 50000, 2000).tolist()
    assert ngram.ngram_tau(rnd, k=8, n=2).tau < 1.1
    mk = ngram.zipf_markov_stream(3000)
    assert 1.2 < ngram.ngram_tau(mk, k=8, n=1).tau < 6.0
    assert ngram.main(["--k", "3", "--n", "1", "--length", "512"]) == 0


# ---- mock-model round logic ------------------------------------------------------------------------------------------------
class EchoTarget(D.ModelRunner):
    """Next token = (token + 1) mod vocab."""

    def __init__(self, vocab):
        self.v = vocab
        self.calls = 0

    def vocab_size(self):
        return self.v

    def forward_single(self, context, token):
        self.calls += 1
        row = np.zeros(self.v, np.float32)
        row[(token + 1) % self.v] = 12.0
        return row


class CountingHead:
    """Proposes token + 1 (right) and a decoy; every candidate uses experts 0..7."""

    def __init__(self, wrong_after=99):
        self.wrong_after = wrong_after

    def candidates(self, context, chain, width):
        last = (list(context) + list(chain))[-1]
        good = last + 1 if len(chain) < self.wrong_after else last + 5
        return [D.Candidate(good, -0.1, list(range(8))), D.Candidate(last + 50, -0.4, list(range(64, 72)))][:width]


def test_eagle_chain_round_accepts_and_keeps_union_small():
    eng = D.Eagle3Engine(D.RouteAwareDrafter(CountingHead(), 2.0), EchoTarget(512), D.Eagle3Config(4, 2, 512, 0.86))
    run, st = eng.step([1, 2, 3], D.FixedRng(0.01))
    assert st.n_drafted == 4 and 1 <= st.verify_depth <= 4 and st.union_size == 8
    assert run.n_accepted() == st.verify_depth
    assert run.all_tokens() == [4 + i for i in range(st.verify_depth + 1)]   # bonus comes from the real row k


def test_eagle_rejection_emits_target_token():
    eng = D.Eagle3Engine(D.RouteAwareDrafter(CountingHead(wrong_after=2), 0.0), EchoTarget(512),
                         D.Eagle3Config(4, 2, 512, 1.0))
    run, st = eng.step([10], D.FixedRng(0.5))
    assert run.accepted == [11, 12] and run.bonus_token == 13 and st.n_accepted == 2


def test_eagle_empty_head_degenerates_and_decode_falls_back():
    class Empty:
        def candidates(self, *a):
            return []
    eng = D.Eagle3Engine(D.RouteAwareDrafter(Empty(), 1.0), EchoTarget(64), D.Eagle3Config(4, 2, 64, 0.0))
    run, st = eng.step([1], D.FixedRng(0.1))
    assert st.n_drafted == 0 and st.verify_depth == 0 and run.n_accepted() == 0
    out, tel = eng.decode([1], D.DecodeStop(5), D.FixedRng(0.1))
    assert out == [2, 3, 4, 5, 6] and tel.snapshot()["spec_rounds"] == 0


def test_eagle_decode_chain_and_tree_match_plain_greedy_and_stop_on_eos():
    for tree in (None, (3, 2)):
        eng = D.Eagle3Engine(D.RouteAwareDrafter(CountingHead(wrong_after=3), 0.0), EchoTarget(256),
                             D.Eagle3Config(5, 2, 256, 0.86))
        out, tel = eng.decode([7], D.DecodeStop(20), D.Rng(1), tree=tree)
        assert out == list(range(8, 28))
        assert tel.mean_accept_length() > 2.0
        out, _ = eng.decode([7], D.DecodeStop(20, eos_token=12), D.Rng(1), tree=tree)
        assert out == [8, 9, 10, 11, 12]


def test_multi_drafter_engine_picks_the_right_drafter():
    class Fixed:
        def __init__(self, delta):
            self.delta = delta

        def propose(self, ctx, k):
            return [ctx[-1] + self.delta * (i + 1) for i in range(k)]

    eng = D.SpecEngine(EchoTarget(1000), D.ChainDrafterPool([Fixed(3), Fixed(1)]), D.SpecConfig(4, 1000, 0.0))
    run, st = eng.step([5], D.Rng(0))
    assert run.accepted == [6, 7, 8, 9] and run.bonus_token == 10 and run.winning_drafter == 1 and st.n_accepted == 4
    out, tel = eng.decode([5], D.DecodeStop(12), D.Rng(0))
    assert out == list(range(6, 18)) and tel.mean_accept_length() == pytest.approx(5.0)


def test_route_aware_drafter_lambda():
    class Rot:
        def candidates(self, c, chain, w):
            i = len(chain)
            return [D.Candidate(10 + i, -0.10, list(range(8 * i, 8 * i + 8))),       # best prob, fresh experts
                    D.Candidate(50 + i, -0.30, list(range(8)))]                      # slightly worse, shared experts
    plain, u0 = D.RouteAwareDrafter(Rot(), 0.0).draft_chain([1], 3, 2)
    aware, u1 = D.RouteAwareDrafter(Rot(), 1.0).draft_chain([1], 3, 2)
    assert plain.tokens == [10, 11, 12] and len(u0) == 24
    assert aware.tokens == [10, 51, 52] and len(u1) == 8
    prop, experts, plan = D.RouteAwareDrafter(Rot(), 1.0).draft_and_plan([1], 3, 2, 0.5)
    assert plan is not None and 1 <= plan.depth <= 3 and len(experts) == 3


def test_spec_telemetry():
    t = D.SpecTelemetry()
    assert t.snapshot()["mean_accept_length"] == 0.0 and t.acceptance_rate() == 0.0
    t.record(D.Eagle3RoundStats(2, 4, 3, 8))
    t.record(D.Eagle3RoundStats(1, 4, 2, 16))
    t.record(D.Eagle3RoundStats(0, 0, 0, 0))
    s = t.snapshot()
    assert s["rounds"] == 3 and s["spec_rounds"] == 2
    assert t.mean_accept_length() == pytest.approx(2.0) and t.mean_union() == pytest.approx(12.0)
    assert t.mean_verify_depth() == pytest.approx(2.5) and t.acceptance_rate() == pytest.approx(3 / 8)
    frame = t.to_sse_frame()
    assert frame.startswith("data: ") and frame.endswith("\n\n") and json.loads(frame[6:])["rounds"] == 3
    assert t.projected_speedup(0.1, 0.15, 4, 0.86, True) > 0


# ---- real engine (PyTorch path, tiny model) ------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def tiny():
    eng = InferenceEngine.build("tiny", weights="fp32", max_seq=256)
    rng = np.random.default_rng(0)
    block = rng.integers(0, 2048, 12).tolist()
    prompt = block * 3
    plain = eng.generate(prompt, 24).tokens
    return eng, prompt, plain


def test_engine_runner_window_equals_sequential(tiny):
    eng, prompt, plain = tiny
    r = D.EngineRunner(eng)
    rows = r.forward_batch(prompt + [plain[0]], plain[1:4])
    assert rows.shape == (4, 2048)
    assert rows.argmax(1).tolist() == plain[1:5]
    single = r.forward_single(prompt, plain[0])           # rolls the cache back and re-feeds one token
    assert np.allclose(single, rows[0], atol=1e-4)
    assert r.forwards == 2


def test_ngram_spec_on_engine_equals_plain_greedy(tiny):
    eng, prompt, plain = tiny
    r = D.EngineRunner(eng)
    se = D.SpecEngine(r, D.ChainDrafterPool([ngram.NGramDrafter(2)]), D.SpecConfig(4, 2048, 0.0))
    out, tel = se.decode(prompt, D.DecodeStop(24), D.Rng(0))
    assert out == plain
    assert r.forwards <= 24


def test_eagle_head_spec_on_engine_equals_plain_greedy_chain_and_tree(tiny):
    eng, prompt, plain = tiny
    aux = default_aux_layers(eng.cfg.model.n_layers)
    for tree in (None, (2, 2)):
        r = D.EngineRunner(eng, aux_layers=aux)
        head = EagleHead(EagleHeadConfig(hidden=256, n_heads=4, n_kv_heads=2, head_dim=32, draft_vocab=512,
                                         target_vocab=2048), eng.weights.embed)
        head.bind(r)
        e3 = D.Eagle3Engine(D.RouteAwareDrafter(head, 0.0), r, D.Eagle3Config(3, 2, 2048, 0.86))
        out, tel = e3.decode(prompt, D.DecodeStop(16), D.Rng(0), tree=tree)
        assert out == plain[:16]
        assert tel.snapshot()["spec_rounds"] >= 1          # the head did draft once target features existed


def test_spec_driver_generate_and_serving_hook(tiny):
    eng, prompt, plain = tiny
    drv = D.SpecDriver(eng, ngram.NGramDrafter(2), depth=4, width=1, floor_fraction=1.0)
    assert drv.generate(prompt, 24) == plain
    assert drv.telemetry.rounds >= 1
    tree = D.SpecDriver(eng, ngram.NGramDrafter(2), tree=(3, 1))
    assert tree.generate(prompt, 24) == plain


def test_tree_beam_budget_and_spec_bench_cli(capsys):
    from inferencehackathon_b200.spec.native import SpecTree
    import json as _json

    def source(prefix, b):                       # child i of any node: token 10 * depth + i, log-prob -i
        d = len(prefix) - 3
        return [(10 * (d + 1) + i, -float(i)) for i in range(b)]

    full = SpecTree.build_from_source(source, [1, 2, 3], 3, 3, 3)
    assert full.n_nodes - 1 == 3 + 9 + 27
    beam = SpecTree.build_from_source(source, [1, 2, 3], 3, 4, 4, max_nodes=16)
    assert beam.n_nodes - 1 == 16                                    # four levels of four
    assert max(beam.depth(i) for i in range(beam.n_nodes)) == 4
    # the best path (always child 0) survives at every level
    assert [beam.tokens[i] for i in range(beam.n_nodes) if beam.depth(i) == 4][0] == 40
    from inferencehackathon_b200.spec import bench as sb
    assert sb.main(["--model", "tiny", "--block", "8", "--repeats", "4", "--new-tokens", "12", "--max-candidates", "8",
                    "--tree", "2x2"]) == 0
    line = _json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["ngram"]["lossless"] and line["eagle_tree"]["lossless"]
    assert line["ngram"]["forwards_per_token"] <= 1.0 + 1e-9


from hypothesis import HealthCheck, given, settings, strategies as st   # noqa: E402


@settings(max_examples=12, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture])
@given(st.integers(1, 7), st.integers(1, 3), st.integers(1, 3), st.integers(2, 20), st.integers(0, 10 ** 6))
def test_greedy_speculation_is_lossless_for_any_depth_drafter_order_and_prompt(tiny, depth, n, min_n, block, seed):
    """The central invariant, over random draft depths, n-gram orders and prompts (repetitive enough that drafts get
    accepted, random enough that many get rejected): greedy speculative decoding emits exactly plain greedy decoding's
    tokens, with no more target forwards than tokens."""
    eng = tiny[0]
    rng = np.random.default_rng(seed)
    prompt = (rng.integers(0, 2048, block).tolist() * 3)[: 40] + rng.integers(0, 2048, 3).tolist()
    plain = eng.generate(prompt, 12).tokens
    r = D.EngineRunner(eng)
    se = D.SpecEngine(r, D.ChainDrafterPool([ngram.NGramDrafter(max(n, min_n), min_n=min(n, min_n))]),
                      D.SpecConfig(depth, 2048, 0.0))
    out, _tel = se.decode(prompt, D.DecodeStop(12), D.Rng(seed))
    assert out == plain and r.forwards <= 12


def _ngram_oracle(ctx, k, n, min_n):
    L = len(ctx)
    for g in range(min(n, L), min_n - 1, -1):
        suffix = ctx[L - g:]
        for end in range(L - 1, g - 1, -1):                                 # latest earlier occurrence first
            if ctx[end - g:end] == suffix:
                return ctx[end:end + k]
    return []


@settings(max_examples=150, deadline=None)
@given(st.integers(1, 4), st.integers(1, 4), st.integers(1, 6),
       st.lists(st.tuples(st.sampled_from(["extend", "rollback", "replace"]), st.integers(1, 9), st.integers(0, 2 ** 31 - 1)),
                min_size=1, max_size=12))
def test_ngram_drafter_with_incremental_index_equals_a_rescan(n, min_n, k, ops):
    """One drafter instance across any sequence of context extensions, rollbacks and rewrites (what speculative rounds
    with rejections produce): its proposal always equals a from-scratch scan for the latest earlier match."""
    n, min_n = max(n, min_n), min(n, min_n)
    d = ngram.NGramDrafter(n, min_n=min_n)
    ctx = []
    for op, amount, seed in ops:
        rng = np.random.default_rng(seed)
        if op == "extend":
            ctx = ctx + rng.integers(0, 3, amount).tolist()                 # a tiny vocabulary: matches are frequent
        elif op == "rollback":
            ctx = ctx[: max(0, len(ctx) - amount)]
        else:
            cut = max(0, len(ctx) - amount)
            ctx = ctx[:cut] + rng.integers(0, 3, amount).tolist()           # the tail is rewritten with other tokens
        assert d.propose(ctx, k) == _ngram_oracle(ctx, k, n, min_n)


@settings(max_examples=8, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture])
@given(st.integers(1, 3), st.integers(1, 3), st.integers(1, 4), st.integers(0, 10 ** 6))
def test_tree_speculation_with_an_untrained_head_is_lossless_for_any_tree_shape(tiny, branch, depth, chain_depth, seed):
    """An EAGLE-style head with random weights drafts badly, which is the point: whatever tree shape it proposes and
    however few of its nodes are accepted, the greedy output equals plain greedy decoding."""
    eng = tiny[0]
    rng = np.random.default_rng(seed)
    prompt = rng.integers(0, 2048, 20).tolist()
    plain = eng.generate(prompt, 10).tokens
    aux = default_aux_layers(eng.cfg.model.n_layers)
    r = D.EngineRunner(eng, aux_layers=aux)
    torch.manual_seed(seed)
    head = EagleHead(EagleHeadConfig(hidden=256, n_heads=4, n_kv_heads=2, head_dim=32, draft_vocab=512, target_vocab=2048),
                     eng.weights.embed)
    head.bind(r)
    e3 = D.Eagle3Engine(D.RouteAwareDrafter(head, 0.0), r, D.Eagle3Config(chain_depth, 2, 2048, 0.86))
    out, _ = e3.decode(prompt, D.DecodeStop(10), D.Rng(seed), tree=(branch, depth))
    assert out == plain
