"""Speculative-decoding control plane (C++): acceptance contracts, losslessness, tree helpers and cost models.

The invariants follow the reference's host tests (engine/src/spec/accept.rs, tree.rs, adaptive_verify.rs,
tree_shape.rs, projection.rs test modules and engine/native/*_test.c): greedy speculative output equals plain
greedy output, the sampled token's distribution equals the target's, row[pos] scores draft[pos], row[k] is a real
bonus row.
"""
import math

import numpy as np
import pytest

from inferencehackathon_b200.spec import native as sp


def _softmax(x):
    e = np.exp(x - x.max())
    return e / e.sum()


def test_chain_greedy_full_accept_uses_bonus_row():
    vocab, k = 16, 4
    rows = np.full((k + 1, vocab), -5.0, np.float32)
    draft = [3, 7, 1, 9]
    for pos, t in enumerate(draft):
        rows[pos, t] = 5.0              # row[pos] scores draft[pos]
    rows[k, 12] = 5.0                   # bonus distribution
    toks, nacc = sp.accept_chain(rows, draft, [0.0] * k, [0.5] * (k + 1), temperature=0.0)
    assert nacc == k and toks == draft + [12]


def test_chain_off_by_one_contract():
    # the draft is only right if row[pos] (not row[pos + 1]) is consulted for draft[pos]
    vocab, k = 8, 3
    rows = np.full((k + 1, vocab), -9.0, np.float32)
    rows[0, 1] = rows[1, 2] = rows[2, 3] = rows[3, 4] = 9.0
    toks, nacc = sp.accept_chain(rows, [1, 2, 3], [0.0] * 3, [0.9] * 4, temperature=0.0)
    assert (toks, nacc) == ([1, 2, 3, 4], 3)
    toks, nacc = sp.accept_chain(rows, [2, 3, 4], [0.0] * 3, [0.9] * 4, temperature=0.0)
    assert (toks, nacc) == ([1], 0)


def test_chain_greedy_rejects_at_first_mismatch_and_corrects():
    vocab, k = 10, 4
    rng = np.random.default_rng(0)
    rows = rng.standard_normal((k + 1, vocab)).astype(np.float32)
    best = rows.argmax(1)
    draft = [int(best[0]), int(best[1]), int((best[2] + 1) % vocab), int(best[3])]
    toks, nacc = sp.accept_chain(rows, draft, [-0.3] * k, rng.random(k + 1), temperature=0.0)
    assert nacc == 2 and toks == [int(best[0]), int(best[1]), int(best[2])]


def test_chain_requires_bonus_row():
    with pytest.raises(AssertionError):
        sp.accept_chain(np.zeros((3, 4), np.float32), [0, 1, 2], [0.0] * 3, [0.1] * 4)


def test_chain_deterministic_drafter_is_lossless():
    # drafter always proposes token 2 (probability 1): first emitted token must follow the target distribution
    vocab = 6
    rng = np.random.default_rng(1)
    logits = rng.standard_normal((2, vocab)).astype(np.float32) * 1.5
    p = _softmax(logits[0].astype(np.float64))
    n = 40000
    counts = np.zeros(vocab)
    us = rng.random((n, 2)).astype(np.float32)
    for i in range(n):
        toks, _ = sp.accept_chain(logits, [2], [0.0], us[i])
        counts[toks[0]] += 1
    assert np.abs(counts / n - p).max() < 0.012


def test_chain_full_distribution_is_lossless_for_sampling_drafter():
    vocab = 7
    rng = np.random.default_rng(2)
    logits = rng.standard_normal((2, vocab)).astype(np.float32) * 2
    q = _softmax(rng.standard_normal(vocab) * 2).astype(np.float32)
    p = _softmax(logits[0].astype(np.float64))
    n = 40000
    counts = np.zeros(vocab)
    xs = rng.choice(vocab, size=n, p=q / q.sum())
    us = rng.random((n, 2)).astype(np.float32)
    for i in range(n):
        toks, _ = sp.accept_chain_full(logits, [int(xs[i])], q[None], us[i])
        counts[toks[0]] += 1
    assert np.abs(counts / n - p).max() < 0.012


def test_multi_drafter_greedy_follows_the_matching_chain_with_real_bonus():
    vocab, k, n = 12, 3, 3
    rows = np.full((n, k + 1, vocab), -6.0, np.float32)
    truth = [4, 5, 6, 7]                          # greedy continuation; the 4th is the bonus
    drafts = np.array([[4, 9, 9], [4, 5, 6], [1, 1, 1]], np.int32)
    for d in range(n):
        for pos in range(k + 1):
            ok = all(drafts[d, j] == truth[j] for j in range(pos))
            rows[d, pos, truth[pos] if ok else 0] = 6.0
    r = sp.accept_multi(rows, drafts, np.full((n, k), -0.5, np.float32), np.full(n * k + 1, 0.5, np.float32), 0.0)
    assert r.tokens == truth and r.n_accepted == 3 and r.winner == 1
    assert r.accept_mask.sum() == 3


def test_multi_drafter_all_reject_samples_residual():
    vocab, k, n = 6, 2, 2
    rows = np.full((n, k + 1, vocab), -8.0, np.float32)
    rows[:, 0, 5] = 8.0
    drafts = np.array([[0, 0], [1, 1]], np.int32)
    r = sp.accept_multi(rows, drafts, np.zeros((n, k), np.float32), np.full(n * k + 1, 0.3, np.float32), 0.0)
    assert r.tokens == [5] and r.n_accepted == 0


def _tree_example():
    t = sp.SpecTree.root(100)
    a = t.add(0, 10, math.log(0.6))
    b = t.add(0, 11, math.log(0.3))
    c = t.add(a, 20, math.log(0.7))
    d = t.add(a, 21, math.log(0.2))
    e = t.add(b, 22, math.log(0.9))
    return t, (a, b, c, d, e)


def test_tree_greedy_walk_equals_plain_greedy():
    t, (a, b, c, d, e) = _tree_example()
    vocab = 32
    rows = np.full((t.n_nodes, vocab), -7.0, np.float32)
    rows[0, 11] = 7.0          # after root the target wants 11 (second child)
    rows[b, 22] = 7.0          # then 22
    rows[e, 30] = 7.0          # leaf: pure target sample
    rows[a, 20] = 7.0
    toks, nodes = sp.accept_tree(t, rows, np.full(16, 0.5, np.float32), 0.0)
    assert toks == [11, 22, 30] and nodes == [b, e]


def test_tree_all_children_rejected_samples_residual():
    t, _ = _tree_example()
    rows = np.full((t.n_nodes, 32), -7.0, np.float32)
    rows[0, 5] = 7.0
    toks, nodes = sp.accept_tree(t, rows, np.full(16, 0.5, np.float32), 0.0)
    assert toks == [5] and nodes == []


def test_tree_chain_matches_chain_accept():
    rng = np.random.default_rng(3)
    vocab, k = 9, 4
    rows = rng.standard_normal((k + 1, vocab)).astype(np.float32)
    draft = [int(x) for x in rows[:k].argmax(1)]
    draft[2] = (draft[2] + 3) % vocab
    lps = [-0.2] * k
    tree = sp.SpecTree.chain(0, draft, lps)
    u = np.full(2 * k + 2, 0.5, np.float32)
    t_toks, t_nodes = sp.accept_tree(tree, rows, u, 0.0)
    c_toks, nacc = sp.accept_chain(rows, draft, lps, u, 0.0)
    assert t_toks == c_toks and len(t_nodes) == nacc


def test_tree_first_token_distribution_is_lossless_for_point_drafts():
    # two children with probability-1 style proposals tried in order: emitted token ~ target distribution
    vocab = 5
    rng = np.random.default_rng(4)
    logits = (rng.standard_normal(vocab) * 1.5).astype(np.float32)
    p = _softmax(logits.astype(np.float64))
    t = sp.SpecTree.root(0)
    t.add(0, 1, 0.0)
    rows = np.tile(logits, (t.n_nodes, 1))
    n = 30000
    counts = np.zeros(vocab)
    us = rng.random((n, 4)).astype(np.float32)
    for i in range(n):
        toks, _ = sp.accept_tree(t, rows, us[i])
        counts[toks[0]] += 1
    assert np.abs(counts / n - p).max() < 0.012


def test_build_from_source_bfs_shape():
    def source(prefix, branch):
        return [(len(prefix) * 10 + j, math.log(0.5 / (j + 1))) for j in range(branch)]
    t = sp.SpecTree.build_from_source(source, [1, 2], 99, depth=3, branch=2)
    assert t.n_nodes == 1 + sp.tree_nodes(2, 3)
    assert all(t.depth(i) <= 3 for i in range(t.n_nodes))
    assert len(t.children(0)) == 2


def test_tree_attn_build_positions_and_slots():
    t, (a, b, c, d, e) = _tree_example()
    ctx = 50
    pos, off, slots = sp.tree_attn_build(t.parent, ctx)
    assert pos.tolist() == [ctx - 1, ctx, ctx, ctx + 1, ctx + 1, ctx + 1]
    anc = lambda i: slots[off[i]:off[i + 1]].tolist()
    assert anc(0) == [] and anc(a) == [ctx + a - 1]
    assert anc(c) == [ctx + a - 1, ctx + c - 1] and anc(e) == [ctx + b - 1, ctx + e - 1]
    m = sp.tree_mask(t.parent)
    assert m[c - 1, a - 1] and m[c - 1, c - 1] and not m[c - 1, b - 1] and not m[a - 1, c - 1]


def test_draft_top_candidates_draft_space_logprobs():
    rng = np.random.default_rng(5)
    dv = 32
    logits = rng.standard_normal(dv).astype(np.float32)
    d2t = (np.arange(dv) * 7 + 3).astype(np.int32)
    toks, lps = sp.draft_top_candidates(logits, 4, d2t)
    order = np.argsort(-logits)[:4]
    assert toks == d2t[order].tolist()
    lsm = logits - (np.log(np.exp(logits - logits.max()).sum()) + logits.max())
    assert np.allclose(lps, lsm[order], atol=1e-5)


def test_sdpa_tree_ref_matches_numpy():
    rng = np.random.default_rng(6)
    t, _ = _tree_example()
    n, n_q, n_kv, hd, ctx = t.n_nodes, 4, 2, 16, 9
    q = rng.standard_normal((n, n_q, hd)).astype(np.float32)
    kc = rng.standard_normal((n_kv, ctx, hd)).astype(np.float32)
    vc = rng.standard_normal((n_kv, ctx, hd)).astype(np.float32)
    kd = rng.standard_normal((n, n_kv, hd)).astype(np.float32)
    vd = rng.standard_normal((n, n_kv, hd)).astype(np.float32)
    qg = rng.random(hd).astype(np.float32) + 0.5
    kg = rng.random(hd).astype(np.float32) + 0.5
    theta, eps = 1e4, 1e-6
    out = sp.sdpa_tree_ref(t.parent, ctx, q, kc, vc, kd, vd, qg, kg, eps, theta)

    def nr(x, g, pos):
        x = x / np.sqrt((x * x).mean() + eps) * g
        half = hd // 2
        ang = pos * theta ** (-np.arange(half) / half)
        c, s = np.cos(ang), np.sin(ang)
        return np.concatenate([x[:half] * c - x[half:] * s, x[half:] * c + x[:half] * s])

    pos, off, slots = sp.tree_attn_build(t.parent, ctx)
    assert np.all(out[0] == 0)
    for i in range(1, n):
        anc_nodes = [s - ctx + 1 for s in slots[off[i]:off[i + 1]]]
        for h in range(n_q):
            kv = h // (n_q // n_kv)
            qq = nr(q[i, h], qg, pos[i])
            keys = np.concatenate([kc[kv], np.stack([nr(kd[a, kv], kg, pos[a]) for a in anc_nodes])])
            vals = np.concatenate([vc[kv], np.stack([vd[a, kv] for a in anc_nodes])])
            w = _softmax(keys @ qq / math.sqrt(hd))
            assert np.allclose(out[i, h], w @ vals, atol=2e-4)


def test_spec_round_host_template():
    vocab, k = 20, 3
    dl = np.full((k, 8), -3.0, np.float32)
    dl[0, 1] = dl[1, 2] = dl[2, 3] = 3.0
    d2t = np.arange(8, dtype=np.int32) + 10

    def verify(tokens):
        assert tokens == [11, 12, 13]
        rows = np.full((k + 1, vocab), -5.0, np.float32)
        rows[0, 11] = rows[1, 12] = rows[2, 0] = rows[3, 1] = 5.0
        return rows

    toks, nacc = sp.spec_round(dl, vocab, verify, [0.5] * (k + 1), d2t=d2t, temperature=0.0)
    assert (toks, nacc) == ([11, 12, 0], 2)


def test_verify_cost_and_adaptive_depth():
    assert sp.verify_cost(8, 0.0) == pytest.approx(1.0)
    assert sp.verify_cost(0, 0.0) == pytest.approx(0.34)
    assert sp.verify_cost(40, 1.0) == pytest.approx(1.0)
    assert sp.verify_cost(16, 0.86) == pytest.approx(0.86 + 0.14 * (0.34 + 0.66 * 2))
    # floor-dominated: verifying deeper is nearly free, so the full depth wins
    plan = sp.adaptive_verify_depth([0.8] * 5, [list(range(8 * i, 8 * i + 8)) for i in range(5)], 0.95)
    assert plan.depth == 5 and plan.union_size == 40
    # no floor and disjoint experts: each extra position costs a lot; low acceptance keeps the depth at 1
    plan = sp.adaptive_verify_depth([0.3] * 5, [list(range(8 * i, 8 * i + 8)) for i in range(5)], 0.0)
    assert plan.depth == 1
    # shared experts make depth cheap again
    plan = sp.adaptive_verify_depth([0.9] * 4, [list(range(8))] * 4, 0.0)
    assert plan.depth == 4 and plan.union_size == 8
    assert plan.emitted == pytest.approx(1 + 0.9 + 0.81 + 0.729 + 0.6561, rel=1e-5)
    assert sp.adaptive_verify_depth([], [], 0.5).depth == 0


def test_tree_shape_model():
    assert sp.level_advance_prob(0.5, 1) == pytest.approx(0.5)
    assert sp.level_advance_prob(0.5, 2) == pytest.approx(0.75)
    assert sp.tree_nodes(3, 2) == 12
    assert sp.tree_expected_accepted(0.8, 0.5, 1, 3) == pytest.approx(0.8 + 0.4 + 0.2)
    wide = sp.tree_expected_accepted(0.8, 0.5, 3, 3)
    assert wide > sp.tree_expected_accepted(0.8, 0.5, 1, 3)
    shape = sp.tree_shape_optimal(2.5, 0.7, verify_flat_cost=1.0, head_level_cost=0.02, node_budget=64)
    assert sp.tree_nodes(shape.branch, shape.depth) <= 64 and shape.speedup > 1.0
    tight = sp.tree_shape_optimal(2.5, 0.7, verify_flat_cost=1.0, head_level_cost=0.02, node_budget=4)
    assert sp.tree_nodes(tight.branch, tight.depth) <= 4 and tight.speedup <= shape.speedup + 1e-6


def test_persistence_reproduces_mean_accept_len():
    for mal, first, depth in [(3.0, 0.8, 5), (2.2, 0.7, 5), (4.5, 0.9, 8)]:
        p = sp.persistence(mal, first, depth)
        acc, pref = 0.0, 1.0
        for i in range(depth):
            pref *= first if i == 0 else p
            acc += pref
        assert 1.0 + acc == pytest.approx(mal, abs=2e-3)
    assert sp.persistence(1.0, 0.8, 5) == 0.0
    assert sp.persistence(100.0, 0.9, 4) == pytest.approx(0.999)
    g = sp.predict_speedup(3.0, 0.8, 5, 24, 0.86, head_eager_cost=0.1, draft_graph_cost=0.15, graphs=True)
    e = sp.predict_speedup(3.0, 0.8, 5, 24, 0.86, head_eager_cost=0.1, draft_graph_cost=0.15, graphs=False)
    assert g > e > 0


def test_route_aware_select_and_union():
    u = sp.ExpertUnion([1, 2, 3, 200])
    assert len(u) == 4 and 200 in u and 5 not in u and u.overlap([1, 5, 200]) == 2
    lps = [-0.1, -0.5]
    ex = [[10, 11, 12], [1, 2, 3]]
    assert sp.route_aware_select(lps, ex, u, 0.0) == 0
    assert sp.route_aware_select(lps, ex, u, 0.5) == 1


# ---- property-based checks (hypothesis) ---------------------------------------------------------------------------------------------
from hypothesis import given, settings, strategies as st   # noqa: E402


@settings(max_examples=120, deadline=None)
@given(st.integers(2, 24), st.integers(1, 8), st.integers(0, 2 ** 31 - 1))
def test_greedy_chain_accept_is_the_longest_matching_prefix_plus_the_targets_token(vocab, k, seed):
    """For any logits and any draft, greedy acceptance emits exactly: the drafted tokens up to the first position where
    the draft differs from the arg-max of the row that scores it, then that row's arg-max (or the bonus row's after a
    full accept); the random numbers and the draft's log-probabilities play no part."""
    rng = np.random.default_rng(seed)
    rows = rng.standard_normal((k + 1, vocab)).astype(np.float32)
    best = rows.argmax(1)
    draft = [int(best[p]) if rng.random() < 0.7 else int(rng.integers(vocab)) for p in range(k)]
    n = 0
    while n < k and draft[n] == int(best[n]):
        n += 1
    toks, nacc = sp.accept_chain(rows, draft, (-rng.random(k)).tolist(), rng.random(k + 1).tolist(), temperature=0.0)
    assert nacc == n and toks == draft[:n] + [int(best[n])]
    # the same through the tree walk over a chain-shaped tree, and through the full-distribution variant
    q = np.full((k, vocab), 1.0 / vocab, np.float32)
    toks_full, nacc_full = sp.accept_chain_full(rows, draft, q, rng.random(k + 1).tolist(), temperature=0.0)
    assert (toks_full, nacc_full) == (toks, nacc)


@settings(max_examples=60, deadline=None)
@given(st.lists(st.integers(0, 1000), min_size=1, max_size=12), st.integers(1, 64))
def test_tree_builder_rows_are_exactly_the_ancestor_chains(raw_parents, context_len):
    """For any tree given as parent indices (node 0 = the last committed token, a parent precedes its child): a draft
    node sees exactly itself and its draft ancestors, its RoPE position is context_len + depth - 1, and its CSR slot list
    is that chain, root side first, with node i in cache slot context_len + i - 1."""
    parent = [-1] + [p % i for i, p in enumerate(raw_parents) if i > 0]
    n = len(parent)
    mask = sp.tree_mask(parent)
    pos, off, slots = sp.tree_attn_build(parent, context_len)
    assert mask.shape == (n - 1, n - 1) and int(pos[0]) == context_len - 1 and int(off[0]) == int(off[1]) if n > 1 else True
    for i in range(1, n):
        chain, j = [], i
        while j > 0:
            chain.append(j)
            j = parent[j]
        chain.reverse()                                                     # root side first, self last
        assert {c + 1 for c in range(n - 1) if mask[i - 1, c]} == set(chain)
        assert int(pos[i]) == context_len + len(chain) - 1
        assert slots[off[i]:off[i + 1]].tolist() == [context_len + a - 1 for a in chain]


@settings(max_examples=150, deadline=None)
@given(st.integers(2, 12), st.integers(1, 6), st.sampled_from([0.0, 0.3, 1.0, 7.5]), st.integers(0, 2 ** 31 - 1))
def test_acceptance_routines_stay_in_bounds_on_adversarial_input(vocab, k, temperature, seed):
    """Drafted token ids outside the vocabulary, log-probabilities of minus infinity, uniforms of exactly 0 and 1 and
    huge logits: every routine returns tokens inside the vocabulary, accepts at most k drafts, emits n_accepted + 1
    tokens, and touches no memory outside its arguments (this test also runs under ASan in ops/sanitize_ctrl.py)."""
    rng = np.random.default_rng(seed)
    rows = (rng.standard_normal((k + 1, vocab)) * rng.choice([1.0, 50.0])).astype(np.float32)
    draft = [int(t) for t in rng.integers(-3, vocab + 3, size=k)]          # some ids are not in the vocabulary
    lps = [float(x) for x in rng.choice([0.0, -0.5, -30.0, -np.inf], size=k)]
    u = [float(x) for x in rng.choice([0.0, 1.0, 0.5, 0.999999], size=k + 1)]
    toks, nacc = sp.accept_chain(rows, draft, lps, u, temperature=temperature)
    assert 0 <= nacc <= k and len(toks) == nacc + 1 and all(0 <= t < vocab for t in toks[nacc:])
    assert toks[:nacc] == draft[:nacc] and all(0 <= t < vocab for t in toks[:nacc])   # an id outside the vocabulary is never accepted
    q = rng.random((k, vocab)).astype(np.float32)
    q /= q.sum(1, keepdims=True)
    toks, nacc = sp.accept_chain_full(rows, draft, q, u, temperature=temperature)
    assert 0 <= nacc <= k and len(toks) == nacc + 1 and all(0 <= t < vocab for t in toks)
    # a chain-shaped tree and a bushy tree over the same ids
    chain = sp.SpecTree.chain(0, draft, lps)
    trows = (rng.standard_normal((chain.n_nodes, vocab)) * 5).astype(np.float32)
    toks, nodes = sp.accept_tree(chain, trows, [float(x) for x in rng.random(4 * chain.n_nodes + 4)], temperature=temperature)
    assert 1 <= len(toks) <= k + 1 and len(nodes) == len(toks) - 1 and all(0 <= t < vocab for t in toks)
    bushy = sp.SpecTree.root(0)
    for i in range(k):
        bushy.add(int(rng.integers(0, bushy.n_nodes)), draft[i], lps[i])
    brows = (rng.standard_normal((bushy.n_nodes, vocab)) * 5).astype(np.float32)
    toks, nodes = sp.accept_tree(bushy, brows, [float(x) for x in rng.random(4 * bushy.n_nodes + 4)], temperature=temperature)
    assert 1 <= len(toks) <= k + 1 and all(0 <= t < vocab for t in toks)
    assert all(bushy.parent[b] == a for a, b in zip([0] + nodes, nodes))    # the accepted nodes form a root path
    # several drafters
    n = 2
    mt = np.stack([rows, rows[::-1].copy()])
    md = rng.integers(-2, vocab + 2, size=(n, k))
    res = sp.accept_multi(mt, md, np.zeros((n, k), np.float32), [float(x) for x in rng.random(n * k + 1)], temperature=temperature)
    assert 0 <= res.n_accepted <= k and len(res.tokens) == res.n_accepted + 1 and all(0 <= t < vocab for t in res.tokens)


@settings(max_examples=80, deadline=None)
@given(st.lists(st.integers(-3, 14), min_size=1, max_size=12), st.integers(1, 32))
def test_tree_builder_terminates_on_malformed_parent_arrays(parent, context_len):
    """Parents that are negative, out of range, self-referencing or cyclic: the builder and the mask return (a walk is
    cut after n steps, an invalid parent counts as the root), every position stays within context_len - 1 + n and every
    slot within the draft rows."""
    n = len(parent)
    pos, off, slots = sp.tree_attn_build(parent, context_len)
    mask = sp.tree_mask(parent)
    assert mask.shape == (max(n - 1, 0), max(n - 1, 0))
    assert all(context_len - 1 <= int(p) <= context_len - 1 + n for p in pos)
    assert all(context_len <= int(s) < context_len + n for s in slots) and int(off[-1]) == len(slots)
    for i in range(1, n):
        assert mask[i - 1, i - 1]                                           # a node always sees itself


@settings(max_examples=100, deadline=None)
@given(st.integers(1, 10), st.integers(0, 2 ** 31 - 1))
def test_cost_models_and_selection_on_arbitrary_input(k, seed):
    """Verify-depth planner, tree-shape model, route-aware selection and the draft-candidate mapping with arbitrary
    (also out-of-range, negative or empty) ids and extreme parameters: results stay in range and finite."""
    rng = np.random.default_rng(seed)
    probs = rng.random(k).tolist()
    experts = [[int(e) for e in rng.integers(-5, 5000, size=int(rng.integers(0, 9)))] for _ in range(k)]
    plan = sp.adaptive_verify_depth(probs, experts, floor_fraction=float(rng.choice([0.0, 0.5, 0.86, 1.0])))
    assert 1 <= plan.depth <= k and np.isfinite([plan.emitted, plan.cost, plan.value]).all() and plan.cost > 0
    assert plan.union_size <= sum(len(e) for e in experts[: plan.depth])
    # fewer experts per position than positions (a short list): treated as empty, no read past the list
    assert 1 <= sp.adaptive_verify_depth(probs, experts[: k // 2]).depth <= k
    shape = sp.tree_shape_optimal(float(rng.uniform(1.0, 9.0)), float(rng.uniform(0.05, 1.0)),
                                  node_budget=int(rng.integers(1, 200)), max_branch=int(rng.integers(1, 9)),
                                  max_depth=int(rng.integers(1, 9)))
    assert shape.branch >= 1 and shape.depth >= 1 and np.isfinite([shape.emitted, shape.speedup]).all()
    for p in (0.0, 0.3, 1.0):
        for b in (1, 4):
            assert 0.0 <= sp.level_advance_prob(p, b) <= 1.0 + 1e-6
    union = sp.ExpertUnion([int(e) for e in rng.integers(-10, 9000, size=12)])
    idx = sp.route_aware_select((-rng.random(k) * 5).tolist(), experts, union, float(rng.choice([0.0, 0.5, 100.0])))
    assert 0 <= idx < k
    dv = int(rng.integers(1, 12))
    d2t = rng.integers(0, 50, size=dv).astype(np.int32)
    toks, lps = sp.draft_top_candidates(rng.standard_normal(dv) * rng.choice([1.0, 80.0]), int(rng.integers(1, 20)), d2t)
    assert 1 <= len(toks) <= dv and all(t in set(d2t.tolist()) for t in toks)
    assert all(np.isfinite(lp) and lp <= 1e-5 for lp in lps) and lps == sorted(lps, reverse=True)


@settings(max_examples=40, deadline=None)
@given(st.lists(st.integers(-2, 8), min_size=2, max_size=7), st.integers(0, 5), st.integers(0, 2 ** 31 - 1))
def test_tree_attention_oracle_is_finite_on_any_parent_array(parent, ctx, seed):
    """The fp32 tree-attention oracle with malformed parent arrays (negative, out of range, cycles) and an empty
    context: it returns, the root row stays zero and every other row is finite."""
    rng = np.random.default_rng(seed)
    n, n_q, n_kv, hd = len(parent), 4, 2, 8
    q = rng.standard_normal((n, n_q, hd)).astype(np.float32)
    out = sp.sdpa_tree_ref(parent, ctx, q, rng.standard_normal((n_kv, ctx, hd)).astype(np.float32),
                           rng.standard_normal((n_kv, ctx, hd)).astype(np.float32),
                           rng.standard_normal((n, n_kv, hd)).astype(np.float32),
                           rng.standard_normal((n, n_kv, hd)).astype(np.float32), np.ones(hd, np.float32), np.ones(hd, np.float32))
    assert out.shape == q.shape and np.isfinite(out).all() and not out[0].any()
