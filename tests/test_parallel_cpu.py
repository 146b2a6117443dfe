"""Tensor-, expert- and hybrid-parallel runs over gloo must reproduce the single-rank model (CPU, world 2/4)."""
import torch

from inferencehackathon_b200 import TINY
from inferencehackathon_b200.parallel.launch import run_cpu_ranks
from inferencehackathon_b200.runtime.engine import InferenceEngine

PROMPT = torch.randint(0, TINY.vocab, (32,), generator=torch.Generator().manual_seed(0)).tolist()


def _run(rank, world, tp, ep, n_new, kv_seq_split=False):
    e = InferenceEngine.build("tiny", tp=tp, ep=ep, rank=rank, world=world, weights="fp32", max_seq=128,
                              kv_seq_split=kv_seq_split)
    pre = e.prefill(PROMPT, return_logits=True)
    logits = pre.logits[0].clone()
    e.reset()
    res = e.generate(PROMPT, n_new)
    return logits, res.tokens, [[r.experts for r in step] for step in res.routes], e.comm.n_collectives


def _single(n_new):
    e = InferenceEngine.build("tiny", weights="fp32", max_seq=128)
    pre = e.prefill(PROMPT, return_logits=True)
    logits = pre.logits[0].clone()
    e.reset()
    res = e.generate(PROMPT, n_new)
    return logits, res.tokens, [[r.experts for r in step] for step in res.routes]


def _check(outs, ref, n_new):
    ref_logits, ref_tokens, ref_routes = ref
    for logits, tokens, routes, ncoll in outs:
        assert torch.allclose(logits, ref_logits, atol=5e-4, rtol=1e-4)
        assert tokens == ref_tokens and len(tokens) == n_new
        assert [[sorted(e) for e in s] for s in routes] == [[sorted(e) for e in s] for s in ref_routes]
        assert ncoll > 0


def test_tp2_matches_single_rank():
    _check(run_cpu_ranks(_run, 2, (2, 1, 12)), _single(12), 12)


def test_ep2_matches_single_rank():
    _check(run_cpu_ranks(_run, 2, (1, 2, 12)), _single(12), 12)


def test_hybrid_tp2_ep4_matches_single_rank():
    _check(run_cpu_ranks(_run, 4, (2, 4, 6)), _single(6), 6)


def test_tp4_with_replicated_kv_heads_matches_single_rank():
    """More tensor-parallel ranks than KV heads (2 KV heads on 4 ranks): each KV head lives on two ranks, as at TP8
    with the four KV heads of the Qwen3 models."""
    assert TINY.n_kv_heads < 4
    _check(run_cpu_ranks(_run, 4, (4, 1, 6)), _single(6), 6)


def test_tp4_with_kv_rows_split_between_the_ranks_that_share_a_head():
    """Two KV heads on four ranks, but the two ranks of a head keep alternate cache rows and merge partial attention
    results (context-parallel split-KV): same logits, tokens and routes as one rank, with half the KV rows per rank."""
    outs = run_cpu_ranks(_run, 4, (4, 1, 6, True))
    _check(outs, _single(6), 6)
    plain = run_cpu_ranks(_run, 4, (4, 1, 6, False))
    assert outs[0][3] > plain[0][3]                     # two more exchanges per layer inside the KV groups


def _split_cache_rows(rank, world):
    e = InferenceEngine.build("tiny", tp=4, rank=rank, world=world, weights="fp32", max_seq=127, kv_seq_split=True)
    e.prefill(PROMPT)
    return tuple(e.cache.k.shape), int((e.cache.k[0, 0].abs().sum(-1) > 0).sum()), e.cfg.parallel.kv_share


def test_kv_split_cache_holds_every_second_row():
    for rank, (shape, written, share) in enumerate(run_cpu_ranks(_split_cache_rows, 4, ())):
        assert share == 2 and shape[2] == 64                               # ceil(127 / 2) rows instead of 127
        assert written == len(PROMPT) // 2                                 # 32 prompt rows: 16 per rank of a pair


def _tree_window(rank, world, tp, kv_seq_split):
    e = InferenceEngine.build("tiny", tp=tp, rank=rank, world=world, weights="fp32", max_seq=128, kv_seq_split=kv_seq_split)
    e.prefill(PROMPT)
    # a 5-node token tree behind the prompt: node 0 is the root, 1 and 2 its children, 3 a child of 1, 4 a child of 2
    parents = [-1, 0, 0, 1, 2]
    mask = torch.zeros(5, 5, dtype=torch.bool)
    depth = []
    for i, p in enumerate(parents):
        j, d = i, 0
        while j >= 0:
            mask[i, j] = True
            j, d = parents[j], d + 1
        depth.append(d - 1)
    start = e.cache.len
    toks = torch.tensor([5, 9, 11, 3, 7])
    with torch.no_grad():
        logits = e.model.forward(toks, e.cache, positions=start + torch.tensor(depth), tree_mask=mask, commit=False)
    return logits.clone(), e.cache.len


def test_tree_verify_window_with_split_kv_rows():
    """A verify window over a token tree (explicit visibility mask, nothing committed) through the split-KV groups."""
    ref_logits, ref_len = _tree_window(0, 1, 1, False)
    for logits, n in run_cpu_ranks(_tree_window, 4, (4, True)):
        assert n == ref_len == len(PROMPT)
        assert torch.allclose(logits, ref_logits, atol=5e-4, rtol=1e-4)


def _fp8_kv_logits(rank, world, split):
    e = InferenceEngine.build("tiny", tp=4, rank=rank, world=world, weights="fp32", kv="fp8", max_seq=128, kv_seq_split=split)
    return e.prefill(PROMPT, return_logits=True).logits[0].clone()


def test_split_kv_rows_with_an_e4m3_cache_match_the_replicated_e4m3_cache():
    """The row split stores the same quantised rows (one scale per row), only on different ranks. The merge sums in
    another order, and a 1e-7 difference in a later layer's K / V can move an element across an e4m3 rounding boundary,
    so the logits agree to a few 1e-4 rather than to fp32 round-off; a wrong row, scale or merge would be off by 1e-1."""
    rep = run_cpu_ranks(_fp8_kv_logits, 4, (False,))
    spl = run_cpu_ranks(_fp8_kv_logits, 4, (True,))
    for a, b in zip(rep, spl):
        assert float((a - b).abs().max()) < 5e-3 * max(1.0, float(a.abs().max()))
