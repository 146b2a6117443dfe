"""Tensor-, expert- and hybrid-parallel runs over gloo must reproduce the single-rank model (CPU, world 2/4)."""
import torch

from inferencehackathon_b200 import TINY
from inferencehackathon_b200.parallel.launch import run_cpu_ranks
from inferencehackathon_b200.runtime.engine import InferenceEngine

PROMPT = torch.randint(0, TINY.vocab, (32,), generator=torch.Generator().manual_seed(0)).tolist()


def _run(rank, world, tp, ep, n_new):
    e = InferenceEngine.build("tiny", tp=tp, ep=ep, rank=rank, world=world, weights="fp32", max_seq=128)
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
