"""Reference model: parameter accounting, layout invariants, KV-cache consistency (CPU)."""
import torch

from inferencehackathon_b200 import TINY, QWEN3_235B_A22B, QWEN3_30B_A3B, ParallelConfig, QuantConfig
from inferencehackathon_b200.models.qwen3_moe import Qwen3MoE
from inferencehackathon_b200.models.weights import random_state_dict, shard_state_dict, shard_geometry
from inferencehackathon_b200.runtime.engine import InferenceEngine


def test_param_counts():
    assert 234e9 < QWEN3_235B_A22B.total_params() < 236e9
    assert 21e9 < QWEN3_235B_A22B.active_params() < 23e9
    assert 30e9 < QWEN3_30B_A3B.total_params() < 31e9


def test_geometry_tp8_replicates_kv():
    g = shard_geometry(QWEN3_235B_A22B, ParallelConfig(tp=8, rank=5, world=8))
    assert (g.nq_local, g.nkv_local, g.kv_head0, g.inter_local) == (8, 1, 2, 192)
    assert g.vocab_local == 18992
    g = shard_geometry(QWEN3_235B_A22B, ParallelConfig(tp=2, ep=8, rank=5, world=8))
    assert (g.nq_local, g.nkv_local, g.n_experts_local, g.expert0, g.inter_local) == (32, 2, 16, 80, 1536)


def test_incremental_decode_matches_full_prefill():
    sd = random_state_dict(TINY, 0)
    w = shard_state_dict(sd, TINY, ParallelConfig(), QuantConfig("fp32", kv="fp32"))
    m = Qwen3MoE(w)
    toks = torch.randint(0, TINY.vocab, (12,), generator=torch.Generator().manual_seed(1))
    c1 = m.new_cache(32)
    full = m.forward(toks, c1)
    c2 = m.new_cache(32)
    m.forward(toks[:8], c2)
    outs = [m.forward(toks[i:i + 1], c2) for i in range(8, 12)]
    inc = torch.cat(outs)
    assert torch.allclose(full[8:], inc, atol=2e-4, rtol=1e-4)


def test_generate_greedy_deterministic():
    e = InferenceEngine.build("tiny", weights="fp32", max_seq=128)
    prompt = torch.randint(0, TINY.vocab, (32,), generator=torch.Generator().manual_seed(0)).tolist()
    a = e.generate(prompt, 16)
    b = e.generate(prompt, 16)
    assert a.tokens == b.tokens and len(a.tokens) == 16
    assert len(a.routes[1]) == TINY.n_layers and len(a.routes[1][0].experts) == TINY.top_k
    assert abs(sum(a.routes[1][0].weights) - 1.0) < 1e-5


def test_fp8_block_weights_close_to_fp32():
    sd = random_state_dict(TINY, 0)
    w32 = shard_state_dict(sd, TINY, ParallelConfig(), QuantConfig("fp32", kv="fp32"))
    w8 = shard_state_dict(sd, TINY, ParallelConfig(), QuantConfig("fp8_block", kv="fp32"))
    a, b = w32.layers[0].wqkv.dequant(), w8.layers[0].wqkv.dequant()
    assert w8.layers[0].wqkv.is_fp8 and (a - b).abs().max() < 0.07 * a.abs().max()
    toks = torch.arange(8)
    m32, m8 = Qwen3MoE(w32), Qwen3MoE(w8)
    l32, l8 = m32.forward(toks, m32.new_cache(16)), m8.forward(toks, m8.new_cache(16))
    assert torch.nn.functional.cosine_similarity(l32.flatten(), l8.flatten(), dim=0) > 0.98


def test_fp8_kv_cache_on_the_pytorch_path_tracks_the_fp32_cache():
    import torch
    from inferencehackathon_b200.runtime.engine import InferenceEngine
    prompt = torch.randint(0, 2048, (24,), generator=torch.Generator().manual_seed(2)).tolist()
    ref = InferenceEngine.build("tiny", device="cpu", backend="torch", max_seq=64, kv="fp32")
    q8 = InferenceEngine.build("tiny", device="cpu", backend="torch", max_seq=64, kv="fp8")
    assert q8.cache.fp8 and q8.cache.k.dtype == torch.float8_e4m3fn
    la = ref.prefill(prompt, return_logits=True).logits.float()
    lb = q8.prefill(prompt, return_logits=True).logits.float()
    scale = float(la.abs().max())
    assert float((la - lb).abs().max()) < 0.05 * scale            # e4m3 rows: ~2^-4 relative steps, averaged by the softmax
    a = ref.generate(prompt, 8).tokens
    b = q8.generate(prompt, 8).tokens
    assert sum(int(x == y) for x, y in zip(a, b)) >= 6


def test_partial_attention_records_merge_to_full_attention():
    """Attention over disjoint row sets, returned as (acc, m, l) records and merged, equals attention over all rows:
    causal and with a tree mask, including a query that sees no row of one set."""
    from inferencehackathon_b200.models.qwen3_moe import _attention, _attention_partial, _merge_partials
    g = torch.Generator().manual_seed(5)
    T, nh, hd, start = 5, 4, 32, 9
    S = start + T
    q = torch.randn(T, nh, hd, generator=g)
    kc, vc = torch.randn(1, S, hd, generator=g), torch.randn(1, S, hd, generator=g)
    positions = torch.arange(start, S)
    for mask in (None, torch.tril(torch.ones(T, T, dtype=torch.bool)) & (torch.rand(T, T, generator=g) < 0.7)
                 | torch.eye(T, dtype=torch.bool)):
        want = _attention(q, kc, vc, positions, mask).reshape(T, nh, hd)
        visible = torch.arange(S)[None, :] <= positions[:, None]
        if mask is not None:
            visible = visible.clone()
            visible[:, start:] = mask
        for share in (2, 3):
            parts = []
            for me in range(share):
                rows = torch.arange(me, S, share)
                parts.append(_attention_partial(q, kc[0, rows], vc[0, rows], visible[:, rows]))
            assert torch.allclose(_merge_partials(parts), want, atol=1e-5, rtol=1e-5)
    # a set that no query sees, and an empty set, contribute nothing
    none = _attention_partial(q, kc[0, :3], vc[0, :3], torch.zeros(T, 3, dtype=torch.bool))
    assert torch.isinf(none[1]).all() and float(none[2].abs().sum()) == 0.0
    full = _attention_partial(q, kc[0], vc[0], torch.arange(S)[None, :] <= positions[:, None])
    empty = _attention_partial(q, kc[0, :0], vc[0, :0], torch.zeros(T, 0, dtype=torch.bool))
    assert torch.allclose(_merge_partials([full, none, empty]), _attention(q, kc, vc, positions, None).reshape(T, nh, hd),
                          atol=1e-5, rtol=1e-5)


def test_torch_kv_scattered_rows_match_contiguous_writes():
    """``write_rows`` (rows anywhere in the cache) stores what ``write`` stores for the same rows: bf16 and e4m3 + scale."""
    from inferencehackathon_b200.models.qwen3_moe import TorchKV
    g = torch.Generator().manual_seed(1)
    k, v = torch.randn(2, 6, 32, generator=g), torch.randn(2, 6, 32, generator=g)
    for dtype in (torch.bfloat16, torch.float8_e4m3fn):
        a, b = TorchKV(1, 2, 16, 32, dtype, "cpu"), TorchKV(1, 2, 16, 32, dtype, "cpu")
        a.write(0, 3, k, v)
        b.write_rows(0, torch.tensor([3, 4, 5]), k[:, :3], v[:, :3])
        b.write_rows(0, torch.tensor([8, 6, 7]), k[:, [5, 3, 4]], v[:, [5, 3, 4]])       # any order
        b.write_rows(0, torch.tensor([], dtype=torch.long), k[:, :0], v[:, :0])          # nothing to write
        ka, va = a.read(0, 9)
        kb, vb = b.read(0, 9)
        assert torch.equal(ka.float(), kb.float()) and torch.equal(va.float(), vb.float())


from hypothesis import given, settings, strategies as st   # noqa: E402


@settings(max_examples=80, deadline=None)
@given(st.integers(2, 40), st.sampled_from([0.0, 0.2, 1.0, 3.0]), st.integers(0, 12), st.sampled_from([1.0, 0.9, 0.5, 0.05]),
       st.integers(0, 2 ** 31 - 1))
def test_sampler_distribution_invariants(vocab, temperature, top_k, top_p, seed):
    """For any logits and settings: the distribution sums to one, greedy is a point mass on the arg-max, top-k keeps at
    most k tokens (the k largest), top-p keeps the smallest prefix of the sorted distribution whose mass reaches p, and
    a draw always comes from the support."""
    from inferencehackathon_b200.runtime.sampler import Sampler, SamplingParams
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(vocab, generator=g) * 3
    s = Sampler(SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p, seed=seed))
    p = s.probs(logits)
    assert p.shape == logits.shape and abs(float(p.sum()) - 1.0) < 1e-5 and float(p.min()) >= 0.0
    support = set(torch.nonzero(p).flatten().tolist())
    if temperature <= 0.0:
        assert support == {int(logits.argmax())}
    else:
        if top_k and top_k < vocab:
            assert support <= set(torch.topk(logits, top_k).indices.tolist())           # random logits have no ties
        if top_p < 1.0:
            ref = Sampler(SamplingParams(temperature=temperature, top_k=top_k, top_p=1.0)).probs(logits)
            sp_, si = torch.sort(ref, descending=True)
            before = sp_.cumsum(0) - sp_
            assert support == set(si[before < top_p].tolist())
        assert int(logits.argmax()) in support
    assert int(s.sample(logits)) in support


@settings(max_examples=60, deadline=None)
@given(st.text(alphabet=st.characters(min_codepoint=32, max_codepoint=126), min_size=0, max_size=40),
       st.sampled_from([256, 2048, 151936]))
def test_byte_tokenizer_round_trips_printable_text(text, vocab):
    from inferencehackathon_b200.serve.tokenizer import ByteTokenizer
    tok = ByteTokenizer(vocab)
    ids = tok.encode(text)
    assert ids and all(0 <= i < vocab for i in ids)
    if text:
        assert tok.decode(ids) == text
    # ids outside the printable range still map to distinct readable pieces
    pieces = {tok.piece(i) for i in (0, 5, 127, 200, vocab - 1)}
    assert len(pieces) == len({0, 5, 127, 200, vocab - 1})
