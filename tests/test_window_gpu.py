"""Multi-token GPU path (prompt chunks, verify windows, token trees) against the PyTorch reference model (B200)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from inferencehackathon_b200 import SMALL
from inferencehackathon_b200.runtime.engine import InferenceEngine


def _prompt(n, seed=3):
    return torch.randint(0, SMALL.vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _forced_routing(ref, eng):
    """Makes the reference model take the expert choices the engine's device router took in its last window (the
    weights still come from the reference's own logits). A router near-tie can be decided either way by rounding noise
    far below any tolerance, and the flipped expert then moves that token's logits by several per cent: comparing with
    the routing pinned removes that lottery, and the agreement of the free routing is checked on its own. Returns a
    function that restores free routing and reports the share of (layer, token) pairs whose expert SETS agreed."""
    ti, _ = eng.gpu.window().routing()
    ti = ti.clone().long()
    stats = {"same": 0, "all": 0}

    def route_fn(L, h, router_w, top_k, renorm):
        logits = h.float() @ router_w.float().t()
        probs = torch.softmax(logits, -1)
        free = torch.topk(probs, top_k, dim=-1).indices
        idx = ti[L, : h.shape[0]]
        stats["same"] += int((free.sort(-1).values == idx.sort(-1).values).all(-1).sum())
        stats["all"] += h.shape[0]
        w = probs.gather(-1, idx)
        if renorm:
            w = w / w.sum(-1, keepdim=True)
        return idx, w, logits

    ref.model.route_fn = route_fn

    def done():
        ref.model.route_fn = None
        return stats["same"] / max(1, stats["all"])
    return done


def _pair(weights, max_seq=512):
    dev = "cuda:0"
    ref = InferenceEngine.build("small", weights=weights, device=dev, backend="torch", max_seq=max_seq)
    eng = InferenceEngine.build("small", weights=weights, device=dev, backend="cuda", max_seq=max_seq)
    ref.model.act_mode = eng.gpu.window().act_mode       # the oracle rounds activations the way the window GEMMs read them
    return ref, eng


def test_grouped_gemm_matches_per_expert_reference():
    """Device-side group table + grouped tcgen05 GEMM == per-expert matmuls."""
    from inferencehackathon_b200.models.quant import quant_block, quant_act_per_token
    from inferencehackathon_b200.ops import lib as K
    from inferencehackathon_b200.runtime.gpu_window import GpuWindow
    K.load()
    d = torch.device("cuda", 0)
    g = torch.Generator(device=d).manual_seed(0)
    E, rows, Kd, pairs, nt = 8, 384, 512, 50, 16
    w = quant_block(torch.randn(E, rows, Kd, device=d, generator=g) * 0.05, 128, 128)
    flat_e = torch.randint(0, E, (pairs,), device=d, generator=g)
    flat_e[:20] = 3                                              # one expert needs two groups
    order, groups, n_groups, gmax = GpuWindow._group_table(flat_e, E, nt)
    x = torch.randn(pairs, Kd, device=d, generator=g)
    xs_sorted = x[order]
    q, s = quant_act_per_token(xs_sorted, 128)
    deq = (q.float().reshape(pairs, Kd // 128, 128) * s[..., None]).reshape(pairs, Kd)
    sT = s.t().contiguous()
    out = torch.full((pairs, rows), float("nan"), device=d)
    err = torch.zeros(1, dtype=torch.int32, device=d)
    a = K.IhbTcArgs()
    K.tc_fill_weight(a, w)
    a.X, a.xscale, a.mode, a.out, a.out_stride = q.contiguous().data_ptr(), sT.data_ptr(), K.TC_DOWN, out.data_ptr(), rows
    a.T, a.T_total, a.tok0, a.err, a.top_k, a.ks = nt, pairs, 0, err.data_ptr(), 1, 1
    a.groups, a.n_groups, a.max_groups = groups.data_ptr(), n_groups.data_ptr(), gmax
    K.tc_gemm(a, False)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    es = flat_e[order]
    ref = torch.stack([deq[i] @ w.select(int(es[i])).dequant().t() for i in range(pairs)])
    assert float((out - ref).abs().max()) < 2e-3 * float(ref.abs().max()) + 1e-3
    assert int(n_groups.item()) == int(((torch.bincount(flat_e, minlength=E) + nt - 1) // nt).sum())


def test_router_grouping_gather_and_combine_kernels():
    """The device-side routing of a window: fused router (fp32 logits from bf16 rows, softmax, top-k, renormalisation),
    expert group table, dispatch gather and weighted combine, each against plain PyTorch."""
    from inferencehackathon_b200.ops import lib as K
    K.load()
    d = torch.device("cuda", 0)
    g = torch.Generator(device=d).manual_seed(1)
    for (T, H, E, k, renorm) in [(37, 512, 16, 4, True), (300, 2048, 128, 8, True), (9, 1024, 200, 8, False), (3, 512, 16, 4, True),
                                 (20, 520, 64, 8, True), (40, 1024, 200, 8, False)]:
        h = torch.randn(T, H, device=d, generator=g)
        W = (torch.randn(E, H, device=d, generator=g) * 0.05).to(torch.bfloat16)
        ti = torch.zeros(T, k, dtype=torch.int32, device=d)
        tw = torch.zeros(T, k, device=d)
        lg = torch.zeros(T, E, device=d)
        K.router_topk_rows(h, W, k, renorm, ti, tw, lg)
        ref_lg = h @ W.float().t()
        assert float((lg - ref_lg).abs().max()) < 1e-3 * float(ref_lg.abs().max()) + 1e-4
        p = torch.softmax(lg, -1)                                 # selection checked on the kernel's own logits
        rw, ri = torch.topk(p, k, dim=-1)
        if renorm:
            rw = rw / rw.sum(-1, keepdim=True)
        assert torch.equal(ti.long(), ri)
        assert float((tw - rw).abs().max()) < 1e-5
        # group table
        nt = 16
        pairs = T * k
        gmax = E + pairs // nt + 1
        order = torch.full((pairs,), -1, dtype=torch.int32, device=d)
        inv = torch.full((pairs,), -7, dtype=torch.int32, device=d)
        groups = torch.zeros(gmax, 4, dtype=torch.int32, device=d)
        ng = torch.zeros(1, dtype=torch.int32, device=d)
        K.moe_group_table(ti, 0, E, nt, order, inv, groups, ng)
        flat = ti.reshape(-1).long()
        assert sorted(order.tolist()) == list(range(pairs))       # a permutation
        assert torch.equal(inv.long()[order.long()], torch.arange(pairs, device=d))
        n = int(ng.item())
        cnt = torch.bincount(flat, minlength=E)
        assert n == int(((cnt + nt - 1) // nt).sum())
        covered = torch.zeros(pairs, dtype=torch.int32, device=d)
        for e_, r0, nr, _ in groups[:n].tolist():
            assert 1 <= nr <= nt
            assert bool((flat[order[r0:r0 + nr].long()] == e_).all())
            covered[r0:r0 + nr] += 1
        assert bool((covered == 1).all())
        # gather and combine
        rows = torch.randint(0, 255, (T, 64), dtype=torch.uint8, device=d, generator=g)
        out = torch.zeros(pairs, 64, dtype=torch.uint8, device=d)
        K.moe_gather_rows(rows, order, k, out)
        assert torch.equal(out, rows[(order // k).long()])
        yg = torch.randn(pairs, H, device=d, generator=g)
        resid = torch.randn(T, H, device=d, generator=g)
        y = torch.zeros(T, H, device=d)
        K.moe_combine_rows(yg, inv, tw, k, y, resid=resid)
        want = resid + (yg[inv.long()].reshape(T, k, H) * tw[..., None]).sum(1)
        assert float((y - want).abs().max()) < 1e-4
        # expert parallel: a rank that holds experts [e0, e0 + El) keeps only its pairs; the others get inv = -1 and add nothing
        e0, El = E // 2, E - E // 2
        K.moe_group_table(ti, e0, El, nt, order, inv, groups, ng)
        local = (flat >= e0) & (flat < e0 + El)
        n_local = int(local.sum())
        assert sorted(order[:n_local].tolist()) == torch.nonzero(local).reshape(-1).tolist()
        assert bool((inv[~local] == -1).all())
        n = int(ng.item())
        assert n == int(((cnt[e0:] + nt - 1) // nt).sum())
        for e_, r0, nr, _ in groups[:n].tolist():
            assert bool((flat[order[r0:r0 + nr].long()] == e_ + e0).all())
        K.moe_combine_rows(yg, inv, tw, k, y, resid=None)
        sel = torch.where(inv >= 0, inv, torch.zeros_like(inv)).long()
        want = (yg[sel].reshape(T, k, H) * (tw * local.reshape(T, k))[..., None]).sum(1)
        assert float((y - want).abs().max()) < 1e-4


def test_dequant_kernel_matches_the_reference_dequantisation():
    from inferencehackathon_b200.models.quant import quant_block
    from inferencehackathon_b200.ops import lib as K
    K.load()
    d = torch.device("cuda", 0)
    g = torch.Generator(device=d).manual_seed(5)
    for shape, rb, kb in [((3, 200, 512), 128, 128), ((384, 1024), 64, 128), ((2, 130, 192), 1, 256)]:
        w = torch.randn(*shape, device=d, generator=g) * 0.07
        qw = quant_block(w, rb, kb)
        out = torch.zeros(shape, dtype=torch.bfloat16, device=d)
        K.dequant_bf16(qw, out)
        assert torch.equal(out, qw.dequant(torch.bfloat16))


def test_window_scratch_dequantisation_mode(monkeypatch):
    """IHB_WINDOW_BF16_SCRATCH=1: no resident bf16 copies, every layer's weights are de-quantised right before its GEMMs
    (what a model that fills the GPU does); same logits as with resident copies."""
    ref, eng = _pair("fp8_block")
    toks = _prompt(70)
    a = eng.logits_for(toks, commit=True)
    monkeypatch.setenv("IHB_WINDOW_BF16_SCRATCH", "1")
    eng2 = InferenceEngine.build("small", weights="fp8_block", device="cuda:0", backend="cuda", max_seq=512)
    b = eng2.logits_for(toks, commit=True)
    assert not eng2.gpu.window()._resident and eng.gpu.window()._resident
    assert torch.equal(a, b)


def test_window_on_the_block_fp8_gemm_path(monkeypatch):
    """IHB_WINDOW_BF16=0 keeps the block-scaled fp8 GEMMs (per-token e4m3 activations) of the window path alive."""
    monkeypatch.setenv("IHB_WINDOW_BF16", "0")
    ref, eng = _pair("fp8_block")
    assert eng.gpu.window().act_mode == "fp8"
    toks = _prompt(150)
    b = eng.logits_for(toks, commit=True)
    done = _forced_routing(ref, eng)
    a = ref.logits_for(toks, commit=True)
    done()
    # e4m3 activations sit on rounding boundaries: a flipped code in one layer moves later rows a little
    assert float((a - b).abs().max()) < 0.06 * float(a.abs().max())
    eng.gpu.check_error()


@pytest.mark.parametrize("weights", ["bf16", "fp8_block"])
def test_window_logits_match_reference_chain_and_chunks(weights):
    ref, eng = _pair(weights)
    toks = _prompt(150)                                          # two token tiles: 128 + 22
    b = eng.logits_for(toks[:150], commit=True)
    done = _forced_routing(ref, eng)
    a = ref.logits_for(toks[:150], commit=True)
    assert done() > 0.97                                         # the device router agrees with the free reference routing
    assert b.shape == a.shape and eng.seq_len == 150
    scale = float(a.abs().max())
    # with the routing pinned the logits agree closely; block-fp8 weights are multiplied as their bf16 copies (0.2 % per
    # weight on top of the bf16 activation rounding both sides share)
    tol = 0.01 if weights == "bf16" else 0.025
    assert float((a - b).abs().max()) < tol * scale
    assert float((a.argmax(-1) == b.argmax(-1)).float().mean()) > 0.9
    # a second window on top of the cached context
    more = _prompt(9, seed=5)
    b2 = eng.logits_for(more)
    done = _forced_routing(ref, eng)
    a2 = ref.logits_for(more)
    done()
    assert float((a2 - b2).abs().max()) < tol * float(a2.abs().max())
    eng.gpu.check_error()


@pytest.mark.parametrize("weights", ["bf16", "fp8_block"])
def test_window_tree_mask_and_rollback(weights):
    ref, eng = _pair(weights)
    ctx = _prompt(40)
    eng.logits_for(ctx)
    done = _forced_routing(ref, eng)
    ref.logits_for(ctx)
    done()
    # root + 5 nodes: 0 -> {1, 2}, 1 -> {3, 4}, 2 -> {5}
    parent = [0, 0, 0, 1, 1, 2]
    n = len(parent)
    depth = [0, 1, 1, 2, 2, 2]
    mask = torch.zeros(n, n, dtype=torch.bool, device="cuda:0")
    for i in range(n):
        j = i
        while True:
            mask[i, j] = True
            if j == 0:
                break
            j = parent[j]
    toks = _prompt(n, seed=9)
    pos = torch.tensor([40 + dpt for dpt in depth], device="cuda:0")
    b = eng.logits_for(toks, commit=False, tree_mask=mask, positions=pos)
    done = _forced_routing(ref, eng)
    a = ref.logits_for(toks, commit=False, tree_mask=mask, positions=pos)
    done()
    assert eng.seq_len == 40 and ref.seq_len == 40
    assert float((a - b).abs().max()) < (0.01 if weights == "bf16" else 0.025) * float(a.abs().max())
    # node 3's row must equal a plain chain root -> 1 -> 3
    chain = [toks[0], toks[1], toks[3]]
    c = eng.logits_for(chain, commit=False)
    assert float((c[2] - b[3]).abs().max()) < (0.02 if weights == "bf16" else 0.06) * float(b.abs().max())


def test_window_prefill_then_persistent_decode_matches_reference():
    ref, eng = _pair("fp8_block")
    ref.model.act_mode = None if eng.gpu.use_mega else ref.model.act_mode
    prompt = _prompt(64)
    want = ref.generate(prompt, 12)
    pe = eng.prefill(prompt)
    got = [pe.next_token]
    for t in want.tokens[:-1]:                                   # teacher forcing
        got.append(eng.decode_step(t).token_id)
    agree = sum(int(x == y) for x, y in zip(want.tokens, got))
    assert agree >= 9, (want.tokens, got)
    eng.gpu.check_error()


def test_speculative_driver_on_gpu_engine_equals_its_own_greedy():
    """n-gram speculative decoding through the batched verify window emits what the same engine's plain greedy
    window decoding emits."""
    from inferencehackathon_b200.spec.driver import DecodeStop, EngineRunner, Rng, SpecConfig, SpecEngine, ChainDrafterPool
    from inferencehackathon_b200.spec.ngram import NGramDrafter
    eng = InferenceEngine.build("small", weights="bf16", device="cuda:0", backend="cuda", max_seq=512)
    block = _prompt(12, seed=11)
    prompt = block * 3
    r = EngineRunner(eng)
    plain = []
    ctx = list(prompt)
    for _ in range(16):
        row = r.forward_single(ctx[:-1], ctx[-1])
        t = int(row.argmax())
        plain.append(t); ctx.append(t)
    r2 = EngineRunner(eng)
    se = SpecEngine(r2, ChainDrafterPool([NGramDrafter(2)]), SpecConfig(4, SMALL.vocab, 0.0))
    out, tel = se.decode(prompt, DecodeStop(16), Rng(0))
    assert out == plain
    assert r2.forwards <= 16


@pytest.mark.parametrize("T,base,nq,nkv,masked", [(40, 0, 8, 1, False), (130, 77, 16, 2, False), (23, 300, 8, 2, True),
                                                   (16, 0, 4, 1, True), (257, 1000, 8, 1, False), (8, 1000, 8, 1, False),
                                                   (5, 4000, 16, 2, True), (600, 0, 8, 1, False)])
def test_window_attention_tensor_core_tiles_against_fp32(T, base, nq, nkv, masked):
    """Both window attention kernels (tensor-core tiles; one CTA per token) against plain fp32 PyTorch on the same
    bf16 cache rows: cached context + the window's own rows, causal or with an explicit visibility mask."""
    import math
    from inferencehackathon_b200.ops import lib as K
    K.load()
    d = torch.device("cuda", 0)
    g = torch.Generator(device=d).manual_seed(T + base)
    max_seq = base + T + 5
    kc = torch.randn(nkv, max_seq, 128, device=d, generator=g).to(torch.bfloat16)
    vc = torch.randn(nkv, max_seq, 128, device=d, generator=g).to(torch.bfloat16)
    qkv = torch.randn(T, (nq + 2 * nkv) * 128, device=d, generator=g)
    mask = None
    vis = torch.ones(T, base + T, dtype=torch.bool, device=d)
    if masked:
        mask = torch.rand(T, T, device=d, generator=g) < 0.4
        mask |= torch.eye(T, dtype=torch.bool, device=d)                 # a token always sees itself
        vis[:, base:] = mask
    else:
        vis[:, base:] = torch.tril(torch.ones(T, T, dtype=torch.bool, device=d))
    q = qkv[:, : nq * 128].reshape(T, nkv, nq // nkv, 128)
    s = torch.einsum("tkgd,ksd->tkgs", q, kc[:, : base + T].float()) / math.sqrt(128)
    s = s.masked_fill(~vis[:, None, None, :], float("-inf"))
    want = torch.einsum("tkgs,ksd->tkgd", torch.softmax(s, -1), vc[:, : base + T].float()).reshape(T, nq * 128)
    mu8 = mask.to(torch.uint8).contiguous() if mask is not None else None
    scratch = torch.full((K.window_attention_scratch_floats(nq, nkv, T),), float("nan"), device=d)
    for mode, scr in ((0, None), (0, scratch), (1, None)):          # mode 0 with scratch: keys sliced over CTAs + merge
        out = torch.full((T, nq * 128), float("nan"), device=d)
        K.window_attention(qkv, kc, vc, nq, nkv, max_seq, base, mu8, out, mode=mode, scratch=scr)
        torch.cuda.synchronize()
        assert float((out - want).abs().max()) < 2e-3, (mode, scr is not None)


@pytest.mark.gpu
@pytest.mark.parametrize("T,base,nq,nkv,masked", [(8, 1024, 8, 1, False), (16, 300, 64, 4, True), (70, 0, 8, 2, False),
                                                  (128, 40, 16, 1, False)])
def test_window_append_and_attention_on_an_e4m3_cache(T, base, nq, nkv, masked):
    """Window rows appended as e4m3 bytes with a scale per row; the tensor-core tiles over that cache (rows de-quantised
    to bf16 on their way into shared memory) against fp32 PyTorch on the same de-quantised rows."""
    import math
    from inferencehackathon_b200.models.qwen3_moe import apply_rope, rmsnorm, rope_tables
    from inferencehackathon_b200.ops import lib as K
    K.load()
    d = torch.device("cuda", 0)
    g = torch.Generator(device=d).manual_seed(T + base + 11)
    max_seq = base + T + 5

    def fp8_rows(x):
        s = x.abs().amax(-1, keepdim=True).clamp_min(1e-12) / 448.0
        return (x / s).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).contiguous(), s[..., 0].contiguous()

    kc, ks = fp8_rows(torch.randn(nkv, max_seq, 128, device=d, generator=g) * 2.0)
    vc, vs = fp8_rows(torch.randn(nkv, max_seq, 128, device=d, generator=g) * 0.5)
    qkv = torch.randn(T, (nq + 2 * nkv) * 128, device=d, generator=g)
    raw = qkv.clone()
    qg = 1.0 + 0.1 * torch.randn(128, device=d, generator=g)
    kg = 1.0 + 0.1 * torch.randn(128, device=d, generator=g)
    cos, sin = rope_tables(torch.arange(max_seq, device=d), 128, 1e6)
    cos, sin = cos.contiguous(), sin.contiguous()
    pos = torch.arange(base, base + T, dtype=torch.int32, device=d)
    K.qk_norm_rope_rows(qkv, nq, nkv, qg, kg, 1e-6, cos, sin, pos, pos, kc, vc, max_seq, k_scale=ks, v_scale=vs)
    torch.cuda.synchronize()
    # appended rows against the fp32 formula, within e4m3's step
    k_raw = raw[:, nq * 128:(nq + nkv) * 128].reshape(T, nkv, 128)
    v_raw = raw[:, (nq + nkv) * 128:].reshape(T, nkv, 128)
    kr = apply_rope(rmsnorm(k_raw, kg, 1e-6), cos[base: base + T], sin[base: base + T])
    for cache, scale, want in ((kc, ks, kr), (vc, vs, v_raw)):
        want = want.permute(1, 0, 2)                                                   # [nkv, T, 128]
        amax = want.abs().amax(-1)
        assert float((scale[:, base: base + T] - amax / 448.0).abs().max()) <= 1e-5 * float(amax.max() / 448.0) + 1e-12
        deq = cache[:, base: base + T].view(torch.float8_e4m3fn).float() * scale[:, base: base + T, None]
        assert float(((deq - want).abs() - 0.0625 * want.abs()).max()) <= float(amax.max()) * 2e-3
    mask = None
    vis = torch.ones(T, base + T, dtype=torch.bool, device=d)
    if masked:
        mask = torch.rand(T, T, device=d, generator=g) < 0.4
        mask |= torch.eye(T, dtype=torch.bool, device=d)
        vis[:, base:] = mask
    else:
        vis[:, base:] = torch.tril(torch.ones(T, T, dtype=torch.bool, device=d))
    n = base + T
    kf = (kc[:, :n].view(torch.float8_e4m3fn).float() * ks[:, :n, None]).to(torch.bfloat16).float()   # as the kernel stages them
    vf = (vc[:, :n].view(torch.float8_e4m3fn).float() * vs[:, :n, None]).to(torch.bfloat16).float()
    q = qkv[:, : nq * 128].reshape(T, nkv, nq // nkv, 128)
    s = torch.einsum("tkgd,ksd->tkgs", q, kf) / math.sqrt(128)
    s = s.masked_fill(~vis[:, None, None, :], float("-inf"))
    want = torch.einsum("tkgs,ksd->tkgd", torch.softmax(s, -1), vf).reshape(T, nq * 128)
    mu8 = mask.to(torch.uint8).contiguous() if mask is not None else None
    scratch = torch.full((K.window_attention_scratch_floats(nq, nkv, T),), float("nan"), device=d)
    for scr in (None, scratch):                                       # with scratch: keys sliced over CTAs + merge
        out = torch.full((T, nq * 128), float("nan"), device=d)
        K.window_attention(qkv, kc, vc, nq, nkv, max_seq, base, mu8, out, mode=0, scratch=scr, k_scale=ks, v_scale=vs)
        torch.cuda.synchronize()
        assert float((out - want).abs().max()) < 2e-3, scr is not None
