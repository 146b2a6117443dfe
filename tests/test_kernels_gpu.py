"""sm_100a kernels against plain PyTorch fp32 references of the same ops (needs a B200)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from inferencehackathon_b200.models.quant import QWeight, quant_block
from inferencehackathon_b200.models.qwen3_moe import apply_rope, rmsnorm, rope_tables, route


def _dev():
    return torch.device("cuda", 0)


def _K():
    from inferencehackathon_b200.ops import lib
    lib.load()
    return lib


def _rand_q(rows, K, fp8, gen, lead=()):
    w = torch.randn(*lead, rows, K, device=_dev(), generator=gen) * 0.02
    return quant_block(w, 128, 128) if fp8 else QWeight(w.to(torch.bfloat16))


def _state(n=16):
    d = _dev()
    return dict(counter=torch.zeros(n, dtype=torch.int32, device=d), err=torch.zeros(1, dtype=torch.int32, device=d),
                epoch=torch.zeros(1, dtype=torch.int32, device=d))


@pytest.mark.parametrize("fp8", [True, False])
@pytest.mark.parametrize("rows,K", [(1024, 4096), (2048, 2048), (640, 512), (1280, 1024)])
@pytest.mark.parametrize("pdl", [False, True])
def test_gemv_store(fp8, rows, K, pdl):
    lib = _K()
    g = torch.Generator(device=_dev()).manual_seed(rows + K)
    qw = _rand_q(rows, K, fp8, g)
    x = torch.randn(K, device=_dev(), generator=g) * 3.0
    x[5] = 70.0                                        # exercises the fp16 pre-scale
    out = torch.zeros(rows, device=_dev())
    st = _state()
    a = lib.IhbGemvArgs()
    lib.fill_weight(a, qw)
    a.x, a.out, a.epi, a.ks, a.err = x.data_ptr(), out.data_ptr(), lib.EPI_STORE, 1, st["err"].data_ptr()
    for _ in range(2):
        lib.gemv(a, pdl)
    torch.cuda.synchronize()
    ref = qw.dequant() @ x
    assert int(st["err"].item()) == 0
    tol = 2e-3 * float(ref.abs().max()) + 1e-3
    assert float((out - ref).abs().max()) < tol


@pytest.mark.parametrize("fp8,K,ks", [(True, 8192, 2), (True, 1024, 1), (False, 4096, 2), (False, 512, 1)])
def test_gemv_residual_norm_tail(fp8, K, ks):
    lib = _K()
    H = 2048
    g = torch.Generator(device=_dev()).manual_seed(K)
    qw = _rand_q(H, K, fp8, g)
    x = torch.randn(K, device=_dev(), generator=g)
    resid0 = torch.randn(H, device=_dev(), generator=g)
    gamma = 1.0 + 0.1 * torch.randn(H, device=_dev(), generator=g)
    st = _state()
    slots = torch.zeros(2 * ks * H, device=_dev())
    for rep in range(3):                                # epoch parity alternates between calls
        resid = resid0.clone()
        xn = torch.zeros(H, device=_dev())
        a = lib.IhbGemvArgs()
        lib.fill_weight(a, qw)
        a.x, a.epi, a.ks = x.data_ptr(), lib.EPI_AR_NORM, ks
        a.counter, a.err = st["counter"].data_ptr(), st["err"].data_ptr()
        a.resid, a.gamma, a.xn_out, a.eps = resid.data_ptr(), gamma.data_ptr(), xn.data_ptr(), 1e-6
        a.comm = lib.single_comm(slots, st["epoch"])
        lib.gemv(a, False)
        torch.cuda.synchronize()
        ref_r = resid0 + qw.dequant() @ x
        ref_n = rmsnorm(ref_r, gamma, 1e-6)
        assert float((resid - ref_r).abs().max()) < 3e-3
        assert float((xn - ref_n).abs().max()) < 3e-3
        assert int(st["epoch"].item()) == rep + 1 and int(st["counter"][0].item()) == 0
    assert int(st["err"].item()) == 0


@pytest.mark.parametrize("ks", [1, 8])
@pytest.mark.parametrize("E,k", [(128, 8), (16, 4)])
def test_router_tail(E, k, ks):
    lib = _K()
    H = 2048
    g = torch.Generator(device=_dev()).manual_seed(E)
    wr = (torch.randn(E, H, device=_dev(), generator=g) * 0.1).to(torch.bfloat16)
    x = torch.randn(H, device=_dev(), generator=g)
    logits = torch.zeros(E, device=_dev())
    sel_idx = torch.zeros(k, dtype=torch.int32, device=_dev())
    sel_w = torch.zeros(k, device=_dev())
    st = _state()
    a = lib.IhbGemvArgs()
    lib.fill_weight(a, QWeight(wr))
    a.x, a.out, a.epi, a.ks = x.data_ptr(), logits.data_ptr(), lib.EPI_ROUTER, ks
    part = torch.zeros(ks * E, device=_dev())
    a.router_partial = part.data_ptr()
    a.counter, a.err = st["counter"].data_ptr(), st["err"].data_ptr()
    a.top_k, a.renorm, a.sel_idx, a.sel_w = k, 1, sel_idx.data_ptr(), sel_w.data_ptr()
    lib.gemv(a, False)
    torch.cuda.synchronize()
    idx, w, ref_logits = route(x[None], wr, k, True)
    assert float((logits - ref_logits[0]).abs().max()) < 2e-3
    assert sel_idx.tolist() == idx[0].tolist()
    assert float((sel_w - w[0]).abs().max()) < 1e-4


@pytest.mark.parametrize("fp8", [True, False])
def test_lm_head_argmax(fp8):
    lib = _K()
    V, H = 18992, 2048
    g = torch.Generator(device=_dev()).manual_seed(7)
    qw = _rand_q(V, H, fp8, g)
    x = torch.randn(H, device=_dev(), generator=g)
    st = _state()
    i32 = dict(dtype=torch.int32, device=_dev())
    cur, pos, ring = torch.zeros(1, **i32), torch.full((1,), 5, **i32), torch.zeros(64, **i32)
    forced, nforced = torch.zeros(64, **i32), torch.zeros(1, **i32)
    part = torch.zeros(1024, dtype=torch.int64, device=_dev())
    logits = torch.zeros(V, device=_dev())
    a = lib.IhbGemvArgs()
    lib.fill_weight(a, qw)
    a.x, a.out, a.epi, a.ks = x.data_ptr(), logits.data_ptr(), lib.EPI_ARGMAX, 1
    a.counter, a.err = st["counter"].data_ptr(), st["err"].data_ptr()
    a.argmax_partial, a.vocab0, a.cur_token, a.pos = part.data_ptr(), 100, cur.data_ptr(), pos.data_ptr()
    a.token_ring, a.token_ring_size, a.forced, a.n_forced = ring.data_ptr(), 64, forced.data_ptr(), nforced.data_ptr()
    a.comm = lib.single_comm(torch.zeros(4, device=_dev()), st["epoch"])
    lib.gemv(a, False)
    torch.cuda.synchronize()
    assert int(cur.item()) == int(logits.argmax().item()) + 100
    assert int(pos.item()) == 6 and int(ring[5].item()) == int(cur.item())
    ref = qw.dequant() @ x
    assert float((logits - ref).abs().max()) < 3e-3
    assert abs(float(ref.max()) - float(logits.max())) < 3e-3


@pytest.mark.parametrize("fp8", [True, False])
@pytest.mark.parametrize("H,I,E,k", [(4096, 1536, 8, 8), (2048, 192, 16, 8), (512, 256, 16, 4), (2048, 768, 8, 8),
                                     (2048, 96, 8, 8)])
def test_moe_gateup_down(fp8, H, I, E, k):
    if not fp8 and H > 2048:
        pytest.skip("bf16 activations of this width do not fit the register fragment")
    lib = _K()
    g = torch.Generator(device=_dev()).manual_seed(H + I)
    wgu = _rand_q(2 * I, H, fp8, g, lead=(E,))
    wd = _rand_q(H, I, fp8, g, lead=(E,))
    x = torch.randn(H, device=_dev(), generator=g)
    sel = torch.randperm(E, device=_dev(), generator=g)[:k].to(torch.int32)
    sw = torch.softmax(torch.randn(k, device=_dev(), generator=g), 0)
    resid0 = torch.randn(H, device=_dev(), generator=g)
    gamma = 1.0 + 0.1 * torch.randn(H, device=_dev(), generator=g)
    resid, xn = resid0.clone(), torch.zeros(H, device=_dev())
    act = torch.zeros(k * I, device=_dev())
    st = _state()
    slots = torch.zeros(2 * H, device=_dev())
    a = lib.IhbMoeArgs()
    a.Wgu, a.Wd, a.wtype = wgu.data.data_ptr(), wd.data.data_ptr(), lib.wtype_of(wgu.data)
    a.H, a.I, a.E_local, a.expert0, a.top_k = H, I, E, 0, k
    if fp8:
        gsc, dsc = lib.kernel_scale(wgu), lib.kernel_scale(wd)
        a.gu_scale, a.d_scale = gsc.data_ptr(), dsc.data_ptr()
        a.gu_rb, a.gu_kb_shift, a.gu_nkb = wgu.rb, lib.kb_shift_of(wgu.kb), gsc.shape[-1]
        a.d_rb, a.d_kb_shift, a.d_nkb = wd.rb, lib.kb_shift_of(wd.kb), dsc.shape[-1]
    a.x, a.sel_idx, a.sel_w, a.act = x.data_ptr(), sel.data_ptr(), sw.data_ptr(), act.data_ptr()
    a.counter, a.err = st["counter"].data_ptr(), st["err"].data_ptr()
    a.resid, a.gamma, a.xn_out, a.eps = resid.data_ptr(), gamma.data_ptr(), xn.data_ptr(), 1e-6
    a.comm = lib.single_comm(slots, st["epoch"])
    lib.moe_gateup(a, False)
    lib.moe_down(a, False)
    torch.cuda.synchronize()
    assert int(st["err"].item()) == 0
    y = torch.zeros(H, device=_dev())
    acts = []
    for s in range(k):
        e = int(sel[s])
        gu = wgu.select(e).dequant() @ x
        aa = torch.nn.functional.silu(gu[:I]) * gu[I:]
        acts.append(aa)
        y += sw[s] * (wd.select(e).dequant() @ aa)
    ref_act = torch.cat(acts)
    assert float((act - ref_act).abs().max()) < 2e-3 * max(1.0, float(ref_act.abs().max()))
    ref_r = resid0 + y
    assert float((resid - ref_r).abs().max()) < 3e-3
    assert float((xn - rmsnorm(ref_r, gamma, 1e-6)).abs().max()) < 3e-3


@pytest.mark.parametrize("nq,nkv", [(8, 1), (16, 1), (64, 4), (8, 2), (4, 4)])
@pytest.mark.parametrize("ctx", [1, 77, 1024, 3000])
def test_rope_kv_and_flash_decode(nq, nkv, ctx):
    lib = _K()
    max_seq = 4096
    d = _dev()
    g = torch.Generator(device=d).manual_seed(nq * 1000 + ctx)
    kc = (torch.randn(nkv, max_seq, 128, device=d, generator=g)).to(torch.bfloat16)
    vc = (torch.randn(nkv, max_seq, 128, device=d, generator=g)).to(torch.bfloat16)
    qkv = torch.randn((nq + 2 * nkv) * 128, device=d, generator=g)
    qg = 1.0 + 0.1 * torch.randn(128, device=d, generator=g)
    kg = 1.0 + 0.1 * torch.randn(128, device=d, generator=g)
    pos = torch.tensor([ctx - 1], dtype=torch.int32, device=d)
    cos, sin = rope_tables(torch.arange(max_seq, device=d), 128, 1e6)
    cos, sin = cos.contiguous(), sin.contiguous()
    raw = qkv.clone()
    lib.qk_norm_rope_kv(qkv, nq, nkv, qg, kg, 1e-6, cos, sin, pos, kc, vc, max_seq, False)
    nsplit = 5
    scratch = torch.zeros(lib.flash_decode_scratch_floats(nq, nsplit), device=d)
    ctrs = torch.zeros(nq, dtype=torch.int32, device=d)
    out = torch.zeros(nq * 128, device=d)
    out_q = torch.zeros(nq * 128, dtype=torch.uint8, device=d)
    out_s = torch.zeros(nq, device=d)
    for _ in range(2):
        lib.flash_decode(qkv, kc, vc, nq, nkv, max_seq, pos, nsplit, scratch, ctrs, out, False, out_q, out_s, True)
    torch.cuda.synchronize()
    # reference
    q = raw[: nq * 128].reshape(1, nq, 128)
    k = raw[nq * 128:(nq + nkv) * 128].reshape(1, nkv, 128)
    v = raw[(nq + nkv) * 128:].reshape(1, nkv, 128)
    c1, s1 = cos[ctx - 1: ctx], sin[ctx - 1: ctx]
    qr = apply_rope(rmsnorm(q, qg, 1e-6), c1, s1)
    kr = apply_rope(rmsnorm(k, kg, 1e-6), c1, s1)
    assert float((qkv[: nq * 128].reshape(1, nq, 128) - qr).abs().max()) < 1e-4
    assert float((kc[:, ctx - 1].float() - kr[0].to(torch.bfloat16).float()).abs().max()) < 2e-2
    assert torch.equal(vc[:, ctx - 1], v[0].to(torch.bfloat16))
    kf, vf = kc[:, :ctx].float(), vc[:, :ctx].float()
    gq = nq // nkv
    qh = qkv[: nq * 128].reshape(nkv, gq, 128)
    sc = torch.einsum("kgd,ksd->kgs", qh, kf) / math.sqrt(128)
    ref = torch.einsum("kgs,ksd->kgd", torch.softmax(sc, -1), vf).reshape(-1)
    assert float((out - ref).abs().max()) < 2e-3
    assert int(ctrs.sum().item()) == 0
    deq = (out_q.view(torch.float8_e4m3fn).float().reshape(nq, 128) * out_s[:, None]).reshape(-1)
    assert float((deq - out).abs().max()) <= 0.07 * float(out.abs().max()) + 1e-6


def _fp8_rows(x):
    """x [..., 128] fp32 -> (e4m3 bytes as uint8, scale [...] fp32): one scale per row = amax / 448."""
    s = x.abs().amax(-1, keepdim=True).clamp_min(1e-12) / 448.0
    q = (x / s).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).contiguous(), s[..., 0].contiguous()


@pytest.mark.parametrize("nq,nkv", [(8, 1), (64, 4), (8, 2), (4, 4)])
@pytest.mark.parametrize("ctx", [1, 77, 1024, 3000])
def test_rope_kv_and_flash_decode_on_an_e4m3_cache(nq, nkv, ctx):
    """The append writes the new K / V rows as e4m3 bytes with amax / 448 as the row's scale; flash decode over that cache
    matches fp32 attention over the de-quantised rows."""
    lib = _K()
    max_seq = 4096
    d = _dev()
    g = torch.Generator(device=d).manual_seed(nq * 1000 + ctx + 7)
    kc, ks = _fp8_rows(torch.randn(nkv, max_seq, 128, device=d, generator=g) * 2.0)
    vc, vs = _fp8_rows(torch.randn(nkv, max_seq, 128, device=d, generator=g) * 0.5)
    qkv = torch.randn((nq + 2 * nkv) * 128, device=d, generator=g)
    qg = 1.0 + 0.1 * torch.randn(128, device=d, generator=g)
    kg = 1.0 + 0.1 * torch.randn(128, device=d, generator=g)
    pos = torch.tensor([ctx - 1], dtype=torch.int32, device=d)
    cos, sin = rope_tables(torch.arange(max_seq, device=d), 128, 1e6)
    cos, sin = cos.contiguous(), sin.contiguous()
    raw = qkv.clone()
    before_k, before_v = kc.clone(), vc.clone()
    lib.qk_norm_rope_kv(qkv, nq, nkv, qg, kg, 1e-6, cos, sin, pos, kc, vc, max_seq, False, k_scale=ks, v_scale=vs)
    nsplit = 5
    scratch = torch.zeros(lib.flash_decode_scratch_floats(nq, nsplit), device=d)
    ctrs = torch.zeros(nq, dtype=torch.int32, device=d)
    out = torch.zeros(nq * 128, device=d)
    for _ in range(2):
        lib.flash_decode(qkv, kc, vc, nq, nkv, max_seq, pos, nsplit, scratch, ctrs, out, False, k_scale=ks, v_scale=vs)
    torch.cuda.synchronize()
    # the appended rows: only row ctx - 1 changed; its scale is amax / 448 and its bytes decode to the row within e4m3's step
    k = raw[nq * 128:(nq + nkv) * 128].reshape(1, nkv, 128)
    v = raw[(nq + nkv) * 128:].reshape(nkv, 128)
    kr = apply_rope(rmsnorm(k, kg, 1e-6), cos[ctx - 1: ctx], sin[ctx - 1: ctx])[0]
    keep = torch.ones(max_seq, dtype=torch.bool, device=d)
    keep[ctx - 1] = False
    assert torch.equal(kc[:, keep], before_k[:, keep]) and torch.equal(vc[:, keep], before_v[:, keep])
    for cache, scale, want in ((kc, ks, kr), (vc, vs, v)):
        amax = want.abs().amax(-1)
        assert float((scale[:, ctx - 1] - amax / 448.0).abs().max()) <= 1e-5 * float(amax.max() / 448.0) + 1e-12
        deq = cache[:, ctx - 1].view(torch.float8_e4m3fn).float() * scale[:, ctx - 1, None]
        assert float(((deq - want).abs() - 0.0625 * want.abs()).max()) <= float(amax.max()) * 2e-3
    kf = kc[:, :ctx].view(torch.float8_e4m3fn).float() * ks[:, :ctx, None]
    vf = vc[:, :ctx].view(torch.float8_e4m3fn).float() * vs[:, :ctx, None]
    qh = qkv[: nq * 128].reshape(nkv, nq // nkv, 128)
    sc = torch.einsum("kgd,ksd->kgs", qh, kf) / math.sqrt(128)
    ref = torch.einsum("kgs,ksd->kgd", torch.softmax(sc, -1), vf).reshape(-1)
    assert float((out - ref).abs().max()) < 2e-3
    assert int(ctrs.sum().item()) == 0


def test_embed_norm_quantised_copy():
    lib = _K()
    d = _dev()
    H, V = 2048, 1000
    g = torch.Generator(device=d).manual_seed(5)
    emb = (torch.randn(V, H, device=d, generator=g)).to(torch.bfloat16)
    gamma = 1.0 + 0.1 * torch.randn(H, device=d, generator=g)
    tok = torch.tensor([123], dtype=torch.int32, device=d)
    resid, xn = torch.zeros(H, device=d), torch.zeros(H, device=d)
    xq, xs = torch.zeros(H, dtype=torch.uint8, device=d), torch.zeros(H // 128, device=d)
    lib.embed_norm(emb, tok, gamma, 1e-6, resid, xn, False, xq, xs, True)
    xb = torch.zeros(2 * H, dtype=torch.uint8, device=d)
    lib.embed_norm(emb, tok, gamma, 1e-6, resid, xn, False, xb, None, False)
    torch.cuda.synchronize()
    ref = rmsnorm(emb[123].float(), gamma, 1e-6)
    assert torch.equal(resid, emb[123].float())
    assert float((xn - ref).abs().max()) < 1e-4
    q2, s2 = lib.act_row(xn, True)
    assert float((xs - s2).abs().max()) < 1e-6
    deq = (xq.view(torch.float8_e4m3fn).float().reshape(-1, 128) * xs[:, None]).reshape(-1)
    assert float((deq - xn).abs().max()) <= 0.07 * float(xn.abs().max())
    assert torch.equal(xb.view(torch.bfloat16), xn.to(torch.bfloat16))


@pytest.mark.parametrize("payload", ["fp32", "bf16"])
def test_counted_allreduce_single_rank_adds_residual_and_norms(payload):
    """With one rank the counted small-message all-reduce is residual add + RMSNorm through the 64-bit fixed-point
    slots: the result must match the fp32 formula to the slot's resolution (2^-28), on every one of the four call
    parities and again after they wrap."""
    from inferencehackathon_b200.ops import lib
    lib.load()
    d = _dev()
    T, H = 5, 4096
    g = torch.Generator(device=d).manual_seed(3)
    slots = torch.zeros(4 * 64 * H, dtype=torch.int64, device=d)
    epoch = torch.zeros(4, dtype=torch.int32, device=d)
    cm = lib.single_comm(slots, epoch)
    counter = torch.zeros(8, dtype=torch.int32, device=d)
    calls = torch.zeros(64, dtype=torch.int32, device=d)
    err = torch.zeros(1, dtype=torch.int32, device=d)
    gamma = torch.rand(H, device=d, generator=g) + 0.5
    for it in range(9):
        T = (5, 2, 7)[it % 3]                            # the number of rows may change from call to call
        x = torch.randn(T, H, device=d, generator=g) * (1 + it)
        if payload == "bf16":
            x = x.to(torch.bfloat16)
        resid = torch.randn(T, H, device=d, generator=g)
        out, outn = torch.empty(T, H, device=d), torch.empty(T, H, device=d)
        outb = torch.empty(T, H, device=d, dtype=torch.bfloat16)
        lib.allreduce_counted(cm, x, out, counter, calls, err, resid=resid, gamma=gamma, out_norm=outn,
                              out_norm_bf16=outb if it % 2 == 0 else None)
        ref = x.float() + resid
        refn = ref * torch.rsqrt(ref.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma
        assert float((out - ref).abs().max()) < 4e-6 * (1 + it)
        assert float((outn - refn).abs().max()) < 1e-5
        if it % 2 == 0:                                  # the bf16 copy is the fp32 normed row, rounded to nearest
            assert torch.equal(outb, outn.to(torch.bfloat16))
    assert int(err.item()) == 0 and calls[:8].tolist() == [9, 9, 6, 6, 6, 3, 3, 0]
    assert int(slots.abs().max()) == 0                   # every reader cleared what it consumed
