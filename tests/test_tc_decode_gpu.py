"""Single-token tcgen05 linear layers with fused epilogues against PyTorch fp32 references (needs a B200)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from inferencehackathon_b200.models.quant import QWeight, quant_block
from inferencehackathon_b200.models.qwen3_moe import rmsnorm


def _dev():
    return torch.device("cuda", 0)


def _K():
    from inferencehackathon_b200.ops import lib
    lib.load()
    return lib


def _weights(rows, K, fp8, gen, lead=()):
    w = torch.randn(*lead, rows, K, device=_dev(), generator=gen) * 0.05
    return quant_block(w, 128, 128) if fp8 else QWeight(w.to(torch.bfloat16))


def _deq_act(lib, x, fp8):
    """Kernel-format activation and the fp32 values it represents."""
    q, s = lib.act_row(x, fp8)
    K = x.shape[-1]
    if fp8:
        v = q.view(torch.float8_e4m3fn).float().reshape(*x.shape[:-1], -1, 128) * s[..., None]
        return q, s, v.reshape(*x.shape[:-1], -1)[..., :K]
    return q, None, x.to(torch.bfloat16).float()


def _base(lib, a, d):
    st = dict(err=torch.zeros(1, dtype=torch.int32, device=d), counter=torch.zeros(4, dtype=torch.int32, device=d),
              epoch=torch.zeros(1, dtype=torch.int32, device=d))
    a.err, a.counter = st["err"].data_ptr(), st["counter"].data_ptr()
    st["part"] = torch.zeros(lib.tc_dec_partial_floats(a), device=d)
    st["tc"] = torch.zeros(4096, dtype=torch.int32, device=d)
    a.partial, a.tile_counters = st["part"].data_ptr(), st["tc"].data_ptr()
    return st


@pytest.mark.parametrize("fp8", [True, False])
@pytest.mark.parametrize("rows,K,ks", [(256, 512, 0), (1280, 4096, 0), (9216, 4096, 0), (4096, 8192, 0), (200, 768, 2),
                                       (4096, 192, 0), (640, 2048, 3)])
def test_dec_store(fp8, rows, K, ks):
    lib, d = _K(), _dev()
    g = torch.Generator(device=d).manual_seed(rows + K)
    qw = _weights(rows, K, fp8, g)
    wt = lib.tile_weight_v2(qw.data)
    x = torch.randn(K, device=d, generator=g)
    xq, xs, xf = _deq_act(lib, x, fp8)
    out = torch.full((rows,), float("nan"), device=d)
    a = lib.IhbTcDecArgs()
    lib.tc_dec_fill_weight(a, qw, wt)
    a.X, a.mode, a.epi, a.out, a.ks = xq.data_ptr(), lib.TC_LINEAR, lib.DEC_STORE, out.data_ptr(), ks
    if fp8:
        a.xscale = xs.data_ptr()
    st = _base(lib, a, d)
    for _ in range(2):
        lib.tc_decode(a, False)
    torch.cuda.synchronize()
    assert int(st["err"].item()) == 0
    ref = qw.dequant() @ xf
    assert float((out - ref).abs().max()) < 2e-3 * float(ref.abs().max()) + 1e-3
    assert int(st["tc"].sum().item()) == 0


@pytest.mark.parametrize("fp8", [True, False])
@pytest.mark.parametrize("H,K", [(2048, 1024), (4096, 8192)])
def test_dec_residual_norm_tail(fp8, H, K):
    lib, d = _K(), _dev()
    g = torch.Generator(device=d).manual_seed(H + K)
    qw = _weights(H, K, fp8, g)
    wt = lib.tile_weight_v2(qw.data)
    x = torch.randn(K, device=d, generator=g)
    xq, xs, xf = _deq_act(lib, x, fp8)
    resid0 = torch.randn(H, device=d, generator=g)
    gamma = 1.0 + 0.1 * torch.randn(H, device=d, generator=g)
    slots = torch.zeros(2 * H, device=d)
    a = lib.IhbTcDecArgs()
    lib.tc_dec_fill_weight(a, qw, wt)
    a.X, a.mode, a.epi = xq.data_ptr(), lib.TC_LINEAR, lib.DEC_AR_NORM
    if fp8:
        a.xscale = xs.data_ptr()
    st = _base(lib, a, d)
    for rep in range(3):
        resid, xn = resid0.clone(), torch.zeros(H, device=d)
        oq = torch.zeros(H * (1 if fp8 else 2), dtype=torch.uint8, device=d)
        osc = torch.zeros(H // 128, device=d)
        a.resid, a.gamma, a.xn_out, a.eps = resid.data_ptr(), gamma.data_ptr(), xn.data_ptr(), 1e-6
        a.xq, a.xs = oq.data_ptr(), osc.data_ptr()
        a.comm = lib.single_comm(slots, st["epoch"])
        lib.tc_decode(a, False)
        torch.cuda.synchronize()
        ref_r = resid0 + qw.dequant() @ xf
        ref_n = rmsnorm(ref_r, gamma, 1e-6)
        assert float((resid - ref_r).abs().max()) < 3e-3 * max(1.0, float(ref_r.abs().max()))
        assert float((xn - ref_n).abs().max()) < 3e-3
        eq, es, _ = _deq_act(lib, xn, fp8)
        if fp8:
            assert float((osc - es).abs().max()) < 1e-6
            assert (oq.view(torch.float8_e4m3fn).float() - eq.view(torch.float8_e4m3fn).float()).abs().max() <= \
                0.13 * eq.view(torch.float8_e4m3fn).float().abs().max()
        else:
            assert torch.equal(oq, eq)
        assert int(st["epoch"].item()) == rep + 1
    assert int(st["err"].item()) == 0


@pytest.mark.parametrize("fp8", [True, False])
def test_dec_argmax(fp8):
    lib, d = _K(), _dev()
    V, H = 18992, 2048
    g = torch.Generator(device=d).manual_seed(11)
    qw = _weights(V, H, fp8, g)
    wt = lib.tile_weight_v2(qw.data)
    x = torch.randn(H, device=d, generator=g)
    xq, xs, xf = _deq_act(lib, x, fp8)
    i32 = dict(dtype=torch.int32, device=d)
    cur, pos, ring = torch.zeros(1, **i32), torch.full((1,), 5, **i32), torch.zeros(64, **i32)
    forced, nforced = torch.zeros(64, **i32), torch.zeros(1, **i32)
    part = torch.zeros(1024, dtype=torch.int64, device=d)
    logits = torch.zeros(V, device=d)
    a = lib.IhbTcDecArgs()
    lib.tc_dec_fill_weight(a, qw, wt)
    a.X, a.mode, a.epi, a.out = xq.data_ptr(), lib.TC_LINEAR, lib.DEC_ARGMAX, logits.data_ptr()
    if fp8:
        a.xscale = xs.data_ptr()
    st = _base(lib, a, d)
    a.argmax_partial, a.vocab0, a.cur_token, a.pos = part.data_ptr(), 100, cur.data_ptr(), pos.data_ptr()
    a.token_ring, a.token_ring_size, a.forced, a.n_forced = ring.data_ptr(), 64, forced.data_ptr(), nforced.data_ptr()
    a.comm = lib.single_comm(torch.zeros(4, device=d), st["epoch"])
    lib.tc_decode(a, False)
    torch.cuda.synchronize()
    ref = qw.dequant() @ xf
    assert int(st["err"].item()) == 0
    assert float((logits - ref).abs().max()) < 2e-3 * float(ref.abs().max()) + 1e-3
    assert int(cur.item()) == int(logits.argmax().item()) + 100
    assert int(pos.item()) == 6 and int(ring[5].item()) == int(cur.item())


@pytest.mark.parametrize("fp8", [True, False])
@pytest.mark.parametrize("H,I,E,k", [(1024, 256, 8, 4), (2048, 192, 16, 8), (4096, 1536, 8, 8), (2048, 768, 8, 8)])
def test_dec_moe(fp8, H, I, E, k):
    lib, d = _K(), _dev()
    g = torch.Generator(device=d).manual_seed(H + I)
    wgu = _weights(2 * I, H, fp8, g, lead=(E,))
    wd = _weights(H, I, fp8, g, lead=(E,))
    wgt = lib.tile_weight_v2(wgu.data.reshape(E, 2, I, H))
    wdt = lib.tile_weight_v2(wd.data)
    x = torch.randn(H, device=d, generator=g)
    xq, xs, xf = _deq_act(lib, x, fp8)
    sel = torch.randperm(E, device=d, generator=g)[:k].to(torch.int32)
    sw = torch.softmax(torch.randn(k, device=d, generator=g), 0)
    esize = 1 if fp8 else 2
    nkb_i = (I * esize + 127) // 128
    act_q = torch.zeros(k, nkb_i * 128, dtype=torch.uint8, device=d)
    act_s = torch.zeros(k, nkb_i, device=d)
    a = lib.IhbTcDecArgs()
    lib.tc_dec_fill_weight(a, wgu, wgt, rows=I)
    a.expert0, a.top_k, a.sel_idx, a.sel_w = 0, k, sel.data_ptr(), sw.data_ptr()
    a.X, a.mode, a.epi = xq.data_ptr(), lib.TC_GATEUP, lib.DEC_ACT
    a.act_q, a.act_s = act_q.data_ptr(), act_s.data_ptr()
    if fp8:
        a.xscale = xs.data_ptr()
    st = _base(lib, a, d)
    lib.tc_decode(a, False)
    torch.cuda.synchronize()
    assert int(st["err"].item()) == 0
    ref_act = torch.zeros(k, I, device=d)
    for s in range(k):
        gu = wgu.select(int(sel[s])).dequant() @ xf
        ref_act[s] = torch.nn.functional.silu(gu[:I]) * gu[I:]
    if fp8:
        got = (act_q.view(torch.float8_e4m3fn).float().reshape(k, nkb_i, 128) * act_s[..., None]).reshape(k, -1)[:, :I]
        tol = 0.07 * float(ref_act.abs().max())
    else:
        got = act_q.view(torch.bfloat16).float()[:, :I]
        tol = 0.01 * float(ref_act.abs().max())
    assert float((got - ref_act).abs().max()) < tol
    # down projection consumes the kernel's own activations
    resid0 = torch.randn(H, device=d, generator=g)
    gamma = 1.0 + 0.1 * torch.randn(H, device=d, generator=g)
    resid, xn = resid0.clone(), torch.zeros(H, device=d)
    slots = torch.zeros(2 * H, device=d)
    b = lib.IhbTcDecArgs()
    lib.tc_dec_fill_weight(b, wd, wdt)
    b.expert0, b.top_k, b.sel_idx, b.sel_w = 0, k, sel.data_ptr(), sw.data_ptr()
    b.X, b.mode, b.epi = act_q.data_ptr(), lib.TC_DOWN, lib.DEC_AR_NORM
    if fp8:
        b.xscale = act_s.data_ptr()
    st2 = _base(lib, b, d)
    b.resid, b.gamma, b.xn_out, b.eps = resid.data_ptr(), gamma.data_ptr(), xn.data_ptr(), 1e-6
    b.comm = lib.single_comm(slots, st2["epoch"])
    lib.tc_decode(b, False)
    torch.cuda.synchronize()
    assert int(st2["err"].item()) == 0
    y = torch.zeros(H, device=d)
    for s in range(k):
        y += sw[s] * (wd.select(int(sel[s])).dequant() @ got[s])
    ref_r = resid0 + y
    assert float((resid - ref_r).abs().max()) < 3e-3 * max(1.0, float(ref_r.abs().max()))
    assert float((xn - rmsnorm(ref_r, gamma, 1e-6)).abs().max()) < 3e-3
