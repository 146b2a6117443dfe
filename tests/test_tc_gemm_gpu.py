"""tcgen05 / TMEM / TMA linear layers against PyTorch fp32 references (needs a B200)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from inferencehackathon_b200.models.quant import QWeight, quant_act_per_token, quant_block


def _dev():
    return torch.device("cuda", 0)


def _K():
    from inferencehackathon_b200.ops import lib
    lib.load()
    return lib


def _acts(T, K, fp8, gen, lead=()):
    """Activations in kernel layout: data [*lead, T, K]; fp8 scales [*lead, K/128, T]; and their fp32 values."""
    x = torch.randn(*lead, T, K, device=_dev(), generator=gen)
    if not fp8:
        xb = x.to(torch.bfloat16)
        return xb.contiguous(), None, xb.float()
    flat = x.reshape(-1, K)
    Kp = ((K + 127) // 128) * 128
    pad = torch.nn.functional.pad(flat, (0, Kp - K))
    q, s = quant_act_per_token(pad, 128)                       # q [N, Kp], s [N, Kp/128]
    deq = (q.float().reshape(-1, Kp // 128, 128) * s[..., None]).reshape(-1, Kp)[:, :K]
    q = q[:, :K].contiguous().reshape(*lead, T, K)
    s = s.reshape(*lead, T, Kp // 128).transpose(-1, -2).contiguous()
    return q, s, deq.reshape(*lead, T, K)


def _weights(rows, K, fp8, gen, lead=()):
    w = torch.randn(*lead, rows, K, device=_dev(), generator=gen) * 0.05
    return quant_block(w, 128, 128) if fp8 else QWeight(w.to(torch.bfloat16))


def _common(lib, a, T):
    d = _dev()
    a.T, a.T_total, a.tok0 = T, T, 0
    err = torch.zeros(1, dtype=torch.int32, device=d)
    a.err = err.data_ptr()
    n = lib.tc_partial_floats(a)
    return err, n


def _pad_rows128(x):
    """[.., K] activations as plain rows padded to a multiple of 128 bytes (single-token kernel input)."""
    raw = x.contiguous().view(torch.uint8).reshape(*x.shape[:-1], -1)
    return torch.nn.functional.pad(raw, (0, (-raw.shape[-1]) % 128)).contiguous()


@pytest.mark.parametrize("fp8", [True, False])
@pytest.mark.parametrize("tiled", [False, True])
@pytest.mark.parametrize("rows,K,T,ks", [(256, 512, 1, 1), (1280, 4096, 1, 0), (4096, 1024, 5, 4), (640, 2048, 17, 0),
                                         (200, 768, 40, 2), (512, 4096, 128, 1), (4096, 192, 1, 0)])
def test_tc_linear(fp8, tiled, rows, K, T, ks):
    lib = _K()
    g = torch.Generator(device=_dev()).manual_seed(rows + K + T)
    qw = _weights(rows, K, fp8, g)
    xq, xs, xf = _acts(T, K, fp8, g)
    out = torch.full((T, rows), float("nan"), device=_dev())
    a = lib.IhbTcArgs()
    lib.tc_fill_weight(a, qw)
    a.X, a.mode, a.out, a.out_stride, a.ks = xq.data_ptr(), lib.TC_LINEAR, out.data_ptr(), rows, ks
    if tiled:
        wt = lib.tile_weight(qw.data)
        a.W, a.tiled = wt.data_ptr(), 1
        if T == 1:
            xrow = _pad_rows128(xq[0])
            a.X, a.x_rows1 = xrow.data_ptr(), 1
    if fp8:
        a.xscale = xs.data_ptr()
    a.T, a.T_total, a.tok0 = T, T, 0
    err = torch.zeros(1, dtype=torch.int32, device=_dev())
    a.err = err.data_ptr()
    a.ks = ks if ks else 16                      # upper bound for the workspace; the launcher may pick fewer
    part = torch.zeros(max(1, lib.tc_partial_floats(a)), device=_dev())
    ctrs = torch.zeros((rows + 127) // 128, dtype=torch.int32, device=_dev())
    a.partial, a.tile_counters, a.ks = part.data_ptr(), ctrs.data_ptr(), ks
    for _ in range(2):
        lib.tc_gemm(a, False)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    ref = xf @ qw.dequant().t()
    tol = 2e-3 * float(ref.abs().max()) + 1e-3
    assert float((out - ref).abs().max()) < tol
    assert int(ctrs.sum().item()) == 0


@pytest.mark.parametrize("fp8", [True, False])
@pytest.mark.parametrize("tiled", [False, True])
@pytest.mark.parametrize("H,I,E,k,T", [(1024, 256, 8, 4, 1), (2048, 192, 16, 8, 1), (1024, 768, 8, 8, 3)])
def test_tc_moe_gateup_down(fp8, tiled, H, I, E, k, T):
    lib = _K()
    d = _dev()
    g = torch.Generator(device=d).manual_seed(H + I + T)
    wgu = _weights(2 * I, H, fp8, g, lead=(E,))
    wd = _weights(H, I, fp8, g, lead=(E,))
    xq, xs, xf = _acts(T, H, fp8, g)
    sel = torch.randperm(E, device=d, generator=g)[:k].to(torch.int32)
    sw = torch.softmax(torch.randn(k, device=d, generator=g), 0)
    err = torch.zeros(1, dtype=torch.int32, device=d)
    # gate/up ------------------------------------------------------------------------------------------------
    act = torch.full((k, T, I), float("nan"), device=d)
    a = lib.IhbTcArgs()
    lib.tc_fill_weight(a, wgu)
    a.rows = I
    a.expert0, a.top_k, a.sel_idx, a.sel_w = 0, k, sel.data_ptr(), sw.data_ptr()
    a.X, a.mode, a.out, a.out_stride = xq.data_ptr(), lib.TC_GATEUP, act.data_ptr(), I
    if tiled:
        wgt = lib.tile_weight(wgu.data.reshape(E, 2, I, H))
        a.W, a.tiled = wgt.data_ptr(), 1
        if T == 1:
            xrow = _pad_rows128(xq[0])
            a.X, a.x_rows1 = xrow.data_ptr(), 1
    if fp8:
        a.xscale = xs.data_ptr()
    a.T, a.T_total, a.tok0, a.err = T, T, 0, err.data_ptr()
    a.ks = 16
    part = torch.zeros(max(1, lib.tc_partial_floats(a)), device=d)
    ctrs = torch.zeros(k * ((I + 127) // 128), dtype=torch.int32, device=d)
    a.partial, a.tile_counters, a.ks = part.data_ptr(), ctrs.data_ptr(), 0
    lib.tc_gemm(a, False)
    torch.cuda.synchronize()
    ref_act = torch.zeros(k, T, I, device=d)
    for s in range(k):
        gu = xf @ wgu.select(int(sel[s])).dequant().t()
        ref_act[s] = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    assert int(err.item()) == 0
    assert float((act - ref_act).abs().max()) < 2e-3 * float(ref_act.abs().max()) + 1e-3
    # down -----------------------------------------------------------------------------------------------------
    aq, asc, af = _acts(T, I, fp8, g, lead=(k,))
    out = torch.full((T, H), float("nan"), device=d)
    b = lib.IhbTcArgs()
    lib.tc_fill_weight(b, wd)
    b.expert0, b.top_k, b.sel_idx, b.sel_w = 0, k, sel.data_ptr(), sw.data_ptr()
    b.X, b.mode, b.out, b.out_stride = aq.data_ptr(), lib.TC_DOWN, out.data_ptr(), H
    if tiled:
        wdt = lib.tile_weight(wd.data)
        b.W, b.tiled = wdt.data_ptr(), 1
        if T == 1:
            arow = _pad_rows128(aq[:, 0])
            b.X, b.x_rows1 = arow.data_ptr(), 1
    if fp8:
        b.xscale = asc.data_ptr()
    b.T, b.T_total, b.tok0, b.err = T, T, 0, err.data_ptr()
    b.ks = 16
    part2 = torch.zeros(max(1, lib.tc_partial_floats(b)), device=d)
    ctrs2 = torch.zeros((H + 127) // 128, dtype=torch.int32, device=d)
    b.partial, b.tile_counters, b.ks = part2.data_ptr(), ctrs2.data_ptr(), 0
    lib.tc_gemm(b, False)
    torch.cuda.synchronize()
    ref = torch.zeros(T, H, device=d)
    for s in range(k):
        ref += sw[s] * (af[s] @ wd.select(int(sel[s])).dequant().t())
    assert int(err.item()) == 0
    assert float((out - ref).abs().max()) < 2e-3 * float(ref.abs().max()) + 1e-3


@pytest.mark.parametrize("fp8", [True, False])
@pytest.mark.parametrize("rows,K,T,tile,ks", [(384, 1024, 300, 128, 1), (1152, 4096, 1024, 128, 2), (200, 512, 70, 32, 4)])
def test_tc_linear_over_many_token_tiles_in_one_launch(fp8, rows, K, T, tile, ks):
    """One launch covers all token tiles of a window (units = row tile x token tile x K split)."""
    lib = _K()
    g = torch.Generator(device=_dev()).manual_seed(rows + K + T)
    qw = _weights(rows, K, fp8, g)
    xq, xs, xf = _acts(T, K, fp8, g)
    out = torch.full((T, rows), float("nan"), device=_dev())
    a = lib.IhbTcArgs()
    lib.tc_fill_weight(a, qw)
    a.X, a.mode, a.out, a.out_stride, a.ks = xq.data_ptr(), lib.TC_LINEAR, out.data_ptr(), rows, ks
    if fp8:
        a.xscale = xs.data_ptr()
    a.T, a.T_total, a.tok0 = T, T, 0
    a.tok_tile, a.tok_tiles = tile, -(-T // tile)
    err = torch.zeros(1, dtype=torch.int32, device=_dev())
    a.err = err.data_ptr()
    part = torch.zeros(max(1, lib.tc_partial_floats(a)), device=_dev())
    ctr = torch.zeros(((rows + 127) // 128) * a.tok_tiles, dtype=torch.int32, device=_dev())
    a.partial, a.tile_counters = part.data_ptr(), ctr.data_ptr()
    lib.tc_gemm(a, False)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    ref = xf @ qw.dequant().t()
    assert float((out - ref).abs().max()) < 3e-3 * float(ref.abs().max()) + 1e-3
