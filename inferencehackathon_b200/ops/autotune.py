"""Launch-configuration sweep for the per-op decode kernels whose host entry points take explicit knobs: the fused
MoE expert GEMVs (rows per tile ``R_gu`` / ``R_d``, ring depth ``S``, grid) and the split-KV flash-decode (number of
splits at a short and a long context), plus the flatness in M of the verify / window attention. It reports, per configuration, the time and the effective HBM bandwidth, and
the best configuration next to what the kernels' own rule picks when the knob is left at 0 -- the check that the
built-in rules are not leaving bandwidth on the table. Same role as the reference's stand-alone autotuner
(kernels/autotune.cu: threads x grid for the expert kernels, splits for flash-decode at ctx 4096 / 32768).

    python -m inferencehackathon_b200.ops.autotune [--tp 8] [--weights fp8_block|bf16] [--iters 50] [--out FILE.json]
    python -m inferencehackathon_b200.ops.autotune --gemm          # dense tcgen05 GEMMs of the prompt path: us, TFLOP/s

Results that fail the kernel's own validation are skipped (the entry point refuses them before launching anything).
Timing: CUDA events around ``iters`` launches that rotate over enough independent weight sets to exceed L2.
"""
from __future__ import annotations

import argparse
import itertools
import json
from typing import Callable, Dict, List

import torch


def _time_us(fn: Callable[[int], None], iters: int) -> float:
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def sweep_experts(tp: int, fp8: bool, iters: int, dev: torch.device) -> Dict:
    """Gate/up + down expert GEMVs of one token at the shapes of Qwen3-235B-A22B split ``tp`` ways."""
    from ..models.quant import store_weight
    from . import lib
    H, I, k = 4096, 1536 // tp, 8
    E = 8                                               # one set = the 8 selected experts; sets rotate to defeat L2
    bytes_set = E * 3 * I * H * (1 if fp8 else 2)
    nsets = max(2, (192 << 20) // bytes_set + 1)
    g = torch.Generator(device=dev).manual_seed(1)

    def mk(rows, cols):
        w = torch.randn(E, rows, cols, device=dev, generator=g) * 0.02
        return store_weight(w, "fp8_block" if fp8 else "bf16")
    sets = [(mk(2 * I, H), mk(H, I)) for _ in range(nsets)]
    x = torch.randn(H, device=dev, generator=g)
    sel = torch.arange(k, dtype=torch.int32, device=dev)
    sw = torch.full((k,), 1.0 / k, device=dev)
    resid, xn, gamma = torch.zeros(H, device=dev), torch.zeros(H, device=dev), torch.ones(H, device=dev)
    act = torch.zeros(k * I, device=dev)
    counter = torch.zeros(8, dtype=torch.int32, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    epoch = torch.zeros(4, dtype=torch.int32, device=dev)
    slots = torch.zeros(2 * H, device=dev)

    def args_for(wgu, wd, R_gu, R_d, S, grid):
        a = lib.IhbMoeArgs()
        a.Wgu, a.Wd, a.wtype = wgu.data.data_ptr(), wd.data.data_ptr(), lib.wtype_of(wgu.data)
        a.H, a.I, a.E_local, a.expert0, a.top_k = H, I, E, 0, k
        if fp8:
            gsc, dsc = lib.kernel_scale(wgu), lib.kernel_scale(wd)
            a.gu_scale, a.d_scale = gsc.data_ptr(), dsc.data_ptr()
            a.gu_rb, a.gu_kb_shift, a.gu_nkb = wgu.rb, lib.kb_shift_of(wgu.kb), gsc.shape[-1]
            a.d_rb, a.d_kb_shift, a.d_nkb = wd.rb, lib.kb_shift_of(wd.kb), dsc.shape[-1]
        a.x, a.sel_idx, a.sel_w, a.act = x.data_ptr(), sel.data_ptr(), sw.data_ptr(), act.data_ptr()
        a.counter, a.err = counter.data_ptr(), err.data_ptr()
        a.resid, a.gamma, a.xn_out, a.eps = resid.data_ptr(), gamma.data_ptr(), xn.data_ptr(), 1e-6
        a.comm = lib.single_comm(slots, epoch)
        a.R_gu, a.R_d, a.S, a.grid = R_gu, R_d, S, grid
        return a

    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    rows: List[Dict] = []
    # grids never exceed the SM count: the down kernel's tail waits for the other CTAs' partial sums, so all CTAs of a
    # launch must be resident together
    for R_gu, R_d, S, gdiv in itertools.product((0, 1, 2, 4, 8), (0, 4, 8, 16, 32), (0, 3, 6, 12), (1, 2)):
        if (R_gu == 0) != (R_d == 0) or (R_gu == 0 and (S or gdiv != 1)):
            continue                                     # (0, 0, 0, default grid) is the kernels' own rule; no mixed cases
        grid = 0 if R_gu == 0 else sms // gdiv
        blocks = [args_for(wgu, wd, R_gu, R_d, S, grid) for wgu, wd in sets]

        def fn(i, blocks=blocks):
            lib.moe_gateup(blocks[i % len(blocks)], False)
            lib.moe_down(blocks[i % len(blocks)], False)
        try:
            fn(0)                                        # one launch pair first: a configuration whose bounded waits
            torch.cuda.synchronize()                     # run out reports through the error word and is not timed
            code = int(err.item())
            if code:
                err.zero_()
                counter.zero_()
                rows.append({"R_gu": R_gu, "R_d": R_d, "S": S, "grid": grid, "error_word": code})
                continue
            us = _time_us(fn, iters)
        except RuntimeError:
            continue                                     # refused by the entry point's validation
        rows.append({"R_gu": R_gu, "R_d": R_d, "S": S, "grid": grid, "us": round(us, 2),
                     "gbs": round(bytes_set / us * 1e-3, 1)})
    timed = [r for r in rows if "us" in r]
    best = min(timed, key=lambda r: r["us"])
    rule = next(r for r in timed if r["R_gu"] == 0)
    return {"shape": {"H": H, "I": I, "top_k": k, "weights": "fp8_block" if fp8 else "bf16", "bytes": bytes_set},
            "rule": rule, "best": best, "rule_vs_best": round(rule["us"] / best["us"], 3), "all": rows}


def _e4m3_rows(x: torch.Tensor):
    """x [..., 128] -> (e4m3 bytes as uint8, one fp32 scale per row = amax / 448): the cache layout of ``kv="fp8"``."""
    s = x.abs().amax(-1, keepdim=True).clamp_min(1e-12) / 448.0
    return (x / s).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).contiguous(), s[..., 0].contiguous()


def sweep_flash_decode(tp: int, iters: int, dev: torch.device, contexts=(4096, 32768), kv8: bool = False) -> Dict:
    """Split count of the split-KV flash-decode kernel at the head counts of one rank (64 / tp query heads, at least
    one KV head); ``kv8``: over an e4m3 cache with a scale per row instead of bf16 rows."""
    from . import lib
    nq, nkv = 64 // tp, max(1, 4 // tp)
    out: Dict = {}
    g = torch.Generator(device=dev).manual_seed(2)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    for ctx in contexts:
        bytes_kv = 2 * nkv * ctx * (128 + 4) if kv8 else 2 * nkv * ctx * 128 * 2
        ncopies = max(2, (192 << 20) // bytes_kv + 1)
        ncopies = min(ncopies, 64)
        ksc = vsc = [None] * ncopies
        if kv8:
            kq = [_e4m3_rows(torch.randn(nkv, ctx, 128, device=dev, generator=g)) for _ in range(ncopies)]
            vq = [_e4m3_rows(torch.randn(nkv, ctx, 128, device=dev, generator=g)) for _ in range(ncopies)]
            kc, ksc = [a for a, _ in kq], [b for _, b in kq]
            vc, vsc = [a for a, _ in vq], [b for _, b in vq]
        else:
            kc = [torch.randn(nkv, ctx, 128, device=dev, generator=g).to(torch.bfloat16) for _ in range(ncopies)]
            vc = [torch.randn(nkv, ctx, 128, device=dev, generator=g).to(torch.bfloat16) for _ in range(ncopies)]
        q = torch.randn(nq * 128, device=dev, generator=g)
        pos = torch.tensor([ctx - 1], dtype=torch.int32, device=dev)
        o = torch.zeros(nq * 128, device=dev)
        rows = []
        for nsplit in (1, 2, 4, 8, 16, 32, 64, 128, 256):
            if nsplit > ctx // 32:
                continue
            scratch = torch.zeros(lib.flash_decode_scratch_floats(nq, nsplit), device=dev)
            ctrs = torch.zeros(nq, dtype=torch.int32, device=dev)

            def fn(i):
                j = i % ncopies
                lib.flash_decode(q, kc[j], vc[j], nq, nkv, ctx, pos, nsplit, scratch, ctrs, o, False,
                                 k_scale=ksc[j], v_scale=vsc[j])
            try:
                us = _time_us(fn, iters)
            except RuntimeError:
                continue
            rows.append({"nsplit": nsplit, "ctas": nsplit * nkv, "us": round(us, 2), "gbs": round(bytes_kv / us * 1e-3, 1)})
        best = min(rows, key=lambda r: r["us"])
        out[str(ctx)] = {"nq": nq, "nkv": nkv, "kv_bytes": bytes_kv, "sms": sms, "best": best, "all": rows}
    return out


def sweep_verify_attention(tp: int, iters: int, dev: torch.device, ctx: int = 4096) -> Dict:
    """Flatness in M of the verify / window attention: M query tokens behind ``ctx`` cached positions, for the
    tensor-core tiles with the keys sliced over CTAs (what the window path runs), the same tiles with one CTA per
    query tile, and the one-CTA-per-token CUDA-core kernel (mode 1). The reference's acceptance bar for
    a verify kernel is T(M) / T(1) near 1 (results/mk_tree_attn/K2_FLATNESS_AB.md: 4.0-4.2x on CUDA cores at M = 8,
    1.03x on tensor cores)."""
    from . import lib
    nq, nkv = 64 // tp, max(1, 4 // tp)
    g = torch.Generator(device=dev).manual_seed(3)
    max_seq = ctx + 64
    bytes_kv = 2 * nkv * max_seq * 128 * 2
    ncopies = min(64, max(2, (192 << 20) // bytes_kv + 1))
    kc = [torch.randn(nkv, max_seq, 128, device=dev, generator=g).to(torch.bfloat16) for _ in range(ncopies)]
    vc = [torch.randn(nkv, max_seq, 128, device=dev, generator=g).to(torch.bfloat16) for _ in range(ncopies)]
    out: Dict = {"ctx": ctx, "nq": nq, "nkv": nkv}
    for mode, split, name in ((0, True, "tensor_core_sliced"), (0, False, "tensor_core"), (1, False, "cuda_core")):
        rows = []
        for M in (1, 4, 8, 16, 32):
            qkv = torch.randn(M, (nq + 2 * nkv) * 128, device=dev, generator=g)
            o = torch.zeros(M, nq * 128, device=dev)
            scr = torch.zeros(lib.window_attention_scratch_floats(nq, nkv, M), device=dev) if split else None

            def fn(i):
                lib.window_attention(qkv, kc[i % ncopies], vc[i % ncopies], nq, nkv, max_seq, ctx, None, o, mode, scr)
            rows.append({"M": M, "us": round(_time_us(fn, iters), 2)})
        for r in rows:
            r["vs_M1"] = round(r["us"] / rows[0]["us"], 3)
        out[name] = rows
    return out


def sweep_window_gemm(iters: int, dev: torch.device) -> List[Dict]:
    """Dense tcgen05 GEMMs of the prompt path (bf16 operands, LINEAR mode, 128-token tiles in one launch) at the
    shapes of a full-width rank and of one rank of TP8: time and TFLOP/s, weight sets rotating so that every launch
    streams its weights from HBM; cuBLAS (``torch.matmul``) on the largest shape for scale."""
    from ..models.quant import QWeight
    from . import lib
    g = torch.Generator(device=dev).manual_seed(0)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    rows_out: List[Dict] = []

    def run(rows, Kd, T, ks, nsets=6):
        Ws = [QWeight((torch.randn(rows, Kd, device=dev, generator=g) * 0.02).to(torch.bfloat16)) for _ in range(nsets)]
        X = torch.randn(T, Kd, device=dev, generator=g).to(torch.bfloat16)
        blocks = []
        for W in Ws:
            a = lib.IhbTcArgs()
            lib.tc_fill_weight(a, W)
            out = torch.zeros(T, rows, device=dev)
            a.X, a.mode, a.out_stride = X.data_ptr(), lib.TC_LINEAR, rows
            a.T_total, a.err = T, err.data_ptr()
            a.T, a.tok0, a.out = T, 0, out.data_ptr()
            if T > 128:
                a.tok_tile, a.tok_tiles = 128, -(-T // 128)
            tiles = ((rows + 127) // 128) * max(1, a.tok_tiles)
            a.ks = ks
            part = torch.zeros(max(1, lib.tc_partial_floats(a)), device=dev)
            ctr = torch.zeros(max(tiles, 1), dtype=torch.int32, device=dev)
            a.partial, a.tile_counters = part.data_ptr(), ctr.data_ptr()
            blocks.append((a, out, part, ctr))
        us = _time_us(lambda i: lib.tc_gemm(blocks[i % nsets][0], False), iters)
        ref = X.float() @ Ws[(iters - 1) % nsets].data.float().t()
        diff = float((blocks[(iters - 1) % nsets][1] - ref).abs().max())
        rows_out.append({"rows": rows, "K": Kd, "T": T, "ks": ks, "us": round(us, 1),
                         "tflops": round(2.0 * rows * Kd * T / us * 1e-6, 1), "maxdiff": diff})

    for rows, Kd, T, ks in [(9216, 4096, 1024, 1), (4096, 8192, 1024, 1), (1280, 4096, 1024, 1), (1280, 4096, 1024, 2),
                            (4096, 1024, 1024, 1), (9216, 4096, 128, 1), (1280, 4096, 128, 1)]:
        run(rows, Kd, T, ks)
    if int(err.item()):
        raise RuntimeError("device error word set during the GEMM sweep")
    x = torch.randn(1024, 4096, device=dev).to(torch.bfloat16)
    w = torch.randn(9216, 4096, device=dev).to(torch.bfloat16)
    us = _time_us(lambda i: torch.matmul(x, w.t()), iters)
    rows_out.append({"rows": 9216, "K": 4096, "T": 1024, "ks": 0, "us": round(us, 1), "tflops": round(2.0 * 9216 * 4096 * 1024 / us * 1e-6, 1),
                     "library": "torch.matmul (cuBLAS)"})
    return rows_out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--weights", default="fp8_block", choices=["fp8_block", "bf16"])
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--out", default="")
    ap.add_argument("--skip-experts", action="store_true")
    ap.add_argument("--gemm", action="store_true", help="only the dense tcgen05 GEMM table of the prompt path")
    ap.add_argument("--flash-kv", action="store_true", help="only flash decode, over bf16 and over e4m3 cache rows")
    a = ap.parse_args(argv)
    from . import lib
    lib.load()
    dev = torch.device("cuda", 0)
    res: Dict = {"tp": a.tp}
    if a.gemm:
        res["window_gemm"] = sweep_window_gemm(a.iters, dev)
        for r in res["window_gemm"]:
            print("gemm", r)
        if a.out:
            with open(a.out, "w") as f:
                json.dump(res, f, indent=1)
        return 0
    if a.flash_kv:
        for name, kv8 in (("bf16", False), ("e4m3", True)):
            res["flash_decode_" + name] = sweep_flash_decode(a.tp, a.iters, dev, kv8=kv8)
            for ctx, r in res["flash_decode_" + name].items():
                print(f"flash-decode {name} cache, ctx {ctx}, nq {r['nq']}, nkv {r['nkv']}: best {r['best']}")
        if a.out:
            with open(a.out, "w") as f:
                json.dump(res, f, indent=1)
        return 0
    if not a.skip_experts:
        res["experts"] = sweep_experts(a.tp, a.weights == "fp8_block", a.iters, dev)
        e = res["experts"]
        print(f"experts: rule {e['rule']['us']} us ({e['rule']['gbs']} GB/s), best {e['best']} -> rule/best {e['rule_vs_best']}")
    res["flash_decode"] = sweep_flash_decode(a.tp, a.iters, dev)
    for ctx, r in res["flash_decode"].items():
        print(f"flash-decode ctx {ctx}: best {r['best']}")
    res["verify_attention"] = sweep_verify_attention(a.tp, a.iters, dev)
    for name in ("tensor_core_sliced", "tensor_core", "cuda_core"):
        print(f"verify attention ctx 4096, {name}: " + ", ".join(f"M={r['M']} {r['us']} us ({r['vs_M1']}x)" for r in res["verify_attention"][name]))
    if a.out:
        with open(a.out, "w") as f:
            json.dump(res, f, indent=1)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
