"""Collective sweep: fused all-reduce + residual + RMSNorm kernel (one-shot / two-shot over symmetric memory, NVLS
multicast or peer mode) against NCCL all-reduce followed by a separate norm, for hidden-state tensors ``[T, H]``.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m inferencehackathon_b200.parallel.ar_sweep [--hidden 4096] [--max-mb 64] [--iters 50]

Every number is device-timed (CUDA events around ``iters`` back-to-back launches), max over ranks. One JSON line per
size is printed by rank 0; each line also carries the maximum deviation of the fused result from the NCCL result.
The reference measures the same trade-off with kernels/nvls_ar.cu, kernels/oneshot_allreduce.cu and nccl-tests
(docs/onbox-collective-latency-e0.md, docs/comms-breakthrough-nvls.md).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def _time(fn, iters: int, dev) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize(dev)
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize(dev)
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--max-mb", type=float, default=64.0)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--out", default="")
    ap.add_argument("--payload", default="fp32", choices=["fp32", "bf16"],
                    help="input type of the counted small-message variant (the one-shot / two-shot kernels take fp32)")
    a = ap.parse_args(argv)
    from ..config import ParallelConfig
    from ..ops import lib as K
    from .launch import init_distributed
    from .symm import SymmetricComm
    rank, world, local = init_distributed()
    dev = torch.device("cuda", local)
    K.load()
    H = a.hidden
    rows = []
    t = 1
    while t * H * 4 <= a.max_mb * (1 << 20):
        rows.append(t)
        t *= 4
    maxn = rows[-1] * H
    par = ParallelConfig(tp=world, ep=1, rank=rank, world=world)
    small_rows = 64                                   # the counted variant: up to 64 rows, slots in the tail region
    comm = SymmetricComm(par, dev, slot_floats=max(2 * maxn, 2 * world * min(maxn, (1 << 20))),
                         extra_bytes=4 * small_rows * H * 8)
    epoch = torch.zeros(1, dtype=torch.int32, device=dev)
    counter = torch.zeros(8, dtype=torch.int32, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    cm = comm.comm_block(epoch)
    cm_small = comm.comm_block(epoch, slot_offset_bytes=comm.extra_off)
    small_counter = torch.zeros(8, dtype=torch.int32, device=dev)
    small_calls = {}
    gamma = torch.ones(H, device=dev)
    lines = []
    for T in rows:
        g = torch.Generator(device=dev).manual_seed(1000 * T + rank)
        x = torch.randn(T, H, device=dev, generator=g)
        resid = torch.randn(T, H, device=dev, generator=torch.Generator(device=dev).manual_seed(7))
        out, outn = torch.empty_like(x), torch.empty_like(x)
        nbytes = T * H * 4

        def nccl():
            y = x.clone()
            dist.all_reduce(y)
            y += resid
            return y, y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma

        ref, refn = nccl()
        rec = {"T": T, "H": H, "bytes": nbytes, "n_gpus": world, "mode": "multicast" if comm.use_multicast else "p2p"}
        for name, algo in (("oneshot", 1), ("twoshot", 2)):
            if algo == 1 and 2 * world * T * H > comm.slots_local.numel():
                continue
            fn = lambda: K.allreduce_norm(cm, x, out, counter, err, resid=resid, gamma=gamma, out_norm=outn, algo=algo)
            fn()
            torch.cuda.synchronize(dev)
            dev_err = max(float((out - ref).abs().max()), float((outn - refn).abs().max()))
            rec[name + "_us"] = round(_time(fn, a.iters, dev), 2)
            rec[name + "_maxdiff"] = dev_err
            if int(err.item()):
                rec[name + "_error"] = int(err.item())
                err.zero_()
        if T <= small_rows:
            # one call counter per shape: the slot layout [4][T * H] depends on T
            cc = small_calls.setdefault(T, torch.zeros(64, dtype=torch.int32, device=dev))
            comm.extra(4 * small_rows * H * 8).zero_()
            comm.barrier_host()
            xin = x.to(torch.bfloat16) if a.payload == "bf16" else x
            fn = lambda: K.allreduce_counted(cm_small, xin, out, small_counter, cc, err, resid=resid, gamma=gamma, out_norm=outn)
            fn()
            torch.cuda.synchronize(dev)
            refc, refcn = ref, refn
            if a.payload == "bf16":
                y = xin.float().clone()
                dist.all_reduce(y)
                y += resid
                refc, refcn = y, y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma
            rec["counted_us"] = round(_time(fn, a.iters, dev), 2)
            rec["counted_maxdiff"] = max(float((out - refc).abs().max()), float((outn - refcn).abs().max()))
            rec["counted_payload"] = a.payload
            if int(err.item()):
                rec["counted_error"] = int(err.item())
                err.zero_()
        rec["nccl_allreduce_us"] = round(_time(lambda: dist.all_reduce(x.clone()), a.iters, dev), 2)
        rec["nccl_plus_norm_us"] = round(_time(nccl, a.iters, dev), 2)
        best = min(v for k, v in rec.items() if k.endswith("shot_us") or k == "counted_us")
        rec["fused_best_us"] = best
        rec["speedup_vs_nccl_plus_norm"] = round(rec["nccl_plus_norm_us"] / best, 2)
        rec["busbw_gbs"] = round(2 * (world - 1) / world * nbytes / best / 1e3, 1)
        if rank == 0:
            print("AR_SWEEP " + json.dumps(rec), flush=True)
            lines.append(rec)
    if rank == 0 and a.out:
        with open(a.out, "w") as f:
            json.dump(lines, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
