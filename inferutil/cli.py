"""``python -m inferutil [--gpu NAME] [--n-gpus N]``: hardware, model, memory, latency-by-plan, takeaways,
speculative-decoding and expert-placement reports (reference: src/inferutil/cli.py:19-269)."""
from __future__ import annotations

import argparse
import random

from .hardware import GPUS, Cluster
from .latency import decode_latency, expected_max_experts_per_gpu
from .model import QWEN3_235B, QWEN3_30B
from .routing import CoActGraph, TokenDAG, greedy_partition, placement_stats, round_robin_placement
from .speculative import memory_feasibility, sweep as spec_sweep


def _b(n: int) -> str:
    return f"{n / 1e9:.2f}B"


def _gb(n: float) -> str:
    return f"{n / 1e9:.1f} GB"


def hardware_summary(cluster) -> str:
    g = cluster.gpu
    return "\n".join([f"== hardware: {cluster.n_gpus} x {g.name} ==",
                      f"  HBM            {_gb(g.hbm_bytes)} per GPU, {_gb(cluster.total_hbm)} total",
                      f"  HBM bandwidth  {g.hbm_bw / 1e12:.2f} TB/s per GPU, {cluster.aggregate_hbm_bw / 1e12:.1f} TB/s aggregate",
                      f"  tensor peak    {g.bf16_flops / 1e12:.0f} TFLOP/s bf16, {g.fp8_flops / 1e12:.0f} TFLOP/s fp8 (dense)",
                      f"  NVLink         {g.nvlink_bw / 1e9:.0f} GB/s per direction; small collective ~{g.collective_latency_s * 1e6:.1f} us"])


def model_summary(cfg) -> str:
    return "\n".join([f"== model: {cfg.name} ==",
                      f"  {cfg.n_layers} layers, hidden {cfg.hidden}, {cfg.n_heads} q / {cfg.n_kv_heads} kv heads x {cfg.head_dim}",
                      f"  {cfg.n_experts} experts, top-{cfg.top_k}, expert inner {cfg.moe_inter}, vocab {cfg.vocab}",
                      f"  parameters: total {_b(cfg.total_params)}, active per token {_b(cfg.active_params)} "
                      f"({100.0 * cfg.active_params / cfg.total_params:.1f}%)",
                      f"  KV cache: {cfg.kv_bytes_per_token(2) / 1024:.0f} KiB per token (bf16)"])


def memory_budget(cfg, cluster) -> str:
    lines = ["== memory budget =="]
    for name, nbytes in (("bf16", 2), ("fp8", 1)):
        w = cfg.total_params * nbytes
        left = cluster.total_hbm - w
        ctx = int(left // cfg.kv_bytes_per_token(2)) if left > 0 else 0
        lines.append(f"  {name}: weights {_gb(w)} -> " + (f"headroom {_gb(left)} = {ctx:,} cached tokens (bf16 KV)"
                                                          if left > 0 else "does not fit"))
    return "\n".join(lines)


def latency_table(cfg, cluster) -> str:
    lines = ["== decode latency at batch 1 (ms per token) ==",
             f"  {'plan':<8}{'dtype':<6}{'seq':>7}{'weight':>9}{'kv':>8}{'compute':>9}{'comms':>8}{'total':>9}{'tok/s':>9}{'imbal':>7}"]
    for dtype in (2, 1):
        for plan in ("floor", "tp", "ep", "hybrid"):
            for seq in (2048, 32768):
                r = decode_latency(cfg, cluster, plan=plan, dtype_bytes=dtype, seq_len=seq,
                                   tp=min(2, cluster.n_gpus) if plan == "hybrid" else None).as_row()
                lines.append(f"  {r['plan']:<8}{r['dtype']:<6}{r['seq']:>7}{r['weight_ms']:>9.3f}{r['kv_ms']:>8.3f}"
                             f"{r['compute_ms']:>9.3f}{r['comms_ms']:>8.3f}{r['total_ms']:>9.3f}{r['tok_per_s']:>9.1f}"
                             f"{r['expert_imbalance']:>7.2f}")
    return "\n".join(lines)


def takeaways(cfg, cluster) -> str:
    n = cluster.n_gpus
    tp = decode_latency(cfg, cluster, plan="tp", dtype_bytes=1, seq_len=2048)
    ep = decode_latency(cfg, cluster, plan="ep", dtype_bytes=1, seq_len=2048)
    long = decode_latency(cfg, cluster, plan="tp", dtype_bytes=1, seq_len=32768)
    emax = expected_max_experts_per_gpu(cfg.top_k, n)
    return "\n".join(["== takeaways ==",
                      f"  1. decode is bandwidth- and latency-bound: compute is {100 * tp.compute_s / tp.total_s:.1f}% of a token.",
                      f"  2. {2 * cfg.n_layers} collectives per token cost {1e3 * tp.comms_s:.2f} ms at "
                      f"{cluster.gpu.collective_latency_s * 1e6:.0f} us each ({100 * tp.comms_s / tp.total_s:.0f}% of the token): "
                      "fuse them into the producing kernels.",
                      f"  3. expert parallelism over {n} GPUs makes the busiest GPU serve {emax:.2f} of {cfg.top_k} experts "
                      f"(x{ep.imbalance:.2f} imbalance): {ep.tokens_per_s:.0f} vs {tp.tokens_per_s:.0f} tok/s for TP-in-expert.",
                      f"  4. at 32k context the KV read is {100 * long.kv_read_s / long.total_s:.0f}% of a token "
                      f"({long.tokens_per_s:.0f} tok/s): KV heads replicate beyond {cfg.n_kv_heads}-way TP."])


def speculative_report() -> str:
    rows = spec_sweep(alphas=[0.6, 0.7, 0.8], ks=[4, 8], n_drafters_list=[1, 2, 4])
    lines = ["== speculative decoding (analytical) ==", f"  {'alpha':>6}{'k':>4}{'N':>4}{'E[acc]':>9}{'speedup':>9}"]
    lines += [f"  {r.alpha:>6.2f}{r.k:>4}{r.n_drafters:>4}{r.e_acc:>9.2f}{r.speedup:>9.2f}" for r in rows]
    f = memory_feasibility()
    lines.append(f"  fp8 target leaves {f['hbm_headroom_gb']} GB: room for {f['max_drafters']} drafters of {f['draft_model_gb']} GB")
    return "\n".join(lines)


def routing_report() -> str:
    """Synthetic clustered routing (tokens prefer one of 8 expert groups) to show what placement can recover."""
    rng = random.Random(0)
    n_layers, n_experts, n_gpus, k = 8, 128, 8, 8
    g = CoActGraph(n_experts=n_experts, n_layers=n_layers)
    dag = TokenDAG()
    perm = list(range(n_experts))
    rng.shuffle(perm)
    for _ in range(400):
        cluster_id = rng.randrange(8)
        prev = None
        for layer in range(n_layers):
            home = [perm[cluster_id * 16 + i] for i in range(16)]
            chosen = rng.sample(home, 6) + rng.sample(range(n_experts), 2)
            g.add_token_step(layer, chosen)
            if prev is not None:
                g.add_cross_layer(layer - 1, prev, chosen)
            prev = chosen
            dag.add_layer(layer, chosen)
    rr = round_robin_placement(n_gpus, n_experts, n_layers)
    gp = greedy_partition(g, n_gpus, n_experts, n_layers)
    a, b = placement_stats(g, rr, "round-robin"), placement_stats(g, gp, "greedy")
    touched = [p["n_gpus_touched"] for p in dag.prefetch_schedule(gp, n_experts)]
    return "\n".join(["== expert placement (synthetic clustered routing) ==",
                      f"  round-robin: {100 * a['cross_gpu_fraction']:.1f}% of co-activation weight crosses GPUs",
                      f"  greedy:      {100 * b['cross_gpu_fraction']:.1f}% crosses GPUs",
                      f"  last token's prefetch plan touches {sum(touched) / max(1, len(touched)):.1f} GPUs per layer"])


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(prog="inferutil")
    ap.add_argument("--gpu", default="H100-SXM-80GB", choices=list(GPUS))
    ap.add_argument("--n-gpus", type=int, default=8)
    ap.add_argument("--model", default="qwen3-235b-a22b", choices=["qwen3-235b-a22b", "qwen3-30b-a3b"])
    args = ap.parse_args(argv)
    cluster = Cluster(GPUS[args.gpu], args.n_gpus)
    cfg = QWEN3_235B if args.model == "qwen3-235b-a22b" else QWEN3_30B
    print("\n\n".join([hardware_summary(cluster), model_summary(cfg), memory_budget(cfg, cluster),
                       latency_table(cfg, cluster), takeaways(cfg, cluster), speculative_report(), routing_report()]))


if __name__ == "__main__":
    main()
