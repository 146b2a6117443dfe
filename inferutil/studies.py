"""Closed-form studies around the B = 1 decode step: every function here is arithmetic on measured inputs (no GPU, no
model weights) and answers one planning question. ``python -m inferutil.studies <command>`` prints the table.

Counterparts in the reference's ``tools/`` directory, each a stand-alone script with its inputs edited in place:
backout_floor.py, comms_floor_reconcile.py, overhead_fork.py, ladder_to_1000.py, latency_budget.py,
predict_matrix.py, spec_floor_model.py, spec_moe_model.py, spec_predict.py, tree_spec_optimizer.py,
stale_tp_ceiling.py, tp_degree_model.py, verify_cost_check.py, whole_engine_mbu_ceiling.py,
validate_routing_model.py, eagle3_analyze.py and diag_analyze.py. Here they are functions with explicit arguments
(defaults: Qwen3-235B-A22B on 8 B200) so that they can be called from tests, the bench harness and the server.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import random
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

from .hardware import GPUS, Cluster, measured_b200
from .latency import decode_latency, expected_max_experts_per_gpu
from .model import QWEN3_235B, MoEConfig

NONEXPERT_SHARE = 0.34          # share of a decode step's weight bytes that every position shares
ROUTED_SHARE = 0.66             # share that scales with the number of distinct experts


# ---- expert union and the floor-aware verify cost --------------------------------------------------------------------
def expert_union(positions: float, n_experts: int = 128, top_k: int = 8, overlap: float = 0.0) -> float:
    """E[distinct experts] lit by ``positions`` independent top-k draws; ``overlap`` (0..1) is the share of positions
    that a route-aware drafter makes coincide with earlier ones."""
    eff = max(0.0, positions * (1.0 - overlap))
    return n_experts * (1.0 - ((n_experts - top_k) / n_experts) ** eff)


def weight_units(union: float, top_k: int = 8, ep_factor: float = 1.0) -> float:
    """Weight bytes of a verify pass in units of one decode step's weight bytes."""
    return NONEXPERT_SHARE + ROUTED_SHARE * (union / top_k) * ep_factor


def floor_verify_cost(floor: float, union: float, top_k: int = 8, ep_factor: float = 1.0) -> float:
    """Verify pass in decode-step units: the fixed share ``floor`` is paid once, the rest follows the union."""
    f = min(1.0, max(0.0, floor))
    return f + (1.0 - f) * weight_units(union, top_k, ep_factor)


def expected_emitted(alpha: float, depth: int, width: int = 1) -> float:
    """Tokens per round including the bonus token; a level is hit when any of ``width`` candidates is accepted."""
    p = 1.0 - (1.0 - min(0.999999, max(0.0, alpha))) ** max(1, width)
    return float(depth + 1) if p >= 1.0 else (1.0 - p ** (depth + 1)) / (1.0 - p)


# ---- backing the floor share out of measured speculative runs -------------------------------------------------------------
def backout_floor(measured: Sequence[Tuple[int, float, float]], n_experts: int = 128, top_k: int = 8) -> dict:
    """``measured``: (draft positions k, accept length tau, realised speedup S). V = tau / S is the verify cost in
    decode-step units; V(k) = F + (1 - F) w(k) with w the weight units of k positions. Two or more sizes
    over-determine F: every pair gives one estimate, and a least-squares fit over all points another."""
    pts = [(k, tau / s, weight_units(expert_union(k, n_experts, top_k), top_k)) for k, tau, s in measured if s > 0]
    per_point = [{"k": k, "V": v, "w": w, "F": (w - v) / (w - 1.0) if abs(w - 1.0) > 1e-9 else None} for k, v, w in pts]
    pair = []
    for i in range(len(pts)):
        for j in range(i + 1, len(pts)):
            (_, v1, w1), (_, v2, w2) = pts[i], pts[j]
            if abs(w2 - w1) > 1e-9:
                pair.append(1.0 - (v2 - v1) / (w2 - w1))        # dV/dw = 1 - F
    # least squares on V = F (1 - w) + w  ->  (V - w) = F (1 - w)
    num = sum((v - w) * (1.0 - w) for _, v, w in pts)
    den = sum((1.0 - w) ** 2 for _, _, w in pts)
    fit = num / den if den else None
    f = fit if fit is not None else (pair[0] if pair else None)
    verdict = None
    if f is not None:
        biggest = max(pts, key=lambda p: p[0])
        union_share = (1.0 - f) * ROUTED_SHARE * expert_union(biggest[0], n_experts, top_k) / top_k / biggest[1]
        verdict = {"union_share_of_verify": union_share, "route_aware_pays": union_share > 0.15}
    return {"points": per_point, "pairwise_F": pair, "F": f, "verdict": verdict}


# ---- which per-collective latency is consistent with the measured step time -----------------------------------------------
def comms_reconcile(tpot_ms: float, n_collectives: int, weight_floor_ms: float, measured_efficiency: float,
                    candidates_us: Iterable[float], kv_ms: float = 0.07) -> List[dict]:
    """A serial step is compute + collectives + host time. For a hypothesised per-collective latency C the rest
    R = TPOT - n C - kv has to hold weight_floor / e plus a non-negative host time, which demands e >= floor / R.
    A hypothesis that demands more efficiency than the kernels were measured to have is inconsistent."""
    rows = []
    for c in candidates_us:
        comms = n_collectives * c / 1e3
        rest = tpot_ms - comms - kv_ms
        need = weight_floor_ms / rest if rest > 0 else float("inf")
        host = rest - weight_floor_ms / measured_efficiency if rest > 0 else float("-inf")
        rows.append({"collective_us": c, "comms_ms": comms, "rest_ms": rest, "required_efficiency": need,
                     "implied_host_ms": host, "consistent": rest > 0 and need <= measured_efficiency + 1e-9})
    return rows


def overhead_fork(tpot_ms: float, weight_floor_ms: float, comms_ms: float, kv_ms: float, launch_ms: float,
                  kernel_efficiency: float, cfg: MoEConfig = QWEN3_235B, n_gpus: int = 8, hbm_bw: float = 7.7e12,
                  dtype_bytes: int = 1) -> dict:
    """Splits the step time not explained by bytes and collectives two ways: (a) launch/host bound (kernels at the
    roofline, the rest is host time) and (b) kernel bound (kernels at the measured efficiency). Also prices the
    head + arg-max, a usual suspect that physics clears."""
    overhead = tpot_ms - weight_floor_ms - comms_ms - kv_ms
    head_ms = cfg.vocab * cfg.hidden * dtype_bytes / n_gpus / hbm_bw * 1e3
    logits_ms = cfg.vocab * 4 / hbm_bw * 1e3
    kernel_ms = weight_floor_ms / kernel_efficiency - weight_floor_ms
    return {"overhead_ms": overhead, "head_plus_argmax_ms": head_ms + logits_ms,
            "head_share_of_tpot": (head_ms + logits_ms) / tpot_ms,
            "fork_a_launch_bound": {"launch_host_ms": overhead, "kernel_ms": 0.0, "top_lever": "one launch per token"},
            "fork_b_kernel_bound": {"kernel_ms": min(overhead, kernel_ms), "launch_host_ms": max(0.0, overhead - kernel_ms),
                                    "top_lever": "kernel efficiency"},
            "graphs_already_on_recovers_ms": min(launch_ms, max(0.0, overhead - kernel_ms))}


# ---- ladder of levers -------------------------------------------------------------------------------------------------------
@dataclass
class Terms:
    overhead: float
    comms: float
    weight: float
    kv: float
    spec: float = 1.0

    @property
    def tpot_ms(self) -> float:
        return (self.overhead + self.comms + self.weight + self.kv) / self.spec

    @property
    def tok_s(self) -> float:
        return 1000.0 / self.tpot_ms


B200_MEASURED_START = Terms(overhead=3.03, comms=0.27, weight=0.43, kv=0.01)   # 3.74 ms: 8 GPUs, persistent kernel
# (comms: 94 layers x 2 x 1.4 us that the all-reduces cost beyond the same phases on one GPU, plus the arg-max exchange;
# weight: bytes at the measured copy bandwidth; overhead: the rest, i.e. 94 x ~32 us of phase latencies)

DEFAULT_RUNGS: List[Tuple[str, Dict[str, float]]] = [
    ("hand-overs inside thread-block clusters through distributed shared memory (12 L2 round trips per layer -> 6)", {"overhead": 2.75}),
    ("o_proj starts on the attention blocks that have arrived (no wait for the last block)", {"overhead": 2.5}),
    ("several tokens per cooperative launch in generation loops (13 us launch boundary per token)", {"overhead": 2.49}),
    ("fp4 expert weights", {"weight": 0.28}),
    ("speculative decoding, tau 2.5 at verify cost 1.25 (needs a verify window near one decode step; today ~4)", {"spec": 2.0}),
]


def ladder(start: Terms = B200_MEASURED_START, rungs: Sequence[Tuple[str, Dict[str, float]]] = DEFAULT_RUNGS) -> List[dict]:
    """Applies the levers in order; a rung REPLACES the named terms (absolute values, ms; ``spec`` is a divisor)."""
    cur = dataclasses.replace(start)
    out = [{"rung": "measured start", "tpot_ms": cur.tpot_ms, "tok_s": cur.tok_s, **dataclasses.asdict(cur)}]
    for label, change in rungs:
        cur = dataclasses.replace(cur, **change)
        out.append({"rung": label, "tpot_ms": cur.tpot_ms, "tok_s": cur.tok_s, **dataclasses.asdict(cur)})
    return out


# ---- single-user latency budget ----------------------------------------------------------------------------------------------
def modelled_tpot_ms(plan: str, tp: int, ep: int, dtype_bytes: int, collective_us: float, efficiency: float,
                     host_ms: float, ctx: int = 512, kv_dtype_bytes: int = 2, gpu: str = "B200-SXM-180GB",
                     n_gpus: int = 8, cfg: MoEConfig = QWEN3_235B) -> float:
    g = dataclasses.replace(GPUS[gpu], collective_latency_s=collective_us * 1e-6)
    b = decode_latency(cfg, Cluster(g, n_gpus), plan=plan, dtype_bytes=dtype_bytes, kv_dtype_bytes=kv_dtype_bytes,
                       seq_len=ctx, tp=tp, ep=ep)
    return (b.weight_read_s + b.kv_read_s) * 1e3 / efficiency + b.comms_s * 1e3 + host_ms


def latency_budget(prompt_tokens: int = 512, new_tokens: int = 256, turns: int = 1, prefill_tok_s: float = 1500.0,
                   prefix_cache: bool = False, spec_tau: float = 1.0, spec_cost: float = 1.0, **tpot_kw) -> dict:
    """TTFT + N x TPOT of a chat: with a prefix cache a later turn prefills only the new user text."""
    tpot = modelled_tpot_ms(**tpot_kw) * spec_cost / max(1.0, spec_tau)
    total, ctx, per_turn = 0.0, 0, []
    for t in range(turns):
        fresh = prompt_tokens if (t == 0 or prefix_cache) else ctx + prompt_tokens
        ttft = fresh / prefill_tok_s * 1e3 + tpot
        turn = ttft + (new_tokens - 1) * tpot
        per_turn.append({"turn": t, "ttft_ms": ttft, "turn_ms": turn})
        total += turn
        ctx += prompt_tokens + new_tokens
    return {"tpot_ms": tpot, "tok_s": 1000.0 / tpot, "turns": per_turn, "total_ms": total}


def predict_matrix(efficiency: float = 0.46, gpu: str = "B200-SXM-180GB", collective_us: Optional[float] = None,
                   n_gpus: int = 8, cfg: MoEConfig = QWEN3_235B) -> List[dict]:
    """Predicted B = 1 tok/s over layout x precision x context: analytical floor and floor x efficiency."""
    g = GPUS[gpu] if gpu in GPUS else measured_b200()
    if collective_us is not None:
        g = dataclasses.replace(g, collective_latency_s=collective_us * 1e-6)
    cl = Cluster(g, n_gpus)
    layouts = [("tp", n_gpus, 1)] + [("hybrid", n_gpus // e, e) for e in (2, 4) if n_gpus % e == 0 and e < n_gpus] + \
              [("ep", 1, n_gpus)]
    rows = []
    for dtype, name in ((1, "fp8"), (2, "bf16")):
        for seq in (2048, 8192, 32768):
            for plan, tp, ep in layouts:
                b = decode_latency(cfg, cl, plan=plan, dtype_bytes=dtype, seq_len=seq, tp=tp, ep=ep)
                real = (b.weight_read_s + b.kv_read_s + b.compute_s) / efficiency + b.comms_s
                rows.append({"dtype": name, "ctx": seq, "plan": plan, "tp": tp, "ep": ep,
                             "floor_tok_s": b.tokens_per_s, "real_tok_s": 1.0 / real})
    return rows


# ---- speculative decoding: unified predictor and tree-shape search ------------------------------------------------------------------
def spec_predict(floor: float, alpha: float, width: int, depth: int, layout: str = "tp", n_ranks: int = 8,
                 draft_ms_per_step: float = 0.0, decode_step_ms: float = 3.74, temperature: float = 0.0,
                 overlap: float = 0.0, n_experts: int = 128, top_k: int = 8) -> dict:
    """speedup = E[emitted] / (verify cost + draft cost). Sampling lowers acceptance (about 0.8x at temperature
    0.7); on expert parallelism the busiest-rank factor of the expert term falls toward 1 as the union fills."""
    a = alpha * (1.0 - 0.2 * min(1.0, temperature / 0.7))
    positions = width * depth
    union = expert_union(positions, n_experts, top_k, overlap)
    ep_factor = 1.0
    if layout == "ep":
        base = expected_max_experts_per_gpu(top_k, n_ranks) / (top_k / n_ranks)
        fill = union / n_experts
        ep_factor = (base * (1.0 - fill) + 1.0 * fill) / base
    cost = floor_verify_cost(floor, union, top_k, ep_factor)
    draft = draft_ms_per_step * depth / decode_step_ms
    emitted = expected_emitted(a, depth, width)
    return {"width": width, "depth": depth, "positions": positions, "union": union, "emitted": emitted,
            "verify_cost": cost, "draft_cost": draft, "speedup": emitted / (cost + draft)}


def tree_optimizer(floor: float, alpha: float, widths=(1, 2, 4, 8), depths=(2, 3, 4, 6, 8), **kw) -> List[dict]:
    rows = [spec_predict(floor, alpha, w, d, **kw) for w in widths for d in depths]
    return sorted(rows, key=lambda r: r["speedup"], reverse=True)


def verify_cost_check(tree_sizes=(1, 2, 3, 5, 8, 16), expert_bytes: float = 18.9e6 * 94, nonexpert_bytes: float = 6.7e9,
                      aggregate_bw: float = 8 * 7.7e12, n_experts: int = 128, top_k: int = 8) -> List[dict]:
    """What a correctly batched verify reads: the union of experts ONCE (a grouped GEMM), not top-k experts per
    position. The ratio is the error of a per-position model and the target a verify kernel is checked against."""
    rows = []
    for m in tree_sizes:
        u = expert_union(m, n_experts, top_k)
        wrong = (nonexpert_bytes + m * top_k * expert_bytes) / aggregate_bw * 1e3
        right = (nonexpert_bytes + u * expert_bytes) / aggregate_bw * 1e3
        rows.append({"positions": m, "union": u, "per_position_ms": wrong, "union_once_ms": right, "ratio": wrong / right})
    return rows


def spec_analyze(base_tok_s: float, spec_tok_s: float, accepted_tokens: float, drafts: float, positions: int,
                 floor_hint: Optional[float] = None, best_plain_tok_s: Optional[float] = None, top_k: int = 8) -> dict:
    """From one speculative run and its matched baseline: S, tau = 1 + accepted / drafts, V = tau / S and the expert
    union that V implies (inverting the floor-aware cost when a floor share is given). V near 1: the verify hides
    under the floor, shaping the tree by routes cannot pay; V well above 1: the union is taxed and it can."""
    s = spec_tok_s / base_tok_s
    tau = 1.0 + accepted_tokens / max(1.0, drafts)
    v = tau / s
    out = {"S": s, "tau": tau, "V": v, "route_aware": "no-go" if v < 1.15 else "go" if v > 1.5 else "marginal"}
    if floor_hint is not None and floor_hint < 1.0:
        w = (v - floor_hint) / (1.0 - floor_hint)
        out["implied_union"] = max(0.0, (w - NONEXPERT_SHARE) / ROUTED_SHARE * top_k)
        out["model_union"] = expert_union(positions)
    if best_plain_tok_s:
        out["vs_best_plain"] = spec_tok_s / best_plain_tok_s
    return out


# ---- layout questions -------------------------------------------------------------------------------------------------------------------
def stale_tp_ceiling(n_layers: int = 94, collective_us: float = 10.0, weight_read_us_per_layer: float = 4.4,
                     other_us_per_layer: float = 45.0, kv_ms: float = 0.02, refresh_every: int = 2) -> dict:
    """If a stale (not yet reduced) activation may feed the next layer, a collective hides behind that layer's
    weight read: only refresh layers wait. Ceiling on the step time IF quality holds."""
    serial = n_layers * (2 * collective_us + weight_read_us_per_layer + other_us_per_layer) / 1e3 + kv_ms
    exposed = 2 * collective_us / refresh_every
    hidden = max(0.0, 2 * collective_us * (1 - 1 / refresh_every) - weight_read_us_per_layer - other_us_per_layer)
    stale = n_layers * (exposed + hidden + weight_read_us_per_layer + other_us_per_layer) / 1e3 + kv_ms
    return {"serial_ms": serial, "stale_ms": stale, "speedup": serial / stale, "tok_s": 1000.0 / stale}


def tp_degree(degrees=(1, 2, 4, 8), collective_us_at_8: float = 10.0, algorithm: str = "oneshot", efficiency: float = 0.5,
              host_ms: float = 0.0, dtype_bytes: int = 1, ctx: int = 512, gpu: str = "B200-SXM-180GB",
              cfg: MoEConfig = QWEN3_235B) -> List[dict]:
    """Single stream on N GPUs with the others idle: the weight read scales as 1 / N, a one-shot collective is flat
    in N, a ring one grows with N - 1."""
    rows = []
    for n in degrees:
        c = collective_us_at_8 if algorithm == "oneshot" else collective_us_at_8 * max(1, n - 1) / 7.0
        if n == 1:
            c = 0.0
        g = dataclasses.replace(GPUS[gpu], collective_latency_s=c * 1e-6)
        b = decode_latency(cfg, Cluster(g, n), plan="tp", dtype_bytes=dtype_bytes, seq_len=ctx, tp=n, ep=1)
        fits = cfg.total_params * dtype_bytes <= 0.9 * n * g.hbm_bytes
        t = (b.weight_read_s + b.kv_read_s) / efficiency + b.comms_s + host_ms / 1e3
        rows.append({"gpus": n, "collective_us": c, "weight_ms": b.weight_read_s * 1e3 / efficiency,
                     "comms_ms": b.comms_s * 1e3, "tpot_ms": t * 1e3, "tok_s": 1.0 / t, "fits": fits})
    return rows


def mbu_ceiling(byte_floor_ms: float, latency_bound_us_per_layer: Dict[str, float], n_layers: int = 94,
                bandwidth_bound_share: float = 1.0, kernel_mbu: float = 0.8, fused_phase_us: float = 3.0) -> dict:
    """Applying a per-kernel bandwidth efficiency to the whole byte budget over-promises: the ops that are latency
    bound (a fixed time per call per layer) do not shrink with bandwidth tuning. Un-fused ceiling = bytes at the
    kernel efficiency + the fixed costs; the fused (one kernel per token) ceiling replaces every fixed cost by one
    phase hand-over."""
    fixed = sum(latency_bound_us_per_layer.values()) * n_layers / 1e3
    bw = byte_floor_ms * bandwidth_bound_share / kernel_mbu
    unfused = bw + fixed
    fused = bw + len(latency_bound_us_per_layer) * fused_phase_us * n_layers / 1e3
    return {"bandwidth_ms": bw, "fixed_ms": fixed, "unfused_ms": unfused, "unfused_tok_s": 1000.0 / unfused,
            "whole_engine_mbu_unfused": byte_floor_ms / unfused, "fused_ms": fused, "fused_tok_s": 1000.0 / fused}


# ---- Monte-Carlo check of the routing formulas the models above rest on -----------------------------------------------------------------------
def validate_routing_model(trials: int = 4000, n_experts: int = 128, top_k: int = 8, n_ranks: int = 8, seed: int = 0,
                           positions=(1, 2, 4, 8, 16, 32)) -> dict:
    rng = random.Random(seed)
    per_rank = n_experts // n_ranks
    union_rows, balance_rows = [], []
    for p in positions:
        tot_u, tot_imb = 0.0, 0.0
        for _ in range(trials):
            lit = set()
            for _ in range(p):
                lit.update(rng.sample(range(n_experts), top_k))
            tot_u += len(lit)
            load = [0] * n_ranks
            for e in lit:
                load[e // per_rank] += 1
            tot_imb += max(load) / (len(lit) / n_ranks)
        union_rows.append({"positions": p, "simulated": tot_u / trials, "formula": expert_union(p, n_experts, top_k)})
        balance_rows.append({"positions": p, "busiest_over_mean": tot_imb / trials})
    busiest = 0.0
    for _ in range(trials):
        load = [0] * n_ranks
        for e in rng.sample(range(n_experts), top_k):
            load[e // per_rank] += 1
        busiest += max(load)
    # experts are drawn without replacement, the closed form assumes independent bins: close, not identical
    return {"union": union_rows, "verify_imbalance": balance_rows,
            "busiest_rank": {"simulated": busiest / trials, "formula": expected_max_experts_per_gpu(top_k, n_ranks)}}


# ---- CLI ----------------------------------------------------------------------------------------------------------------------------------------
# ---- strong-scaling fit ------------------------------------------------------------------------------------------------------------
# this engine, Qwen3-235B-A22B block-fp8, context 1024, ms per token at 1 / 2 / 4 / 8 B200s (persistent kernel)
B200_SCALING_MS = ((1, 8.14), (2, 6.23), (4, 4.52), (8, 3.744))


def scaling_fit(points: Sequence[Tuple[int, float]] = B200_SCALING_MS, bytes_per_token: float = 21.7e9,
                hbm_bw: float = 6.5616e12, n_layers: int = 94) -> dict:
    """Least-squares fit of ``t(N) = a * (bytes / N) / bw + fixed`` to measured ms per token at N GPUs: ``a`` is the
    inverse bandwidth efficiency of the byte-proportional part (1 = streaming at the measured copy bandwidth) and
    ``fixed`` the part that more GPUs do not shrink (the per-layer latency chain plus the head and the token turn-around),
    reported per layer. Also: the time each term takes at every N, and what N GPUs would give with the fixed part halved."""
    xs = [bytes_per_token / n / hbm_bw * 1e3 for n, _ in points]            # ms of HBM time at the copy bandwidth
    ys = [ms for _, ms in points]
    k = len(points)
    mx, my = sum(xs) / k, sum(ys) / k
    sxx = sum((x - mx) ** 2 for x in xs)
    a = sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / sxx if sxx > 0 else 0.0
    fixed = my - a * mx
    rows = []
    for (n, ms), x in zip(points, xs):
        pred = a * x + fixed
        rows.append({"n_gpus": n, "measured_ms": ms, "fit_ms": pred, "byte_part_ms": a * x, "fixed_ms": fixed,
                     "fixed_share": fixed / pred, "tok_s": 1000.0 / ms, "tok_s_if_fixed_halves": 1000.0 / (a * x + fixed / 2)})
    return {"bandwidth_efficiency": 1.0 / a if a > 0 else float("inf"), "fixed_ms": fixed,
            "fixed_us_per_layer": fixed * 1e3 / n_layers, "rows": rows,
            "max_fit_error_ms": max(abs(r["fit_ms"] - r["measured_ms"]) for r in rows)}


def _table(rows: List[dict]) -> str:
    if not rows:
        return ""
    cols = list(rows[0].keys())

    def fmt(v):
        if isinstance(v, float):
            return f"{v:.3f}"
        return str(v)
    width = {c: max(len(c), *(len(fmt(r.get(c))) for r in rows)) for c in cols}
    lines = ["  ".join(c.rjust(width[c]) for c in cols)]
    lines += ["  ".join(fmt(r.get(c)).rjust(width[c]) for c in cols) for r in rows]
    return "\n".join(lines)


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m inferutil.studies")
    sub = p.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("floor", help="back the floor share out of (k, tau, S) triples")
    s.add_argument("triples", nargs="+", help="k:tau:S")
    s = sub.add_parser("reconcile", help="which per-collective latency fits the measured step time")
    s.add_argument("--tpot-ms", type=float, default=3.74)
    s.add_argument("--collectives", type=int, default=188)
    s.add_argument("--weight-floor-ms", type=float, default=0.43)
    s.add_argument("--efficiency", type=float, default=0.45)
    s.add_argument("--candidates", type=float, nargs="+", default=[3, 5, 10, 16, 25, 35])
    sub.add_parser("ladder", help="tok/s after each lever")
    s = sub.add_parser("budget", help="TTFT + N x TPOT of a chat")
    s.add_argument("--plan", default="tp"); s.add_argument("--tp", type=int, default=8); s.add_argument("--ep", type=int, default=1)
    s.add_argument("--dtype", type=int, default=1); s.add_argument("--collective-us", type=float, default=10.0)
    s.add_argument("--eff", type=float, default=0.45); s.add_argument("--host-ms", type=float, default=0.0)
    s.add_argument("--prompt", type=int, default=512); s.add_argument("--new", type=int, default=256)
    s.add_argument("--turns", type=int, default=1); s.add_argument("--prefix-cache", action="store_true")
    s.add_argument("--spec-tau", type=float, default=1.0); s.add_argument("--spec-cost", type=float, default=1.0)
    s = sub.add_parser("matrix", help="predicted tok/s over layout x precision x context")
    s.add_argument("--eff", type=float, default=0.46); s.add_argument("--gpu", default="B200-SXM-180GB")
    s.add_argument("--collective-us", type=float, default=None)
    s = sub.add_parser("tree", help="best speculative tree shapes")
    s.add_argument("--floor", type=float, default=0.8); s.add_argument("--alpha", type=float, default=0.7)
    s.add_argument("--layout", default="tp"); s.add_argument("--draft-ms", type=float, default=0.0)
    s.add_argument("--temp", type=float, default=0.0); s.add_argument("--overlap", type=float, default=0.0)
    s = sub.add_parser("tp-degree", help="fewer GPUs for one stream?")
    s.add_argument("--algorithm", default="oneshot", choices=["oneshot", "ring"])
    s.add_argument("--collective-us", type=float, default=10.0)
    sub.add_parser("verify-cost", help="union-once vs per-position verify bytes")
    s = sub.add_parser("stale-tp", help="ceiling of hiding collectives behind the next layer")
    s.add_argument("--collective-us", type=float, default=10.0); s.add_argument("--refresh", type=int, default=2)
    s = sub.add_parser("routing-check", help="Monte-Carlo check of the union / busiest-rank formulas")
    s.add_argument("--trials", type=int, default=2000)
    s = sub.add_parser("scaling-fit", help="byte-proportional and fixed part of ms per token over the GPU count")
    s.add_argument("points", nargs="*", help="N:ms pairs (default: this engine's measured 1 / 2 / 4 / 8 B200 figures)")
    s = sub.add_parser("spec-analyze", help="S, tau, V and the go/no-go from one speculative run")
    s.add_argument("--base", type=float, required=True); s.add_argument("--spec", type=float, required=True)
    s.add_argument("--accepted", type=float, required=True); s.add_argument("--drafts", type=float, required=True)
    s.add_argument("--positions", type=int, default=5); s.add_argument("--floor", type=float, default=None)
    a = p.parse_args(argv)
    if a.cmd == "floor":
        meas = [tuple(float(x) for x in t.split(":")) for t in a.triples]
        print(json.dumps(backout_floor([(int(k), tau, s_) for k, tau, s_ in meas]), indent=1))
    elif a.cmd == "reconcile":
        print(_table(comms_reconcile(a.tpot_ms, a.collectives, a.weight_floor_ms, a.efficiency, a.candidates)))
    elif a.cmd == "ladder":
        print(_table([{k: v for k, v in r.items()} for r in ladder()]))
    elif a.cmd == "budget":
        r = latency_budget(a.prompt, a.new, a.turns, prefix_cache=a.prefix_cache, spec_tau=a.spec_tau,
                           spec_cost=a.spec_cost, plan=a.plan, tp=a.tp, ep=a.ep, dtype_bytes=a.dtype,
                           collective_us=a.collective_us, efficiency=a.eff, host_ms=a.host_ms, ctx=a.prompt)
        print(f"TPOT {r['tpot_ms']:.3f} ms ({r['tok_s']:.1f} tok/s), total {r['total_ms']:.1f} ms")
        print(_table(r["turns"]))
    elif a.cmd == "matrix":
        print(_table(predict_matrix(a.eff, a.gpu, a.collective_us)))
    elif a.cmd == "tree":
        print(_table(tree_optimizer(a.floor, a.alpha, layout=a.layout, draft_ms_per_step=a.draft_ms,
                                    temperature=a.temp, overlap=a.overlap)[:10]))
    elif a.cmd == "tp-degree":
        print(_table(tp_degree(algorithm=a.algorithm, collective_us_at_8=a.collective_us)))
    elif a.cmd == "verify-cost":
        print(_table(verify_cost_check()))
    elif a.cmd == "stale-tp":
        print(json.dumps(stale_tp_ceiling(collective_us=a.collective_us, refresh_every=a.refresh), indent=1))
    elif a.cmd == "routing-check":
        print(json.dumps(validate_routing_model(a.trials), indent=1))
    elif a.cmd == "scaling-fit":
        pts = [(int(t.split(":")[0]), float(t.split(":")[1])) for t in a.points] or B200_SCALING_MS
        r = scaling_fit(pts)
        print(f"byte part streams at {100 * r['bandwidth_efficiency']:.0f} % of the copy bandwidth; fixed part "
              f"{r['fixed_ms']:.2f} ms = {r['fixed_us_per_layer']:.1f} us per layer; worst fit error {r['max_fit_error_ms']:.2f} ms")
        print(_table(r["rows"]))
    elif a.cmd == "spec-analyze":
        print(json.dumps(spec_analyze(a.base, a.spec, a.accepted, a.drafts, a.positions, a.floor), indent=1))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
