"""Roofline model of one decoded token at batch 1 (reference: src/inferutil/latency.py:31-165).

token time = active-weight read + KV read + compute + per-layer collectives, under a parallel plan:
``tp`` (everything split over all GPUs, 2 collectives per layer), ``ep`` / ``hybrid`` (attention over ``tp`` GPUs,
experts owned by ``ep`` GPUs, the busiest owner sets the pace, 3 collectives per layer) and ``floor`` (perfect split,
no communication).
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache
from math import comb

from .hardware import Cluster
from .model import MoEConfig


@lru_cache(maxsize=None)
def _prob_max_at_most(balls: int, bins: int, cap: int) -> float:
    """P(no bin holds more than ``cap``) for ``balls`` thrown uniformly into ``bins``: count the capped
    compositions with a polynomial power, divide by bins ** balls."""
    if cap * bins < balls:
        return 0.0
    # ways[j] = number of ordered assignments (labelled balls) using j balls with every bin <= cap,
    # built bin by bin with exponential generating function coefficients (j! * [x^j] (sum_{i<=cap} x^i/i!)^bins)
    ways = [1.0] + [0.0] * balls
    for _ in range(bins):
        nxt = [0.0] * (balls + 1)
        for used, w in enumerate(ways):
            if w == 0.0:
                continue
            for take in range(0, min(cap, balls - used) + 1):
                nxt[used + take] += w * comb(balls - used, take)
        ways = nxt
    return ways[balls] / float(bins ** balls)


def expected_max_experts_per_gpu(top_k: int, ep: int) -> float:
    """E[load of the busiest owner] when ``top_k`` expert choices fall uniformly on ``ep`` owners."""
    if ep <= 1:
        return float(top_k)
    # E[max] = sum_{m >= 1} P(max >= m)
    return sum(1.0 - _prob_max_at_most(top_k, ep, m - 1) for m in range(1, top_k + 1))


@dataclass
class DecodeBreakdown:
    plan: str
    dtype_bytes: int
    seq_len: int
    weight_read_s: float
    kv_read_s: float
    compute_s: float
    comms_s: float
    imbalance: float

    @property
    def total_s(self) -> float:
        return self.weight_read_s + self.kv_read_s + self.compute_s + self.comms_s

    @property
    def tokens_per_s(self) -> float:
        t = self.total_s
        return 1.0 / t if t else float("inf")

    def as_row(self) -> dict:
        def ms(x):
            return round(1e3 * x, 3)
        return {"plan": self.plan, "dtype": "bf16" if self.dtype_bytes >= 2 else f"{self.dtype_bytes * 8}b",
                "seq": self.seq_len, "weight_ms": ms(self.weight_read_s), "kv_ms": ms(self.kv_read_s),
                "compute_ms": ms(self.compute_s), "comms_ms": ms(self.comms_s), "total_ms": ms(self.total_s),
                "tok_per_s": round(self.tokens_per_s, 1), "expert_imbalance": round(self.imbalance, 2)}


def decode_latency(cfg: MoEConfig, cluster: Cluster, *, plan: str = "hybrid", dtype_bytes: int = 2,
                   kv_dtype_bytes: int = 2, seq_len: int = 32768, tp: int | None = None, ep: int | None = None,
                   ideal_routing: bool = False, measured_max_experts: float | None = None,
                   kv_seq_split: bool = False) -> DecodeBreakdown:
    """``kv_seq_split``: the ranks that share a KV head (tp above the number of KV heads) split its cache rows between them
    instead of replicating them (two more small exchanges per layer, counted in ``comms``)."""
    gpu, n = cluster.gpu, cluster.n_gpus
    tp, ep = tp or n, ep or n
    layers = cfg.n_layers
    head_bytes = cfg.vocab * cfg.hidden * dtype_bytes
    attn_b = cfg.active_attn_params * dtype_bytes
    router_b = cfg.router_params * dtype_bytes
    expert_b = cfg.one_expert_params * dtype_bytes
    imbalance, comms = 1.0, 0.0
    if plan == "floor":
        weight_s = cfg.active_params * dtype_bytes / cluster.aggregate_hbm_bw
    elif plan == "tp":
        per_layer = (attn_b + router_b + cfg.top_k * expert_b) / n
        weight_s = (layers * per_layer + head_bytes / n) / gpu.hbm_bw
        comms = 2 * layers * gpu.collective_latency_s
    elif plan in ("ep", "hybrid"):
        fair = cfg.top_k / ep
        if measured_max_experts is not None:
            busiest = measured_max_experts
        elif ideal_routing:
            busiest = fair
        else:
            busiest = expected_max_experts_per_gpu(cfg.top_k, ep)
        imbalance = busiest / fair
        per_layer = attn_b / tp + router_b + busiest * expert_b
        weight_s = (layers * per_layer + head_bytes / n) / gpu.hbm_bw
        comms = 3 * layers * gpu.collective_latency_s
    else:
        raise ValueError(f"unknown plan {plan!r}")
    shards = n if plan == "floor" else min(tp, cfg.n_kv_heads)
    if kv_seq_split and plan != "floor" and tp > cfg.n_kv_heads:
        shards = tp                                        # every rank reads 1 / tp of the KV bytes
        comms += 2 * layers * gpu.collective_latency_s     # query gather + partial-record exchange inside a head's group
    kv_s = seq_len * cfg.kv_bytes_per_token(kv_dtype_bytes) / shards / gpu.hbm_bw
    flops = 2 * cfg.active_params + 4 * cfg.n_heads * cfg.head_dim * seq_len
    peak = gpu.fp8_flops if dtype_bytes < 2 else gpu.bf16_flops
    return DecodeBreakdown(plan=plan, dtype_bytes=dtype_bytes, seq_len=seq_len, weight_read_s=weight_s,
                           kv_read_s=kv_s, compute_s=flops / (peak * n), comms_s=comms, imbalance=imbalance)
