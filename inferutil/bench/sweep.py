"""Analytical sweeps over context depth, quantisation and tp x ep layout (reference: src/inferutil/bench/sweep.py:28-149)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

from ..hardware import Cluster
from ..latency import decode_latency
from ..model import MoEConfig
from .attribution import dominant_of_breakdown, lever_hint
from .config import BenchConfig
from .efficiency import compute_efficiency, peak_flops_for_dtype


@dataclass(frozen=True)
class SweepPoint:
    label: str
    seq_len: int
    plan: str
    dtype_bytes: float
    kv_dtype_bytes: int
    tp: int
    ep: int
    decode_tok_s: float
    tpot_ms: float
    mbu_decode: Optional[float]
    mfu_decode: Optional[float]
    kv_byte_share: Optional[float]
    regime: str
    dominant_term: str
    hint: str


def realized_efficiency(cfg: MoEConfig, cluster: Cluster, config: BenchConfig, measured_tok_s: float):
    """``(measured / analytical floor, floor tok/s)``: feed the ratio back as ``--efficiency``."""
    floor = decode_latency(cfg, cluster, plan=config.plan, dtype_bytes=config.dtype_bytes,
                           kv_dtype_bytes=config.kv_dtype_bytes, seq_len=config.seq_len, tp=config.tp,
                           ep=config.ep).tokens_per_s
    return (measured_tok_s / floor if floor else None), floor


def _point(cfg: MoEConfig, cluster: Cluster, *, label: str, plan: str, dtype_bytes: float, kv_dtype_bytes: int,
           tp: int, ep: int, seq_len: int, efficiency: float = 1.0) -> SweepPoint:
    b = decode_latency(cfg, cluster, plan=plan, dtype_bytes=dtype_bytes, kv_dtype_bytes=kv_dtype_bytes,
                       seq_len=seq_len, tp=tp, ep=ep)
    rate = b.tokens_per_s * efficiency
    w_bytes = cfg.active_params * dtype_bytes
    kv_bytes = seq_len * cfg.kv_bytes_per_token(kv_dtype_bytes)
    peak = cluster.n_gpus * peak_flops_for_dtype(cluster.gpu.bf16_flops, cluster.gpu.fp8_flops, dtype_bytes)
    e = compute_efficiency(active_params=cfg.active_params, weight_bytes=w_bytes, bytes_per_token=w_bytes + kv_bytes,
                           kv_bytes=kv_bytes, prompt_tokens=seq_len, prefill_tok_s=None, decode_tok_s=rate,
                           peak_flops=peak, peak_bw=cluster.aggregate_hbm_bw)
    dom = dominant_of_breakdown(b.weight_read_s, b.kv_read_s, b.comms_s, b.compute_s)
    return SweepPoint(label, seq_len, plan, dtype_bytes, kv_dtype_bytes, tp, ep, rate,
                      1000.0 / rate if rate else float("inf"), e.mbu_decode, e.mfu_decode, e.kv_byte_share,
                      e.regime_decode, dom, lever_hint(dom))


def depth_sweep(cfg: MoEConfig, cluster: Cluster, config: BenchConfig, depths: List[int],
                efficiency: float = 1.0) -> List[SweepPoint]:
    return [_point(cfg, cluster, label=f"ctx{d}", plan=config.plan, dtype_bytes=config.dtype_bytes,
                   kv_dtype_bytes=config.kv_dtype_bytes, tp=config.tp, ep=config.ep, seq_len=d, efficiency=efficiency)
            for d in depths]


def _variant(base: BenchConfig, name: str, **changes) -> BenchConfig:
    fields = dict(plan=base.plan, dtype_bytes=base.dtype_bytes, kv_dtype_bytes=base.kv_dtype_bytes, tp=base.tp,
                  ep=base.ep, prompt_tokens=base.prompt_tokens, decode_tokens=base.decode_tokens)
    fields.update(changes)
    return BenchConfig(name=name, **fields)


def quant_grid(base: BenchConfig, dtypes=(2, 1, 0.5), kv_dtypes=(2, 1)) -> List[BenchConfig]:
    return [_variant(base, f"w{d}b-kv{kv}b", dtype_bytes=d, kv_dtype_bytes=kv) for d in dtypes for kv in kv_dtypes]


def _divisors(n: int) -> List[int]:
    return [d for d in range(1, n + 1) if n % d == 0]


def layout_grid(base: BenchConfig, n_gpus: int) -> List[BenchConfig]:
    return [_variant(base, f"tp{tp}-ep{ep}", tp=tp, ep=ep) for tp in _divisors(n_gpus) for ep in _divisors(n_gpus)]


def full_grid(base: BenchConfig, n_gpus: int, dtypes=(2, 1, 0.5), kv_dtypes=(2, 1)) -> List[BenchConfig]:
    return [_variant(base, f"w{d}b-kv{kv}b-tp{tp}-ep{ep}", dtype_bytes=d, kv_dtype_bytes=kv, tp=tp, ep=ep)
            for d in dtypes for kv in kv_dtypes for tp in _divisors(n_gpus) for ep in _divisors(n_gpus)]


def config_sweep(cfg: MoEConfig, cluster: Cluster, configs: List[BenchConfig], efficiency: float = 1.0) -> List[SweepPoint]:
    pts = [_point(cfg, cluster, label=c.name, plan=c.plan, dtype_bytes=c.dtype_bytes, kv_dtype_bytes=c.kv_dtype_bytes,
                  tp=c.tp, ep=c.ep, seq_len=c.seq_len, efficiency=efficiency) for c in configs]
    return sorted(pts, key=lambda p: p.decode_tok_s, reverse=True)
