"""Turn a measured per-token latency into the ``x_summary`` optimisation block: floor breakdown
(weight / comms / kv / overhead, ms), regime, next lever, % of ceiling and % of roofline
(reference: server/optimization_telemetry.py:15-56, constants for 8xH100). The constants come from a
:class:`Profile` so that the same block can be computed for the machine the engine actually runs on."""
from __future__ import annotations

from dataclasses import dataclass

KV_BYTES = {"bf16": 2, "fp8": 1}
_DTYPE_BYTES = {"bf16": 2.0, "fp8": 1.0, "int4": 0.5}


@dataclass(frozen=True)
class Profile:
    """Node and model constants behind the breakdown."""
    agg_bw: float                 # aggregate HBM bandwidth, bytes/s
    active_params: float          # parameters read per token
    kv_bytes_per_token_elem: int  # 2 (k+v) * kv heads * head dim * layers (elements)
    n_collectives: int            # serial collectives per token
    ceiling_tok_s: float          # fp8 + optimal speculation

    def weight_ms(self, dtype: str) -> float:
        return 1e3 * self.active_params * _DTYPE_BYTES.get(dtype, 2.0) / self.agg_bw


# the reference's 8xH100 / Qwen3-235B-A22B constants (weight 1.61 / 0.80 / 0.40 ms)
H100X8 = Profile(agg_bw=8 * 3.35e12, active_params=21.57e9, kv_bytes_per_token_elem=2 * 4 * 128 * 94,
                 n_collectives=188, ceiling_tok_s=2000.0)
B200X8 = Profile(agg_bw=8 * 6.56e12, active_params=21.57e9, kv_bytes_per_token_elem=2 * 4 * 128 * 94,
                 n_collectives=188, ceiling_tok_s=4000.0)
B200X1 = Profile(agg_bw=6.56e12, active_params=21.57e9, kv_bytes_per_token_elem=2 * 4 * 128 * 94,
                 n_collectives=0, ceiling_tok_s=600.0)

WEIGHT_MS = {k: round(H100X8.weight_ms(k), 2) for k in _DTYPE_BYTES}
ROOFLINE_TOK_S = {k: round(1000.0 / v) * 1.0 for k, v in WEIGHT_MS.items()}
CEILING_TOK_S = H100X8.ceiling_tok_s
N_COLLECTIVES = H100X8.n_collectives


def kv_ms(ctx: int, kv_dtype: str = "bf16", profile: Profile = H100X8) -> float:
    return 1e3 * profile.kv_bytes_per_token_elem * KV_BYTES.get(kv_dtype, 2) * max(ctx, 0) / profile.agg_bw


def floor_breakdown(tpot_ms: float, weight_dtype: str = "bf16", kv_dtype: str = "bf16", collective_us: float = 16.0,
                    ctx: int = 512, profile: Profile = H100X8) -> dict:
    """``overhead`` is the residual: kernel inefficiency + launch + host time."""
    weight = profile.weight_ms(weight_dtype if weight_dtype in _DTYPE_BYTES else "bf16")
    comms = profile.n_collectives * collective_us / 1e3
    kv = kv_ms(ctx, kv_dtype, profile)
    return {"weight": round(weight, 3), "comms": round(comms, 3), "kv": round(kv, 3),
            "overhead": round(max(tpot_ms - weight - comms - kv, 0.0), 3)}


def summary_fields(tpot_ms: float, decode_tok_s: float, weight_dtype: str = "bf16", kv_dtype: str = "bf16",
                   collective_us: float = 16.0, ctx: int = 512, profile: Profile = H100X8) -> dict:
    bd = floor_breakdown(tpot_ms, weight_dtype, kv_dtype, collective_us, ctx, profile)
    floor_bound = bd["comms"] + bd["overhead"] + bd["kv"] >= bd["weight"]
    roof = 1000.0 / profile.weight_ms(weight_dtype if weight_dtype in _DTYPE_BYTES else "bf16")
    return {"floor_breakdown_ms": bd,
            "regime": "floor-bound" if floor_bound else "weight-bound",
            "next_lever": "spec + comms + kernels (fix the floor)" if floor_bound else "quant / route-aware (weight now pays)",
            "pct_of_ceiling": round(100.0 * decode_tok_s / profile.ceiling_tok_s, 1),
            "pct_of_roofline": round(100.0 * decode_tok_s / roof, 1)}
