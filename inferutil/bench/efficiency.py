"""MFU / MBU / arithmetic intensity / roofline regime (reference: src/inferutil/bench/efficiency.py:31-144)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


def flops_per_token(active_params: int, *, seq_len: int = 0, n_layers: int = 0, d_model: int = 0,
                    include_attention: bool = False) -> float:
    f = 2.0 * active_params
    if include_attention and seq_len and n_layers and d_model:
        f += 2.0 * n_layers * seq_len * d_model
    return f


def mfu(tok_s: Optional[float], active_params: int, peak_flops: float) -> Optional[float]:
    if tok_s is None or not peak_flops or not active_params:
        return None
    return tok_s * flops_per_token(active_params) / peak_flops


def mbu(tok_s: Optional[float], bytes_per_token: Optional[float], peak_bw: float) -> Optional[float]:
    if tok_s is None or bytes_per_token is None or not peak_bw:
        return None
    return tok_s * bytes_per_token / peak_bw


def achieved_tflops(tok_s: Optional[float], active_params: int) -> Optional[float]:
    if tok_s is None or not active_params:
        return None
    return tok_s * flops_per_token(active_params) * 1e-12


def arithmetic_intensity_decode(active_params: int, bytes_per_token: Optional[float]) -> Optional[float]:
    return flops_per_token(active_params) / bytes_per_token if bytes_per_token else None


def arithmetic_intensity_prefill(active_params: int, weight_bytes: Optional[float], prompt_tokens: int) -> Optional[float]:
    return flops_per_token(active_params) * prompt_tokens / weight_bytes if weight_bytes else None


def roofline_ridge(peak_flops: float, peak_bw: float) -> Optional[float]:
    return peak_flops / peak_bw if peak_bw else None


def classify_regime(ai: Optional[float], ridge: Optional[float]) -> str:
    if ai is None or ridge is None:
        return "unknown"
    return "compute-bound" if ai >= ridge else "memory-bound"


def peak_flops_for_dtype(bf16_flops: float, fp8_flops: float, dtype_bytes: float) -> float:
    return bf16_flops if dtype_bytes >= 2 else fp8_flops


@dataclass(frozen=True)
class Efficiency:
    mfu_prefill: Optional[float]
    mfu_decode: Optional[float]
    mbu_decode: Optional[float]
    achieved_tflops_prefill: Optional[float]
    achieved_tflops_decode: Optional[float]
    ai_decode: Optional[float]
    ai_prefill: Optional[float]
    roofline_ridge: Optional[float]
    regime_decode: str = "unknown"
    regime_prefill: str = "unknown"
    kv_byte_share: Optional[float] = None


def compute_efficiency(*, active_params: int, weight_bytes: float, bytes_per_token: float, kv_bytes: float,
                       prompt_tokens: int, prefill_tok_s: Optional[float], decode_tok_s: Optional[float],
                       peak_flops: float, peak_bw: float) -> Efficiency:
    """``peak_flops`` / ``peak_bw`` are node aggregates; ``bytes_per_token`` includes the KV bytes."""
    ridge = roofline_ridge(peak_flops, peak_bw)
    ai_d = arithmetic_intensity_decode(active_params, bytes_per_token)
    ai_p = arithmetic_intensity_prefill(active_params, weight_bytes, prompt_tokens)
    return Efficiency(mfu_prefill=mfu(prefill_tok_s, active_params, peak_flops),
                      mfu_decode=mfu(decode_tok_s, active_params, peak_flops),
                      mbu_decode=mbu(decode_tok_s, bytes_per_token, peak_bw),
                      achieved_tflops_prefill=achieved_tflops(prefill_tok_s, active_params),
                      achieved_tflops_decode=achieved_tflops(decode_tok_s, active_params),
                      ai_decode=ai_d, ai_prefill=ai_p, roofline_ridge=ridge,
                      regime_decode=classify_regime(ai_d, ridge), regime_prefill=classify_regime(ai_p, ridge),
                      kv_byte_share=(kv_bytes / bytes_per_token if bytes_per_token else None))
