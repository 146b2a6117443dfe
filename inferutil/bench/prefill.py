"""Batched-prefill roofline (reference: src/inferutil/bench/prefill.py:32-63)."""
from __future__ import annotations

from ..hardware import Cluster
from ..model import MoEConfig
from .efficiency import peak_flops_for_dtype


def expected_distinct_experts(n_experts: int, top_k: int, prompt_tokens: int) -> float:
    """E[experts of a layer touched by a prompt] = E (1 - ((E - k) / E) ** P)."""
    if n_experts <= 0 or prompt_tokens <= 0:
        return 0.0
    return n_experts * (1.0 - ((n_experts - top_k) / n_experts) ** prompt_tokens)


def prefill_weight_bytes(cfg: MoEConfig, dtype_bytes: float, prompt_tokens: int) -> float:
    experts_all = cfg.n_layers * cfg.n_experts * cfg.one_expert_params
    touched = cfg.n_layers * cfg.one_expert_params * expected_distinct_experts(cfg.n_experts, cfg.top_k, prompt_tokens)
    return dtype_bytes * (cfg.total_params - experts_all + touched)


def prefill_latency(cfg: MoEConfig, cluster: Cluster, *, dtype_bytes: float, kv_dtype_bytes: int,
                    prompt_tokens: int) -> float:
    """max(weight read, compute) + KV write, on node aggregates."""
    if prompt_tokens <= 0:
        return 0.0
    bw = cluster.aggregate_hbm_bw
    peak = cluster.n_gpus * peak_flops_for_dtype(cluster.gpu.bf16_flops, cluster.gpu.fp8_flops, dtype_bytes)
    read_s = prefill_weight_bytes(cfg, dtype_bytes, prompt_tokens) / bw
    math_s = 2.0 * cfg.active_params * prompt_tokens / peak
    return max(read_s, math_s) + prompt_tokens * cfg.kv_bytes_per_token(kv_dtype_bytes) / bw
