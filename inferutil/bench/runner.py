"""Fixed-window B=1 benchmark driver over the ``Engine`` seam (reference: src/inferutil/bench/runner.py:10-72).
Per repeat: prefill ``range(prompt_tokens)``, discard warm-up steps, time ``decode_tokens - 1`` steps; telemetry
brackets only the last repeat's timed window."""
from __future__ import annotations

from ..hardware import Cluster
from ..model import MoEConfig
from .config import BenchConfig
from .metrics import BenchResult, build_result, summarize_telemetry
from .telemetry import NullTelemetry


def run_benchmark(engine, config: BenchConfig, cfg: MoEConfig, cluster: Cluster, telemetry=None, reference_ids=None,
                  collect_ids: bool = False) -> BenchResult:
    if config.decode_tokens < 2:
        raise ValueError("decode_tokens must be >= 2 (need inter-token samples)")
    telemetry = telemetry or NullTelemetry()
    engine.reset(plan=config.plan, dtype_bytes=config.dtype_bytes, kv_dtype_bytes=config.kv_dtype_bytes,
                 tp=config.tp, ep=config.ep, seq_len=config.seq_len)
    tok_s_runs, ttft_runs, e2e_runs = [], [], []
    steps, gpu_samples = [], []
    ttft = prefill_rate = 0.0
    for rep in range(config.repeats):
        pre = engine.prefill(list(range(config.prompt_tokens)))
        ttft = pre.seconds + pre.first_token_seconds
        ttft_runs.append(ttft)
        prefill_rate = pre.n_prompt_tokens / pre.seconds if pre.seconds else 0.0   # 0, not inf: stays valid JSON
        for _ in range(config.warmup_steps):
            engine.decode_step()
        last = rep == config.repeats - 1
        if last:
            telemetry.start()
        steps = [engine.decode_step() for _ in range(config.decode_tokens - 1)]
        if last:
            gpu_samples = telemetry.stop()
        window = sum(s.seconds for s in steps)
        tok_s_runs.append(len(steps) / window if window else float("inf"))
        e2e_runs.append(ttft + window)
    seconds = [s.seconds for s in steps]
    ids = [s.token_id for s in steps]
    quality = None
    if reference_ids is not None:
        from .quality import match_rate
        quality = match_rate(ids, reference_ids)
    result = build_result(cfg=cfg, cluster=cluster, config=config, ttft_s=ttft, prefill_tok_per_s=prefill_rate,
                          decode_step_seconds=seconds,
                          telemetry_summary=summarize_telemetry(gpu_samples, config.decode_tokens, sum(seconds)),
                          decode_tok_per_s_samples=tok_s_runs, step_breakdowns=[s.breakdown for s in steps],
                          quality=quality, ttft_samples=ttft_runs, e2e_samples=e2e_runs)
    if collect_ids:
        object.__setattr__(result, "generated_token_ids", ids)
    return result
