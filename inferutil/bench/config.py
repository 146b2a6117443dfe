"""Benchmark configuration (reference: src/inferutil/bench/config.py:7-30)."""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, fields


@dataclass(frozen=True)
class BenchConfig:
    name: str
    plan: str                  # "tp" | "ep" | "hybrid"
    dtype_bytes: int           # 2 = bf16, 1 = fp8
    kv_dtype_bytes: int
    tp: int
    ep: int
    prompt_tokens: int = 512
    decode_tokens: int = 128
    seed: int = 0
    warmup_steps: int = 8
    repeats: int = 5

    @property
    def seq_len(self) -> int:
        return self.prompt_tokens + self.decode_tokens


def config_id(config: BenchConfig) -> str:
    """12 hex characters derived from every field, in declaration order."""
    text = "|".join(str(getattr(config, f.name)) for f in fields(config))
    return hashlib.sha256(text.encode()).hexdigest()[:12]
