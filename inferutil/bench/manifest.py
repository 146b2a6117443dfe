"""Reproducibility manifest written beside every stored run (reference: src/inferutil/bench/manifest.py:25-87)."""
from __future__ import annotations

import hashlib
import platform
import socket
import subprocess
import sys
from dataclasses import asdict, fields
from typing import Optional

from ..hardware import Cluster
from ..model import MoEConfig
from .config import BenchConfig, config_id

SCHEMA = "inferutil/bench/manifest/1"


def model_hash(cfg: MoEConfig) -> str:
    text = "|".join(str(getattr(cfg, f.name)) for f in fields(cfg))
    return hashlib.sha256(text.encode()).hexdigest()[:12]


def _git(*args: str) -> Optional[str]:
    try:
        p = subprocess.run(["git", *args], capture_output=True, text=True, timeout=2)
        return p.stdout.strip() if p.returncode == 0 else None
    except Exception:
        return None


def _git_commit() -> str:
    return _git("rev-parse", "HEAD") or "unknown"


def _git_dirty() -> bool:
    return bool(_git("status", "--porcelain"))


def build_manifest(cfg: MoEConfig, cluster: Cluster, config: BenchConfig, *, peak_bw_measured: Optional[float] = None,
                   cli: Optional[str] = None, runid: Optional[str] = None,
                   driver_version: Optional[str] = None) -> dict:
    g = cluster.gpu
    return {
        "schema": SCHEMA,
        "runid": runid,
        "host": {"hostname": socket.gethostname(), "platform": platform.platform(),
                 "python": sys.version.split()[0], "driver_version": driver_version or "unknown"},
        "code": {"git_commit": _git_commit(), "git_dirty": _git_dirty()},
        "model": {"name": cfg.name, "hash": model_hash(cfg), "total_params": cfg.total_params,
                  "active_params": cfg.active_params},
        "hardware": {"gpu": g.name, "n_gpus": cluster.n_gpus, "hbm_bw_per_gpu": g.hbm_bw,
                     "aggregate_hbm_bw": cluster.aggregate_hbm_bw, "peak_bw_measured": peak_bw_measured,
                     "bf16_flops": g.bf16_flops, "fp8_flops": g.fp8_flops},
        "bench": {"config": asdict(config), "config_id": config_id(config), "seed": config.seed,
                  "repeats": config.repeats, "warmup_steps": config.warmup_steps},
        "cli": cli,
    }
