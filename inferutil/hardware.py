"""Accelerator and node descriptions for the roofline model (SI units: bytes, bytes/s, FLOP/s).

Same public names as the reference's ``inferutil.hardware`` (src/inferutil/hardware.py:17-66) with the B200 added,
both at its nominal figures and at the figures measured on the benchmark pool.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, replace

GB = 10 ** 9
TB = 10 ** 12
TFLOP = 10 ** 12


@dataclass(frozen=True)
class GPU:
    name: str
    hbm_bytes: int
    hbm_bw: float
    bf16_flops: float
    fp8_flops: float
    nvlink_bw: float                    # one direction, per GPU
    collective_latency_s: float = 5e-6  # fixed cost of one small collective


def _gpu(name, hbm_gb, bw_tb, bf16_tf, fp8_tf, nvlink_gb, lat=5e-6) -> GPU:
    return GPU(name, int(hbm_gb * GB), bw_tb * TB, bf16_tf * TFLOP, fp8_tf * TFLOP, nvlink_gb * GB, lat)


H100_SXM = _gpu("H100-SXM-80GB", 80, 3.35, 989.4, 1978.9, 450)
H200_SXM = _gpu("H200-SXM-141GB", 141, 4.8, 989.4, 1978.9, 450)
B200_SXM = _gpu("B200-SXM-180GB", 180, 7.7, 2250.0, 4500.0, 900, 3e-6)


def measured_b200(path: str | None = None) -> GPU:
    """B200 with the copy bandwidth and bf16 matmul rate measured on this machine pool (file written by the
    benchmark driver); falls back to the nominal part when the file is absent."""
    path = path or os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            m = json.load(f)
        bf16 = float(m["bf16_tflops"]) * TFLOP
        # collective: what one in-kernel all-reduce adds to a layer at 8 GPUs (tagged-slot scheme, measured 6.5 us:
        # 13 us per layer for two all-reduces beyond the same phases on one GPU)
        return replace(B200_SXM, name="B200-SXM-180GB-measured", hbm_bw=float(m["hbm_gbs"]) * GB,
                       bf16_flops=bf16, fp8_flops=2 * bf16, collective_latency_s=6.5e-6)
    except (OSError, KeyError, ValueError):
        return B200_SXM


@dataclass(frozen=True)
class Cluster:
    gpu: GPU
    n_gpus: int = 8

    @property
    def total_hbm(self) -> int:
        return self.n_gpus * self.gpu.hbm_bytes

    @property
    def aggregate_hbm_bw(self) -> float:
        return self.n_gpus * self.gpu.hbm_bw


GPUS = {g.name: g for g in (H100_SXM, H200_SXM, B200_SXM)}
