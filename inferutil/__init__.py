"""inferutil — latency-oriented multi-GPU MoE inference utilities: an analytical roofline model of B=1 decode and
a benchmark harness with an ``Engine`` seam (``inferutil.bench``). Same import name and public surface as the
reference package so that its report/compare tooling and the engine adapter interoperate."""
from .hardware import GPUS, H100_SXM, H200_SXM, B200_SXM, Cluster, GPU, measured_b200
from .model import MoEConfig, QWEN3_235B, QWEN3_30B
from .latency import decode_latency, DecodeBreakdown, expected_max_experts_per_gpu
from .speculative import (SpecConfig, expected_accepted_single, expected_accepted_multi, sweep as spec_sweep,
                          memory_feasibility)
from .routing import (CoActGraph, ingest_telemetry, greedy_partition, round_robin_placement, placement_stats,
                      TokenDAG)

__all__ = ["GPUS", "H100_SXM", "H200_SXM", "B200_SXM", "Cluster", "GPU", "measured_b200", "MoEConfig", "QWEN3_235B",
           "QWEN3_30B", "decode_latency", "DecodeBreakdown", "expected_max_experts_per_gpu", "SpecConfig",
           "expected_accepted_single", "expected_accepted_multi", "spec_sweep", "memory_feasibility", "CoActGraph",
           "ingest_telemetry", "greedy_partition", "round_robin_placement", "placement_stats", "TokenDAG"]
