"""Blackwell-native single-stream (B=1) MoE inference engine.

PyTorch framework layer (model, weights, KV cache, sampler, speculative driver, server) on top of hand-written
sm_100a CUDA kernels that fuse the decode GEMVs with their NVLink collectives.
"""
from .config import (EngineConfig, ModelConfig, ParallelConfig, QuantConfig, SpecConfig, ServerConfig,
                     MODEL_PRESETS, TINY, SMALL, QWEN3_30B_A3B, QWEN3_235B_A22B, get_model_config)

__version__ = "0.1.0"

__all__ = ["EngineConfig", "ModelConfig", "ParallelConfig", "QuantConfig", "SpecConfig", "ServerConfig",
           "MODEL_PRESETS", "TINY", "SMALL", "QWEN3_30B_A3B", "QWEN3_235B_A22B", "get_model_config", "__version__"]
