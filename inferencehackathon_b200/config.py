"""Configuration tree: model shapes, parallel layout, quantisation, engine, speculative decoding, server.

The reference fixes its model shapes at compile time (kernels/common.cuh:12-26) and spreads its knobs over
``#define``s, positional argv and ``getenv`` (kernels/decode_step_tp8.cu:90-124, kernels/k1_attn_prologue.cu:739-797).
Here every shape is a runtime value carried by one frozen dataclass tree; environment variables only override
tuning knobs (see :func:`env_flag`).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field, replace
from typing import Optional


@dataclass(frozen=True)
class ModelConfig:
    """Qwen3-MoE decoder shape. Defaults are Qwen3-235B-A22B (src/inferutil/model.py:25-60)."""

    name: str = "qwen3-235b-a22b"
    hidden: int = 4096
    n_layers: int = 94
    n_q_heads: int = 64
    n_kv_heads: int = 4
    head_dim: int = 128
    n_experts: int = 128
    top_k: int = 8
    moe_inter: int = 1536
    vocab: int = 151936
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    norm_topk_prob: bool = True
    tie_embeddings: bool = False

    @property
    def q_dim(self) -> int:
        return self.n_q_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def q_per_kv(self) -> int:
        return self.n_q_heads // self.n_kv_heads

    def truncated(self, n_layers: int) -> "ModelConfig":
        """Same architecture with fewer layers (for a model that does not fit on the GPUs at hand)."""
        return replace(self, n_layers=n_layers, name=f"{self.name}-L{n_layers}")

    # parameter accounting -------------------------------------------------------------------------------
    def attn_params_per_layer(self) -> int:
        h, qd, kvd = self.hidden, self.q_dim, self.kv_dim
        return h * qd + 2 * h * kvd + qd * h + 2 * self.head_dim

    def expert_params(self) -> int:
        return 3 * self.hidden * self.moe_inter

    def layer_params(self) -> int:
        return (self.attn_params_per_layer() + self.n_experts * self.expert_params()
                + self.n_experts * self.hidden + 2 * self.hidden)

    def total_params(self) -> int:
        emb = self.vocab * self.hidden
        head = 0 if self.tie_embeddings else self.vocab * self.hidden
        return self.n_layers * self.layer_params() + emb + head + self.hidden

    def active_params(self) -> int:
        per_layer = (self.attn_params_per_layer() + self.top_k * self.expert_params()
                     + self.n_experts * self.hidden + 2 * self.hidden)
        return self.n_layers * per_layer + self.vocab * self.hidden + self.hidden


TINY = ModelConfig(name="tiny-qwen3-moe", hidden=256, n_layers=4, n_q_heads=8, n_kv_heads=2, head_dim=32,
                   n_experts=16, top_k=4, moe_inter=128, vocab=2048)
QWEN3_30B_A3B = ModelConfig(name="qwen3-30b-a3b", hidden=2048, n_layers=48, n_q_heads=32, n_kv_heads=4,
                            head_dim=128, n_experts=128, top_k=8, moe_inter=768, vocab=151936)
QWEN3_235B_A22B = ModelConfig()
# head_dim-128 miniature for GPU kernel tests
SMALL = ModelConfig(name="small-qwen3-moe", hidden=512, n_layers=2, n_q_heads=8, n_kv_heads=2, head_dim=128,
                    n_experts=16, top_k=4, moe_inter=256, vocab=4096)

MODEL_PRESETS = {
    "tiny": TINY,
    "small": SMALL,
    SMALL.name: SMALL,
    TINY.name: TINY,
    "qwen3-30b-a3b": QWEN3_30B_A3B,
    "qwen3-235b-a22b": QWEN3_235B_A22B,
}


def get_model_config(name: str, n_layers: Optional[int] = None) -> ModelConfig:
    cfg = MODEL_PRESETS[name.lower()]
    if n_layers is not None and n_layers != cfg.n_layers:
        cfg = cfg.truncated(n_layers)
    return cfg


@dataclass(frozen=True)
class ParallelConfig:
    """Tensor/expert-parallel layout over ``world = tp`` or ``world = ep`` ranks (hybrid: ``ep == world``,
    attention TP over groups of ``tp`` consecutive ranks). Data and pipeline parallelism do not exist for a
    single B=1 stream, as in the reference (only TP8 and EP8 are implemented there,
    kernels/decode_step_tp8.cu:18-41, kernels/ep_moe_sharded.cu:85-90; hybrid is analytical,
    src/inferutil/latency.py:130-145)."""

    tp: int = 1
    ep: int = 1
    rank: int = 0
    world: int = 1
    # Ranks that share one KV head (tp above the number of KV heads) and split its cache rows between them: rank i of
    # such a group keeps the rows r with r % kv_share == i and the group merges its partial attention results. 1: every
    # rank keeps all rows of its KV head (the layout of the reference, kernels/decode_step_tp8.cu:153-160, and of the CUDA
    # pipelines here). PyTorch path only.
    kv_share: int = 1

    @property
    def plan(self) -> str:
        if self.ep > 1 and self.tp > 1:
            return "hybrid"
        if self.ep > 1:
            return "ep"
        return "tp"

    @property
    def tp_rank(self) -> int:
        return self.rank % self.tp

    @property
    def tp_group_index(self) -> int:
        return self.rank // self.tp

    @property
    def ep_rank(self) -> int:
        return self.rank % self.ep if self.ep > 1 else 0

    def validate(self, cfg: ModelConfig) -> None:
        if self.ep > 1:
            if self.world != self.ep:
                raise ValueError("with expert parallelism the world size equals ep")
            if self.ep % self.tp:
                raise ValueError("hybrid layout needs tp to divide ep")
            if cfg.n_experts % self.ep:
                raise ValueError("ep must divide the number of experts")
        elif self.world != self.tp:
            raise ValueError("pure tensor parallelism needs world == tp")
        if cfg.n_q_heads % self.tp:
            raise ValueError("tp must divide the number of query heads")
        if self.ep == 1 and cfg.moe_inter % self.tp:
            raise ValueError("tp must divide the expert intermediate size")
        if self.tp > cfg.n_kv_heads and self.tp % cfg.n_kv_heads:
            raise ValueError("tp above n_kv_heads must be a multiple of it (KV heads replicate)")
        if self.kv_share > 1 and (self.tp <= cfg.n_kv_heads or self.kv_share != self.tp // cfg.n_kv_heads):
            raise ValueError("kv_share must equal tp / n_kv_heads (the ranks that hold the same KV head)")


@dataclass(frozen=True)
class QuantConfig:
    """Weight storage. ``fp8_block`` = e4m3 with one fp32 scale per (block_rows x block_cols) weight block
    (128x128 on the unsharded matrix) and per-token activation scales where activations are quantised (the
    tcgen05 GEMMs); the M=1 GEMV keeps activations in fp16, which is at least as precise. The reference
    quantises per output row with a per-tensor activation amax (kernels/common.cuh:32-36,
    kernels/gemm_engine.cuh:144-173)."""

    weights: str = "bf16"          # "fp32" | "bf16" | "fp8_block"
    block: int = 128
    kv: str = "bf16"               # "fp32" | "bf16" | "fp8" (e4m3 rows with a scale per position; on GPUs: the per-kernel pipeline)

    @property
    def weight_bytes(self) -> float:
        return {"fp32": 4, "bf16": 2, "fp8_block": 1}[self.weights]


@dataclass(frozen=True)
class SpecConfig:
    """Speculative decoding (engine/src/spec/engine.rs:10-20, engine/src/spec/eagle3_engine.rs:38-52)."""

    mode: str = "off"              # "off" | "ngram" | "eagle3"
    draft_len: int = 8
    ngram_n: int = 2
    tree_depth: int = 4
    tree_width: int = 4
    max_nodes: int = 16
    draft_vocab: int = 0           # 0 = target vocabulary
    floor_fraction: float = 0.86
    aux_layers: tuple = ()


@dataclass(frozen=True)
class EngineConfig:
    model: ModelConfig = field(default_factory=ModelConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    quant: QuantConfig = field(default_factory=QuantConfig)
    spec: SpecConfig = field(default_factory=SpecConfig)
    max_seq: int = 2048
    seed: int = 0
    backend: str = "auto"          # "torch" (reference ops) | "cuda" (sm_100a kernels) | "auto"
    use_graph: bool = True
    comm: str = "auto"             # "nccl" | "fused" | "auto"
    distinct_layers: int = 0       # >0: only this many distinct layer weight sets are held; layers alias them


@dataclass(frozen=True)
class ServerConfig:
    """Environment contract of the reference server (server/backend.py:136-143, server/main.py:16-33)."""

    backend: str = "mock"          # BACKEND: mock | vllm | engine
    vllm_url: str = "http://localhost:8001"
    vllm_model: str = "qwen3-235b-a22b"
    stream_delay: float = 0.0
    engine_model: str = "tiny"

    @staticmethod
    def from_env() -> "ServerConfig":
        return ServerConfig(
            backend=os.environ.get("BACKEND", "mock").lower(),
            vllm_url=os.environ.get("VLLM_URL", "http://localhost:8001"),
            vllm_model=os.environ.get("VLLM_MODEL", "qwen3-235b-a22b"),
            stream_delay=float(os.environ.get("STREAM_DELAY", "0") or 0),
            engine_model=os.environ.get("ENGINE_MODEL", "tiny"),
        )


def env_flag(name: str, default: int) -> int:
    """Integer tuning knob from the environment (the reference reads K1_PIPE, K2_SPLITS, ... the same way)."""
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    return int(v)
