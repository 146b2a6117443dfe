"""MoE architecture description with parameter and KV-cache accounting (reference: src/inferutil/model.py:25-110).

The default instance is Qwen3-235B-A22B; ``QWEN3_30B`` is Qwen3-30B-A3B.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class MoEConfig:
    name: str = "Qwen3-235B-A22B"
    hidden: int = 4096
    n_layers: int = 94
    n_heads: int = 64
    n_kv_heads: int = 4
    head_dim: int = 128
    n_experts: int = 128
    top_k: int = 8
    moe_inter: int = 1536
    n_shared_experts: int = 0
    vocab: int = 151936
    tie_embeddings: bool = False

    # dimensions
    @property
    def q_dim(self) -> int:
        return self.head_dim * self.n_heads

    @property
    def kv_dim(self) -> int:
        return self.head_dim * self.n_kv_heads

    # parameters per component
    @property
    def attn_params(self) -> int:
        return 2 * self.hidden * self.q_dim + 2 * self.hidden * self.kv_dim

    @property
    def one_expert_params(self) -> int:
        return 3 * self.moe_inter * self.hidden

    @property
    def router_params(self) -> int:
        return self.n_experts * self.hidden

    @property
    def moe_params_per_layer(self) -> int:
        return self.router_params + (self.n_experts + self.n_shared_experts) * self.one_expert_params

    @property
    def layer_params(self) -> int:
        return self.moe_params_per_layer + self.attn_params

    @property
    def embed_params(self) -> int:
        return self.vocab * self.hidden * (1 if self.tie_embeddings else 2)

    @property
    def total_params(self) -> int:
        return self.embed_params + self.n_layers * self.layer_params

    # what one decoded token touches
    @property
    def active_attn_params(self) -> int:
        return self.attn_params

    @property
    def active_moe_params_per_layer(self) -> int:
        return self.router_params + (self.top_k + self.n_shared_experts) * self.one_expert_params

    @property
    def active_layer_params(self) -> int:
        return self.active_attn_params + self.active_moe_params_per_layer

    @property
    def active_params(self) -> int:
        return self.vocab * self.hidden + self.n_layers * self.active_layer_params

    def kv_bytes_per_token(self, dtype_bytes: int = 2) -> int:
        return 2 * dtype_bytes * self.kv_dim * self.n_layers


QWEN3_235B = MoEConfig()
QWEN3_30B = MoEConfig(name="Qwen3-30B-A3B", hidden=2048, n_layers=48, n_heads=32, n_kv_heads=4, head_dim=128,
                      n_experts=128, top_k=8, moe_inter=768)
