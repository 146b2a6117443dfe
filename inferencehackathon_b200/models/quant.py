"""Block-scaled fp8 (e4m3) weight quantisation and per-token activation quantisation.

A weight matrix ``W[rows, K]`` is stored as e4m3 bytes plus one fp32 scale per ``rb x kb`` block:
``W ~= q * scale[row // rb, k // kb]``. The unsharded layout uses 128 x 128 blocks; a tensor-parallel shard
whose boundaries cut through a block (192-row expert shards at TP8) keeps the same values by shrinking the block
to the largest size that divides the shard offset (64), see :func:`reblock_scales`.

The reference uses one scale per output row instead (tools/conifer_weight_convert.py:40-47) and a per-tensor
activation scale (kernels/gemm_engine.cuh:144-173).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

E4M3_MAX = 448.0


@dataclass
class QWeight:
    """A (possibly quantised) weight with leading batch dims: ``data[..., rows, K]``.

    ``scale`` is ``None`` for fp32/bf16 storage, else ``[..., ceil(rows/rb), ceil(K/kb)]`` fp32 and ``data`` is
    ``torch.float8_e4m3fn``.
    """

    data: torch.Tensor
    scale: Optional[torch.Tensor] = None
    rb: int = 128
    kb: int = 128

    @property
    def is_fp8(self) -> bool:
        return self.scale is not None

    @property
    def shape(self):
        return self.data.shape

    def to(self, device) -> "QWeight":
        return QWeight(self.data.to(device), None if self.scale is None else self.scale.to(device),
                       self.rb, self.kb)

    def dequant(self, dtype=torch.float32) -> torch.Tensor:
        if self.scale is None:
            return self.data.to(dtype)
        return dequant_block(self.data, self.scale, self.rb, self.kb).to(dtype)

    def select(self, idx) -> "QWeight":
        """Index the leading (expert) dimension."""
        return QWeight(self.data[idx], None if self.scale is None else self.scale[idx], self.rb, self.kb)

    def nbytes(self) -> int:
        n = self.data.numel() * self.data.element_size()
        if self.scale is not None:
            n += self.scale.numel() * 4
        return n


def quant_block(w: torch.Tensor, rb: int = 128, kb: int = 128) -> QWeight:
    """Quantise ``w[..., rows, K]`` to e4m3 with one scale per ``rb x kb`` block (amax / 448)."""
    *lead, rows, K = w.shape
    nrb, nkb = math.ceil(rows / rb), math.ceil(K / kb)
    wf = w.float()
    pad_r, pad_k = nrb * rb - rows, nkb * kb - K
    if pad_r or pad_k:
        wf = torch.nn.functional.pad(wf, (0, pad_k, 0, pad_r))
    blocks = wf.reshape(*lead, nrb, rb, nkb, kb)
    amax = blocks.abs().amax(dim=(-3, -1)).clamp_min(1e-12)            # [..., nrb, nkb]
    scale = (amax / E4M3_MAX).float()
    q = (blocks / scale[..., :, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX)
    q = q.reshape(*lead, nrb * rb, nkb * kb)[..., :rows, :K].contiguous().to(torch.float8_e4m3fn)
    return QWeight(q, scale.contiguous(), rb, kb)


def dequant_block(q: torch.Tensor, scale: torch.Tensor, rb: int, kb: int) -> torch.Tensor:
    *lead, rows, K = q.shape
    s = scale.repeat_interleave(rb, dim=-2)[..., :rows, :].repeat_interleave(kb, dim=-1)[..., :K]
    return q.float() * s


def reblock_scales(scale: torch.Tensor, rb: int, kb: int, row0: int, rows: int, k0: int, K: int):
    """Scales of the sub-matrix ``[row0:row0+rows, k0:k0+K]`` of a block-quantised weight.

    Returns ``(scale_sub, rb_sub, kb_sub)`` where the new block sizes are the largest divisors of the old ones
    that also divide the shard offsets and extents, so every new block lies inside exactly one old block.
    """
    rb2 = math.gcd(math.gcd(rb, row0), rows) if (row0 % rb or rows % rb) else rb
    kb2 = math.gcd(math.gcd(kb, k0), K) if (k0 % kb or K % kb) else kb
    r_idx = (row0 + torch.arange(0, rows, rb2, device=scale.device)) // rb
    k_idx = (k0 + torch.arange(0, K, kb2, device=scale.device)) // kb
    sub = scale.index_select(-2, r_idx).index_select(-1, k_idx).contiguous()
    return sub, rb2, kb2


def quant_act_per_token(x: torch.Tensor, group: int = 128):
    """Per-token, per-``group``-channel e4m3 activation quantisation: returns ``(q[T, K] e4m3, s[T, K/group])``."""
    T, K = x.shape
    g = x.float().reshape(T, K // group, group)
    amax = g.abs().amax(dim=-1).clamp_min(1e-12)
    s = amax / E4M3_MAX
    q = (g / s[..., None]).clamp(-E4M3_MAX, E4M3_MAX).reshape(T, K).to(torch.float8_e4m3fn)
    return q, s.contiguous()


def store_weight(w: torch.Tensor, mode: str, rb: int = 128, kb: int = 128) -> QWeight:
    """Store ``w`` as ``mode`` in {"fp32", "bf16", "fp8_block"}."""
    if mode == "fp32":
        return QWeight(w.float().contiguous())
    if mode == "bf16":
        return QWeight(w.to(torch.bfloat16).contiguous())
    if mode == "fp8_block":
        return quant_block(w, rb, kb)
    raise ValueError(f"unknown weight storage {mode!r}")
