"""Token samplers. The reference engine only has greedy argmax (kernels/decode_step_tp8.cu:321-364); the server
contract carries ``temperature`` (server/schemas.py:12-19), so temperature / top-k / top-p sampling is provided
on top of the same logits."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: Optional[int] = None

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0


class Sampler:
    def __init__(self, params: Optional[SamplingParams] = None):
        self.params = params or SamplingParams()
        self._gen: Optional[torch.Generator] = None

    def _generator(self, device) -> Optional[torch.Generator]:
        if self.params.seed is None:
            return None
        if self._gen is None or self._gen.device != torch.device(device):
            self._gen = torch.Generator(device=device).manual_seed(self.params.seed)
        return self._gen

    def probs(self, logits: torch.Tensor) -> torch.Tensor:
        """Sampling distribution for ``logits[..., V]`` after temperature, top-k and top-p filtering."""
        p = self.params
        if p.greedy:
            out = torch.zeros_like(logits, dtype=torch.float32)
            out.scatter_(-1, logits.argmax(dim=-1, keepdim=True), 1.0)
            return out
        z = logits.float() / p.temperature
        if p.top_k and p.top_k < z.shape[-1]:
            kth = torch.topk(z, p.top_k, dim=-1).values[..., -1:]
            z = z.masked_fill(z < kth, float("-inf"))
        probs = torch.softmax(z, dim=-1)
        if p.top_p < 1.0:
            sp, si = torch.sort(probs, dim=-1, descending=True)
            keep = (sp.cumsum(dim=-1) - sp) < p.top_p
            sp = sp * keep
            probs = torch.zeros_like(probs).scatter_(-1, si, sp)
            probs = probs / probs.sum(dim=-1, keepdim=True)
        return probs

    def sample(self, logits: torch.Tensor) -> torch.Tensor:
        if self.params.greedy:
            return logits.argmax(dim=-1)
        probs = self.probs(logits)
        flat = probs.reshape(-1, probs.shape[-1])
        tok = torch.multinomial(flat, 1, generator=self._generator(flat.device)).reshape(probs.shape[:-1])
        return tok
