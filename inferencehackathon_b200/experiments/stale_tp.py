"""Stale tensor parallelism, quality probe: how much staleness of the per-layer all-reduce does greedy decoding
tolerate? On most layers the real reduced activation is replaced by a cached one, so that a real implementation
could overlap (or skip) the collective; this probe only measures the quality cost.

Reference: experiments/stale_tp/stale_tp.py (StaleScheduler :98-260, modes and policies :24-52). The decision logic
is pure Python; ``StaleCollectives`` applies it to this engine's collectives object instead of a vLLM monkey patch.

Per forward pass there are ``period`` tensor-parallel all-reduces (2 per layer: slot 0 after o_proj, slot 1 after the
experts). mode "layer": layers with ``layer % K == 0`` do the real all-reduce and cache it per slot, the others
reuse the latest cached value of their slot (staleness across depth, within a token). mode "temporal": every K-th
decode step is exact and caches per call index, the steps between reuse the previous values (staleness across
tokens). policy "proxy" substitutes the cached reduced value, policy "local" the un-reduced local partial (a lower
bound). ``K = 1`` or ``enable = False`` is exact. ``decode_only`` keeps multi-token passes (prefill) exact.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

REAL, REAL_FALLBACK, STALE, LOCAL, EXACT = "real", "real_fallback", "stale", "local", "exact"


@dataclass
class StaleConfig:
    enable: bool = True
    K: int = 2
    mode: str = "layer"                 # "layer" | "temporal"
    policy: str = "proxy"               # "proxy" | "local"
    decode_only: bool = True
    period: int = 188
    collectives_per_layer: int = 2


class StaleScheduler:
    """Per all-reduce call: do the real collective or substitute. Deterministic, no tensor introspection: cached
    values are opaque handles."""

    def __init__(self, cfg: StaleConfig):
        self.cfg = cfg
        self.K = max(1, cfg.K)
        self.period = max(1, cfg.period)
        self.cpl = max(1, cfg.collectives_per_layer)
        self._call = 0
        self._step = 0
        self._by_slot: Dict[int, object] = {}
        self._by_idx: Dict[int, object] = {}
        self.stats = {k: 0 for k in (REAL, REAL_FALLBACK, STALE, LOCAL, EXACT)}

    def reconfigure(self, **kw) -> None:
        """Change K / mode / policy / enable between sweep points; the caches start clean."""
        for k, v in kw.items():
            setattr(self.cfg, k, v)
        self.K = max(1, self.cfg.K)
        self._by_slot.clear()
        self._by_idx.clear()
        self._call = 0

    def _advance(self) -> None:
        self._call += 1
        if self._call >= self.period:
            self._call = 0
            if self.cfg.mode == "layer":
                self._by_slot.clear()
            self._step += 1

    def decide(self, token_count: int):
        """-> (action, call index, cached handle or None). The caller reports the value of a real all-reduce with
        ``record``; both advance nothing else."""
        cfg = self.cfg
        idx = self._call
        if not cfg.enable or self.K == 1 or (cfg.decode_only and token_count != 1):
            return EXACT, idx, None
        layer, slot = idx // self.cpl, idx % self.cpl
        if cfg.mode == "layer":
            refresh, cached = layer % self.K == 0, self._by_slot.get(slot)
        else:
            refresh, cached = self._step % self.K == 0, self._by_idx.get(idx)
        if refresh:
            return REAL, idx, None
        if cfg.policy == "local":
            return LOCAL, idx, None
        if cached is None:
            return REAL_FALLBACK, idx, None
        return STALE, idx, cached

    def record(self, action: str, idx: int, value=None) -> None:
        """Account for the call; ``value`` is the result of a real all-reduce (cached for later substitution)."""
        self.stats[action] += 1
        if action in (REAL, REAL_FALLBACK) and value is not None:
            if self.cfg.mode == "layer":
                self._by_slot[idx % self.cpl] = value
            else:
                self._by_idx[idx] = value
        if action == EXACT and self.cfg.decode_only is False:
            pass
        self._advance()

    def end_of_multi_token_pass(self) -> None:
        """A multi-token pass is exact and must not shift the call index of the decode steps that follow."""
        self._call = 0

    @property
    def stale_fraction(self) -> float:
        n = sum(self.stats.values())
        return (self.stats[STALE] + self.stats[LOCAL]) / n if n else 0.0


class StaleCollectives:
    """Wraps a collectives object: ``all_reduce_tp`` goes through the scheduler, everything else passes through."""

    def __init__(self, inner, scheduler: StaleScheduler):
        self._inner = inner
        self.scheduler = scheduler

    def __getattr__(self, name):
        return getattr(self._inner, name)

    def all_reduce_tp(self, x):
        sch = self.scheduler
        action, idx, cached = sch.decide(int(x.shape[0]))
        if action == STALE and getattr(cached, "shape", None) == x.shape:
            sch.record(STALE, idx)
            return cached.clone()
        if action == LOCAL:
            sch.record(LOCAL, idx)
            return x
        if action == STALE:
            action = REAL_FALLBACK
        y = self._inner.all_reduce_tp(x)
        sch.record(action, idx, y.detach().clone() if action != EXACT else None)
        return y


def install(model, cfg: Optional[StaleConfig] = None) -> StaleScheduler:
    """Routes ``model``'s tensor-parallel all-reduces through a scheduler (period = 2 x layers)."""
    cfg = cfg or StaleConfig()
    cfg.period = 2 * model.cfg.n_layers
    sch = StaleScheduler(cfg)
    model.comm = StaleCollectives(model.comm, sch)
    return sch


def uninstall(model) -> None:
    if isinstance(model.comm, StaleCollectives):
        model.comm = model.comm._inner


def probe(engine, prompts: Sequence[Sequence[int]], new_tokens: int = 32, Ks=(1, 2, 4, 8), modes=("layer", "temporal"),
          policy: str = "proxy") -> List[dict]:
    """Greedy agreement with the exact run per (mode, K): exact-match rate and mean common-prefix share. ``engine``
    is an ``InferenceEngine`` on the PyTorch backend."""
    from .quality import compare_ids
    model = engine.model
    exact = [engine.generate(list(p), new_tokens).tokens for p in prompts]
    sch = install(model, StaleConfig(enable=False))
    rows = []
    try:
        for mode in modes:
            for K in Ks:
                sch.reconfigure(enable=True, K=K, mode=mode, policy=policy)
                sch.stats = {k: 0 for k in sch.stats}
                outs = []
                for p in prompts:
                    sch.reconfigure()
                    sch._step = 0
                    outs.append(engine.generate(list(p), new_tokens).tokens)
                c = compare_ids(exact, outs)
                rows.append({"mode": mode, "K": K, "policy": policy, "stale_fraction": sch.stale_fraction, **c})
    finally:
        uninstall(model)
    return rows
