"""Live routing pipeline: real ``layer -> experts`` records in, predictions, prefetch actions and hit rates out.

The native control plane (``csrc/ctrl/routing.cpp``: Markov / proxy predictors, prefetch scheduler over a placement map,
accuracy tracker) is driven here by the routing a model actually produced, one layer record at a time: the engine's own
device router (``EngineBackend``), or a vLLM's gate modules through the routing feed (``serve/vllm_tools.py``). For
every record of layer L the pipeline
  1. scores the prediction that was made for L when L - 1 completed (scheduler hit rate, per-layer accuracy),
  2. lets the Markov predictor observe the transition (experts of L - 1) -> (experts of L),
  3. predicts the experts of L + 1 from those of L and hands the prediction to the prefetch scheduler, which turns it
     into WarmExpert / EarlyDispatch actions for the GPUs that hold those experts (``sink``).
The reference defines the same parts (engine/src/routing/{predictor,scheduler,stats}.rs) and a prefetch-sink trait,
but nothing feeds them real routing (its server simulates routing unless the vLLM hook is attached, and the sink is never
connected to the engine).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

from .native import (MARKOV, AccuracyTracker, ExpertPrediction, PlacementMap, PrefetchAction, PrefetchScheduler,
                     RoutePredictor)


class RoutingPipeline:
    def __init__(self, n_layers: int, n_experts: int, top_k: int = 8, n_gpus: int = 8,
                 placement: Optional[PlacementMap] = None, sink: Optional[Callable[[PrefetchAction], None]] = None,
                 warmup_tokens: int = 4):
        self.n_layers, self.n_experts, self.top_k = n_layers, n_experts, top_k
        self.placement = placement or PlacementMap.round_robin(n_layers, n_gpus, n_experts)
        # the Markov predictor needs no hidden states: it works from any source of routing records
        self.predictor = RoutePredictor(n_layers, 1, n_experts)
        self.predictor.enable_markov()
        self.scheduler = PrefetchScheduler(self.placement, sink=sink, record=sink is None)
        self.accuracy = AccuracyTracker(n_layers, top_k)
        self.warmup_tokens = warmup_tokens             # tokens observed before predictions are issued
        self.tokens = 0
        self.records = 0
        self._prev_layer = -1
        self._prev_experts: List[int] = []
        self._pending: Optional[ExpertPrediction] = None

    def on_layer(self, layer: int, experts: Sequence[int]) -> Optional[ExpertPrediction]:
        """One routing record; returns the prediction issued for ``layer + 1`` (None during warm-up / at the last layer)."""
        experts = [int(e) for e in experts]
        self.records += 1
        if layer == 0:
            self.tokens += 1
        if self._pending is not None and self._pending.layer == layer:
            self.scheduler.on_layer_complete(layer, experts)
            self.accuracy.record(self._pending, layer, experts)
        self._pending = None
        if self._prev_layer == layer - 1 and self._prev_experts:
            self.predictor.markov_observe(layer - 1, self._prev_experts, experts)
        self._prev_layer, self._prev_experts = layer, experts
        if layer + 1 >= self.n_layers or self.tokens <= self.warmup_tokens:
            return None
        pred = self.predictor.predict(layer, current_experts=experts, top_k=self.top_k, kind=MARKOV)
        if pred.experts:
            self.scheduler.on_prediction(pred)
            self._pending = pred
            return pred
        return None

    def on_token(self, layers: Dict[int, Sequence[int]]) -> None:
        """All records of one token, in layer order (the shape the routing feed reader and the engine deliver)."""
        for layer in sorted(layers):
            self.on_layer(layer, layers[layer])

    def stats(self) -> Dict:
        return {"tokens": self.tokens, "records": self.records,
                "prefetch_hit_rate": round(self.scheduler.hit_rate(), 4),
                "prefetched": self.scheduler.total_prefetched(), "hits": self.scheduler.total_hits(),
                "mean_layer_hit_rate": round(self.accuracy.mean_hit_rate(), 4),
                "expected_hits_per_layer": round(self.accuracy.mean_hit_rate() * self.top_k, 3)}
