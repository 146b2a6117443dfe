"""ctypes bindings of the expert-routing control plane (``libihb_ctrl.so``, ``csrc/ctrl/routing.cpp``).

Placement optimiser, next-layer route predictors, prefetch scheduler, accuracy tracker and trace collector.
Reference counterparts: engine/src/routing/{optimizer,predictor,scheduler,stats,types}.rs.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..spec.native import lib as _base_lib

_f = C.POINTER(C.c_float)
_i = C.POINTER(C.c_int)
_u = C.POINTER(C.c_uint)
_d = C.POINTER(C.c_double)
SINK_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int)
PREFETCH_WARM, PREFETCH_DISPATCH = 0, 1
PROXY, LINEAR, MARKOV, ENSEMBLE = 0, 1, 2, 3
KIND_NAMES = {PROXY: "DirectProxy", LINEAR: "LearnedLinear", MARKOV: "MarkovTransition", ENSEMBLE: "Ensemble"}

_declared = False


def lib() -> C.CDLL:
    global _declared
    L = _base_lib()
    if not _declared:
        vp = C.c_void_p
        L.ihb_placement_optimize.restype = None
        L.ihb_placement_optimize.argtypes = [_u, C.c_int, C.c_int, C.c_int, C.c_double, _i, _i, _d]
        L.ihb_pred_create.restype = vp
        L.ihb_pred_create.argtypes = [C.c_int, C.c_int, C.c_int]
        L.ihb_pred_destroy.argtypes = [vp]
        L.ihb_pred_set_router.argtypes = [vp, C.c_int, _f]
        L.ihb_pred_linear_from_proxy.argtypes = [vp]
        L.ihb_pred_linear_update.argtypes = [vp, C.c_int, _f, _f, C.c_int, C.c_float]
        L.ihb_pred_markov_enable.argtypes = [vp]
        L.ihb_pred_markov_observe.argtypes = [vp, C.c_int, _i, C.c_int, _i, C.c_int]
        L.ihb_pred_predict.restype = C.c_int
        L.ihb_pred_predict.argtypes = [vp, C.c_int, C.c_int, _f, _i, C.c_int, C.c_int, _f, _i, _f]
        L.ihb_sched_create.restype = vp
        L.ihb_sched_create.argtypes = [C.c_int, C.c_int, C.c_int, _i, _i]
        L.ihb_sched_destroy.argtypes = [vp]
        L.ihb_sched_set_sink.argtypes = [vp, SINK_FN, vp, C.c_int]
        L.ihb_sched_gpus_for.restype = C.c_int
        L.ihb_sched_gpus_for.argtypes = [vp, C.c_int, C.c_int, _i]
        L.ihb_sched_on_prediction.restype = C.c_int
        L.ihb_sched_on_prediction.argtypes = [vp, C.c_int, _i, C.c_int]
        L.ihb_sched_on_layer_complete.argtypes = [vp, C.c_int, _i, C.c_int]
        L.ihb_sched_hit_rate.restype = C.c_float
        L.ihb_sched_hit_rate.argtypes = [vp]
        L.ihb_sched_total_hits.restype = C.c_ulonglong
        L.ihb_sched_total_hits.argtypes = [vp]
        L.ihb_sched_total_prefetched.restype = C.c_ulonglong
        L.ihb_sched_total_prefetched.argtypes = [vp]
        L.ihb_sched_drain.restype = C.c_int
        L.ihb_sched_drain.argtypes = [vp, _i, C.c_int]
        L.ihb_acc_create.restype = vp
        L.ihb_acc_create.argtypes = [C.c_int, C.c_int]
        L.ihb_acc_destroy.argtypes = [vp]
        L.ihb_acc_record.argtypes = [vp, C.c_int, _i, C.c_int, _i, C.c_int]
        L.ihb_acc_hit_rate.restype = C.c_float
        L.ihb_acc_hit_rate.argtypes = [vp, C.c_int]
        L.ihb_acc_tokens.restype = C.c_ulonglong
        L.ihb_acc_tokens.argtypes = [vp, C.c_int]
        L.ihb_acc_mean_hit_rate.restype = C.c_float
        L.ihb_acc_mean_hit_rate.argtypes = [vp]
        L.ihb_acc_reset.argtypes = [vp]
        L.ihb_trace_create.restype = vp
        L.ihb_trace_create.argtypes = [C.c_int, C.c_int, C.c_int]
        L.ihb_trace_destroy.argtypes = [vp]
        L.ihb_trace_push.restype = C.c_int
        L.ihb_trace_push.argtypes = [vp, C.c_int, _f, _f]
        L.ihb_trace_count.restype = C.c_int
        L.ihb_trace_count.argtypes = [vp, C.c_int]
        L.ihb_trace_drain_layer.restype = C.c_int
        L.ihb_trace_drain_layer.argtypes = [vp, C.c_int, _f, _f]
        L.ihb_trace_clear.argtypes = [vp]
        _declared = True
    return L


def _fa(x):
    return np.ascontiguousarray(x, dtype=np.float32)


def _ia(x):
    return np.ascontiguousarray(x, dtype=np.int32)


# ---- placement ------------------------------------------------------------------------------------------------------------
@dataclass
class PlacementMap:
    """``primary[layer, expert] = gpu``; ``replica[layer, expert] = gpu`` or -1.
    Reference: engine/src/routing/scheduler.rs:83-147."""
    primary: np.ndarray
    replica: np.ndarray
    n_gpus: int

    @property
    def n_layers(self) -> int:
        return self.primary.shape[0]

    @property
    def n_experts(self) -> int:
        return self.primary.shape[1]

    @classmethod
    def round_robin(cls, n_layers: int, n_gpus: int, n_experts: int) -> "PlacementMap":
        prim = np.tile(np.arange(n_experts, dtype=np.int32) % n_gpus, (n_layers, 1))
        return cls(prim, np.full((n_layers, n_experts), -1, np.int32), n_gpus)

    @classmethod
    def contiguous(cls, n_layers: int, n_gpus: int, n_experts: int) -> "PlacementMap":
        """Expert ``e`` on GPU ``e // (E / n_gpus)``: the layout of the expert-parallel engine."""
        per = max(1, n_experts // n_gpus)
        prim = np.tile(np.minimum(np.arange(n_experts, dtype=np.int32) // per, n_gpus - 1), (n_layers, 1))
        return cls(prim.astype(np.int32), np.full((n_layers, n_experts), -1, np.int32), n_gpus)

    def gpu_for(self, layer: int, expert: int) -> int:
        return int(self.primary[layer, expert % self.n_experts])

    def gpus_for(self, layer: int, expert: int) -> Tuple[int, Optional[int]]:
        r = int(self.replica[layer, expert % self.n_experts])
        return self.gpu_for(layer, expert), (r if r >= 0 else None)

    def is_replicated(self, layer: int, expert: int) -> bool:
        return self.replica[layer, expert % self.n_experts] >= 0

    def set(self, layer: int, expert: int, gpu: int) -> None:
        self.primary[layer, expert] = gpu

    def set_replica(self, layer: int, expert: int, gpu: int) -> None:
        self.replica[layer, expert] = gpu

    def n_replicated_experts(self) -> int:
        return int((self.replica >= 0).sum())

    def to_json(self) -> Dict:
        """``{placement: {layer: {expert: gpu}}, replicas: {layer: {expert: gpu}}}`` (string keys)."""
        placement = {str(l): {str(e): int(g) for e, g in enumerate(row)} for l, row in enumerate(self.primary)}
        replicas = {}
        for l, row in enumerate(self.replica):
            hot = {str(e): int(g) for e, g in enumerate(row) if g >= 0}
            if hot:
                replicas[str(l)] = hot
        return {"placement": placement, "replicas": replicas}

    @classmethod
    def from_json(cls, obj: Dict, n_gpus: Optional[int] = None) -> "PlacementMap":
        """Inverse of :meth:`to_json`. Layers or experts a document leaves out are placed round robin; anything that is
        not a table of non-negative integers raises ``ValueError`` (never an index or type error from the inside)."""
        try:
            pl = obj["placement"]
            rows = {int(l): {int(e): int(g) for e, g in row.items()} for l, row in pl.items()}
            reps = {int(l): {int(e): int(g) for e, g in row.items()} for l, row in (obj.get("replicas") or {}).items()}
        except (KeyError, TypeError, ValueError, AttributeError, OverflowError) as err:
            raise ValueError(f"not a placement document: {type(err).__name__}: {err}") from None
        ids = [l for l in rows] + [e for r in rows.values() for e in r] + [g for r in rows.values() for g in r.values()]
        ids += [l for l in reps] + [e for r in reps.values() for e in r] + [g for r in reps.values() for g in r.values()]
        if not rows or not any(rows.values()) or min(ids) < 0 or max(ids) > 1 << 20:
            raise ValueError("not a placement document: empty, or an id that is negative or absurdly large")
        n_layers = max(list(rows) + list(reps)) + 1
        n_experts = max(e for r in list(rows.values()) + list(reps.values()) for e in r) + 1
        stated = obj.get("stats", {}).get("n_gpus") if isinstance(obj.get("stats"), dict) else None
        ng = int(n_gpus or stated or max(g for r in rows.values() for g in r.values()) + 1)
        prim = (np.arange(n_experts, dtype=np.int32)[None, :] % ng).repeat(n_layers, 0)
        rep = np.full((n_layers, n_experts), -1, np.int32)
        for l, row in rows.items():
            for e, g in row.items():
                prim[l, e] = g
        for l, row in reps.items():
            for e, g in row.items():
                rep[l, e] = g
        return cls(prim, rep, ng)


def optimize_placement(activation_counts, n_gpus: int, hot_mult: float = 2.0) -> Tuple[PlacementMap, Dict]:
    """Per layer the best of three placements by peak GPU load: heaviest expert first onto the least-loaded GPU; the
    same with every expert firing more than ``hot_mult`` x the layer mean split into two halves placed on two GPUs
    (primary + replica, each taking half its traffic); round robin. A layer therefore never ends up above round robin,
    nor with a replica that raises its peak. Returns the map and the JSON document ``{placement, replicas, stats}``.
    Reference: engine/src/routing/optimizer.rs:61-232 (heaviest first, then a replica for every hot expert on the
    least-loaded other GPU, which on skewed counts can undo the balance)."""
    counts = np.ascontiguousarray(activation_counts, dtype=np.uint32)
    n_layers, n_experts = counts.shape
    prim = np.zeros((n_layers, n_experts), np.int32)
    rep = np.zeros((n_layers, n_experts), np.int32)
    stats = np.zeros(4, np.float64)
    lib().ihb_placement_optimize(counts.ctypes.data_as(_u), n_layers, n_experts, n_gpus, hot_mult,
                                 prim.ctypes.data_as(_i), rep.ctypes.data_as(_i), stats.ctypes.data_as(_d))
    pm = PlacementMap(prim, rep, n_gpus)
    doc = pm.to_json()
    doc["stats"] = {"n_layers": n_layers, "n_experts": n_experts, "n_gpus": n_gpus,
                    "round_robin_mean_imbalance": round(float(stats[0]), 3),
                    "optimized_mean_imbalance": round(float(stats[1]), 3),
                    "improvement_pct": round(float(stats[2]), 1),
                    "total_replicated_expert_layers": int(stats[3])}
    return pm, doc


# ---- predictors -----------------------------------------------------------------------------------------------------------
@dataclass
class ExpertPrediction:
    layer: int
    experts: List[int]
    scores: List[float]
    source: str


class RoutePredictor:
    """Predicts the experts of layer ``L + 1`` from the hidden state (and/or expert choice) of layer ``L``.

    ``kind``: PROXY applies the next layer's router matrix to the current hidden state (no training); LINEAR is a
    per-layer matrix initialised from the proxy and refined by SGD on traces; MARKOV uses expert co-occurrence
    counts only; ENSEMBLE mixes the L2-normalised scores with ``weights``.
    Reference: engine/src/routing/predictor.rs:21-449."""

    def __init__(self, n_layers: int, hidden: int, n_experts: int):
        self.n_layers, self.hidden, self.n_experts = n_layers, hidden, n_experts
        self._h = lib().ihb_pred_create(n_layers, hidden, n_experts)
        self.weights = [1.0, 0.0, 0.0]

    def __del__(self):
        if getattr(self, "_h", None):
            lib().ihb_pred_destroy(self._h)
            self._h = None

    def set_router(self, layer: int, w) -> None:
        a = _fa(w)
        assert a.size == self.n_experts * self.hidden
        lib().ihb_pred_set_router(self._h, layer, a.ctypes.data_as(_f))

    def init_linear_from_proxy(self) -> None:
        lib().ihb_pred_linear_from_proxy(self._h)

    def linear_update(self, layer: int, hidden_batch, target_scores, lr: float = 1e-3) -> None:
        hb, t = _fa(hidden_batch).reshape(-1, self.hidden), _fa(target_scores).reshape(-1, self.n_experts)
        lib().ihb_pred_linear_update(self._h, layer, hb.ctypes.data_as(_f), t.ctypes.data_as(_f), hb.shape[0], lr)

    def enable_markov(self) -> None:
        lib().ihb_pred_markov_enable(self._h)

    def markov_observe(self, layer: int, experts_l: Sequence[int], experts_l1: Sequence[int]) -> None:
        a, b = _ia(experts_l), _ia(experts_l1)
        lib().ihb_pred_markov_observe(self._h, layer, a.ctypes.data_as(_i), a.size, b.ctypes.data_as(_i), b.size)

    def predict(self, layer: int, hidden=None, current_experts: Optional[Sequence[int]] = None, top_k: int = 8,
                kind: int = PROXY) -> ExpertPrediction:
        ids = np.zeros(top_k, np.int32)
        sc = np.zeros(top_k, np.float32)
        h = _fa(hidden) if hidden is not None else None
        ce = _ia(current_experts) if current_experts is not None else None
        w = _fa(self.weights)
        n = lib().ihb_pred_predict(self._h, kind, layer, h.ctypes.data_as(_f) if h is not None else None,
                                   ce.ctypes.data_as(_i) if ce is not None else None, ce.size if ce is not None else 0,
                                   top_k, w.ctypes.data_as(_f), ids.ctypes.data_as(_i), sc.ctypes.data_as(_f))
        return ExpertPrediction(layer + 1, ids[:n].tolist(), sc[:n].tolist(), KIND_NAMES[kind])


# ---- scheduler ------------------------------------------------------------------------------------------------------------
@dataclass
class PrefetchAction:
    kind: str          # "WarmExpert" | "EarlyDispatch"
    layer: int
    expert_id: int
    gpu_id: int


class PrefetchScheduler:
    """Turns a prediction for layer ``L + 1`` into ``WarmExpert`` + ``EarlyDispatch`` actions for every GPU hosting
    a predicted expert and scores the predictions when the layer's real routing is known. ``sink(action)`` is
    called per action (``None``: actions are only recorded and can be drained).
    Reference: engine/src/routing/scheduler.rs:46-227."""

    def __init__(self, placement: PlacementMap, sink: Optional[Callable[[PrefetchAction], None]] = None,
                 record: bool = True):
        self.placement = placement
        p, r = _ia(placement.primary), _ia(placement.replica)
        self._h = lib().ihb_sched_create(placement.n_layers, placement.n_experts, placement.n_gpus,
                                         p.ctypes.data_as(_i), r.ctypes.data_as(_i))
        self._cb = None
        if sink is not None:
            def _cb(_ctx, kind, layer, expert, gpu):
                sink(PrefetchAction("WarmExpert" if kind == PREFETCH_WARM else "EarlyDispatch", layer, expert, gpu))
            self._cb = SINK_FN(_cb)
            lib().ihb_sched_set_sink(self._h, self._cb, None, int(record))
        elif not record:
            lib().ihb_sched_set_sink(self._h, SINK_FN(), None, 0)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().ihb_sched_destroy(self._h)
            self._h = None

    def on_prediction(self, prediction: ExpertPrediction) -> int:
        e = _ia(prediction.experts)
        return lib().ihb_sched_on_prediction(self._h, prediction.layer, e.ctypes.data_as(_i), e.size)

    def on_layer_complete(self, layer: int, actual_experts: Sequence[int]) -> None:
        a = _ia(actual_experts)
        lib().ihb_sched_on_layer_complete(self._h, layer, a.ctypes.data_as(_i), a.size)

    def hit_rate(self) -> float:
        return float(lib().ihb_sched_hit_rate(self._h))

    def total_hits(self) -> int:
        return int(lib().ihb_sched_total_hits(self._h))

    def total_prefetched(self) -> int:
        return int(lib().ihb_sched_total_prefetched(self._h))

    def drain(self, cap: int = 4096) -> List[PrefetchAction]:
        buf = np.zeros(4 * cap, np.int32)
        n = lib().ihb_sched_drain(self._h, buf.ctypes.data_as(_i), cap)
        return [PrefetchAction("WarmExpert" if buf[4 * i] == PREFETCH_WARM else "EarlyDispatch", int(buf[4 * i + 1]),
                               int(buf[4 * i + 2]), int(buf[4 * i + 3])) for i in range(n)]


# ---- stats ----------------------------------------------------------------------------------------------------------------
@dataclass
class LayerAccuracy:
    layer: int
    n_tokens: int
    hit_rate: float
    expected_hits: float


class AccuracyTracker:
    """Per-layer fraction of predicted experts that were really selected. Reference: routing/stats.rs:17-84."""

    def __init__(self, n_layers: int, top_k: int):
        self.n_layers, self.top_k = n_layers, top_k
        self._h = lib().ihb_acc_create(n_layers, top_k)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().ihb_acc_destroy(self._h)
            self._h = None

    def record(self, prediction: ExpertPrediction, actual_layer: int, actual_experts: Sequence[int]) -> None:
        p, a = _ia(prediction.experts), _ia(actual_experts)
        lib().ihb_acc_record(self._h, actual_layer, p.ctypes.data_as(_i), p.size, a.ctypes.data_as(_i), a.size)

    def hit_rate(self, layer: int) -> float:
        return float(lib().ihb_acc_hit_rate(self._h, layer))

    def expected_hits(self, layer: int) -> float:
        return self.hit_rate(layer) * self.top_k

    def mean_hit_rate(self) -> float:
        return float(lib().ihb_acc_mean_hit_rate(self._h))

    def layer_summaries(self) -> List[LayerAccuracy]:
        return [LayerAccuracy(l, int(lib().ihb_acc_tokens(self._h, l)), self.hit_rate(l), self.expected_hits(l))
                for l in range(self.n_layers)]

    def reset(self) -> None:
        lib().ihb_acc_reset(self._h)


class TraceCollector:
    """Bounded buffer of (layer, hidden state, router logits) triples used to train the learned predictor.
    Reference: routing/stats.rs:90-167."""

    def __init__(self, hidden: int, n_experts: int, max_traces: int):
        self.hidden, self.n_experts, self.max_traces = hidden, n_experts, max_traces
        self._h = lib().ihb_trace_create(hidden, n_experts, max_traces)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().ihb_trace_destroy(self._h)
            self._h = None

    def push(self, layer: int, hidden, logits) -> bool:
        h, l = _fa(hidden), _fa(logits)
        assert h.size == self.hidden and l.size == self.n_experts
        return bool(lib().ihb_trace_push(self._h, layer, h.ctypes.data_as(_f), l.ctypes.data_as(_f)))

    def n_traces(self) -> int:
        return int(lib().ihb_trace_count(self._h, -1))

    def is_full(self) -> bool:
        return self.n_traces() >= self.max_traces

    def drain_layer(self, layer: int) -> Tuple[np.ndarray, np.ndarray, int]:
        n = int(lib().ihb_trace_count(self._h, layer))
        h = np.zeros((max(n, 1), self.hidden), np.float32)
        l = np.zeros((max(n, 1), self.n_experts), np.float32)
        got = lib().ihb_trace_drain_layer(self._h, layer, h.ctypes.data_as(_f), l.ctypes.data_as(_f))
        return h[:got], l[:got], got

    def clear(self) -> None:
        lib().ihb_trace_clear(self._h)
