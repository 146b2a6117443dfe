"""Adapter that plugs the real engine into the ``inferutil.bench`` ``Engine`` seam (the reference only ships the
analytical ``MockEngine`` there, src/inferutil/bench/__init__.py:4-7): step seconds are device-timed, routes are the
router's real choices, the breakdown splits the measured step by the analytical shape."""
from __future__ import annotations

from typing import Optional

from inferutil.bench.engine import DecodeStep, ExpertRoute, PrefillResult, StepBreakdown
from inferutil.hardware import Cluster, measured_b200
from inferutil.latency import decode_latency
from inferutil.model import MoEConfig

from .engine import InferenceEngine, expert_gpu


def moe_config_of(engine: InferenceEngine) -> MoEConfig:
    m = engine.cfg.model
    return MoEConfig(name=m.name, hidden=m.hidden, n_layers=m.n_layers, n_heads=m.n_q_heads, n_kv_heads=m.n_kv_heads,
                     head_dim=m.head_dim, n_experts=m.n_experts, top_k=m.top_k, moe_inter=m.moe_inter, vocab=m.vocab)


class B200Engine:
    def __init__(self, engine: InferenceEngine, cluster: Optional[Cluster] = None, expose_routes: bool = True):
        self.engine = engine
        self.cluster = cluster or Cluster(measured_b200(), max(1, engine.cfg.parallel.world))
        self.expose_routes = expose_routes
        self.cfg = moe_config_of(engine)
        self._shape = (1.0, 0.0, 0.0, 0.0)
        self._i = 0

    @classmethod
    def from_cli(cls, args) -> "B200Engine":
        eng = InferenceEngine.build(args.engine_model, weights=args.engine_weights, device=args.engine_device,
                                    max_seq=args.prompt + args.decode + 64)
        return cls(eng)

    def reset(self, *, plan, dtype_bytes, kv_dtype_bytes, tp, ep, seq_len) -> None:
        b = decode_latency(self.cfg, self.cluster, plan=plan if plan in ("tp", "ep", "hybrid") else "tp",
                           dtype_bytes=dtype_bytes, kv_dtype_bytes=kv_dtype_bytes, seq_len=seq_len,
                           tp=min(tp, self.cluster.n_gpus), ep=min(ep, self.cluster.n_gpus))
        t = b.total_s or 1.0
        self._shape = (b.weight_read_s / t, b.kv_read_s / t, b.comms_s / t, b.compute_s / t)
        self.engine.reset()
        self._i = 0

    def prefill(self, token_ids) -> PrefillResult:
        vocab = self.engine.cfg.model.vocab
        self.engine.reset()
        pre = self.engine.prefill([int(t) % vocab for t in token_ids])
        first = self.engine.decode_step()
        self._i = 0
        return PrefillResult(len(token_ids), pre.seconds, first.seconds)

    def decode_step(self) -> DecodeStep:
        st = self.engine.decode_step()
        i = self._i
        self._i += 1
        routes = ()
        if self.expose_routes:
            m, p = self.engine.cfg.model, self.engine.cfg.parallel
            routes = tuple(ExpertRoute(r.layer, int(e), expert_gpu(int(e), m, p)) for r in st.routes for e in r.experts)
        w, kv, comms, comp = self._shape
        return DecodeStep(i, st.seconds, routes, StepBreakdown(w * st.seconds, kv * st.seconds, comms * st.seconds,
                                                               comp * st.seconds), st.token_id)
