"""Streaming backends behind ``POST /v1/chat/completions`` (reference: server/backend.py:15-143):

* :class:`MockBackend` - the deterministic mock,
* :class:`VLLMBackend` - proxy to a vLLM server over HTTP, re-framing its SSE and stamping wall-clock ``t_ms``,
* :class:`EngineBackend` - this repository's engine: real tokens, REAL router selections in ``x_telemetry``
  (the reference synthesises them in both of its backends, server/mock_engine.py:34-48, server/backend.py:100-125),
  device-timed ``t_ms``, real speculative counts.
"""
from __future__ import annotations

import json
import os
import threading
import time
import urllib.request
from abc import ABC, abstractmethod
from typing import Iterator, Optional

from .mock_engine import mock_stream
from .optimization_telemetry import B200X1, B200X8, H100X8, summary_fields
from .schemas import ChatRequest
from .spec_metrics import accept_stats, fetch_metrics

VLLM_URL = os.environ.get("VLLM_URL", "http://localhost:8001")


class Backend(ABC):
    @abstractmethod
    def stream(self, req: ChatRequest, topo: dict) -> Iterator[dict]:
        ...


class MockBackend(Backend):
    def stream(self, req: ChatRequest, topo: dict) -> Iterator[dict]:
        yield from mock_stream(req, topo)


def _synthetic_telemetry(token_index: int, t_ms: float, topo: dict) -> dict:
    """vLLM does not expose routing: cycle through the placement so that the GPU view stays alive."""
    n_layers, n_e = topo.get("num_layers", 94), topo.get("experts_per_layer", 128)
    layer = token_index % n_layers
    row = topo.get("placement", {}).get(str(layer), {})
    ids = [(7 * token_index + 13 * k) % n_e for k in range(8)]
    return {"token_index": token_index, "t_ms": round(t_ms, 2),
            "experts": [{"layer": layer, "expert_id": e, "gpu": row.get(str(e), e % 8)} for e in ids],
            "spec": {"proposed": 8, "accepted": 0}}


class VLLMBackend(Backend):
    def __init__(self, url: Optional[str] = None, scrape_spec: bool = True, routing_sock: Optional[str] = None):
        self.url = url or VLLM_URL
        self.scrape_spec = scrape_spec
        # a vLLM started through serve/vllm_tools.py streams its routers' choices over this socket; without it the
        # telemetry cycles through the placement
        sock = routing_sock if routing_sock is not None else os.environ.get("VLLM_ROUTING_SOCK", "")
        self.feed = None
        self.pipeline = None
        if sock:
            from .vllm_tools import RoutingFeedReader
            on_record = None
            if os.environ.get("ROUTE_PIPELINE"):
                # the fed routing also drives the native predictor + prefetch scheduler (x_summary.route_prediction)
                from ..routing.pipeline import RoutingPipeline
                self.pipeline = RoutingPipeline(int(os.environ.get("VLLM_NUM_LAYERS", "94")),
                                                int(os.environ.get("VLLM_NUM_EXPERTS", "128")), 8)
                on_record = lambda _tok, layer, experts: self.pipeline.on_layer(layer, experts)   # noqa: E731
            self.feed = RoutingFeedReader(sock, on_record=on_record)

    def _telemetry(self, n: int, t_ms: float, topo: dict) -> dict:
        if self.feed is not None:
            from .vllm_tools import telemetry_from_feed
            tel = telemetry_from_feed(self.feed, n, t_ms, topo, all_layers=bool(os.environ.get("X_TELEMETRY_ALL_LAYERS")))
            if tel is not None:
                return tel
        return _synthetic_telemetry(n, t_ms, topo)

    def stream(self, req: ChatRequest, topo: dict) -> Iterator[dict]:
        body = json.dumps({"model": os.environ.get("VLLM_MODEL", "qwen3-235b-fp8"),
                           "messages": [{"role": m.role, "content": m.content} for m in req.messages],
                           "temperature": req.temperature, "max_tokens": req.max_tokens, "stream": True,
                           "chat_template_kwargs": {"enable_thinking": False}}).encode()
        request = urllib.request.Request(f"{self.url}/v1/chat/completions", data=body,
                                         headers={"Content-Type": "application/json"}, method="POST")
        before = fetch_metrics(self.url) if self.scrape_spec else ""
        t0 = time.time()
        t_first = None
        n = 0
        pending = b""
        done = False
        with urllib.request.urlopen(request, timeout=120) as resp:
            for raw in resp:
                pending += raw
                while b"\n\n" in pending and not done:
                    frame, pending = pending.split(b"\n\n", 1)
                    text = frame.decode(errors="replace").strip()
                    if not text.startswith("data:"):
                        continue
                    payload = text[5:].strip()
                    if payload == "[DONE]":
                        done = True
                        break
                    try:
                        chunk = json.loads(payload)
                    except json.JSONDecodeError:
                        continue
                    if chunk.get("choices", [{}])[0].get("delta", {}).get("content"):
                        now = time.time()
                        t_first = t_first or now
                        chunk["x_telemetry"] = self._telemetry(n, 1e3 * (now - t0), topo)
                        n += 1
                    yield chunk
                if done:
                    break
        elapsed = time.time() - t0
        ttft = (t_first - t0) if t_first else 0.0
        rate = round(max(n - 1, 0) / max(elapsed - ttft if t_first else elapsed, 1e-3), 1)
        spec = accept_stats(before, fetch_metrics(self.url)) if self.scrape_spec else {"accept_rate": 0.0}
        extra = summary_fields(round(1000.0 / rate, 2), rate, weight_dtype="bf16", collective_us=17.0) if rate > 0 else {}
        yield {"x_summary": {"ttft_ms": round(1e3 * ttft, 1), "decode_tok_per_s": rate,
                             "prefill_tokens": sum(len(m.content.split()) for m in req.messages),
                             "completion_tokens": n, "spec_accept_rate": spec["accept_rate"], **extra,
                             **({"route_prediction": self.pipeline.stats()} if self.pipeline is not None else {})}}


class EngineBackend(Backend):
    """Serves one request at a time from an :class:`InferenceEngine` (B=1 by design)."""

    def __init__(self, engine, tokenizer=None, label: str = "b200moe", spec_driver=None):
        from ..runtime.engine import expert_gpu
        from .tokenizer import ByteTokenizer
        self.engine = engine
        self.tok = tokenizer or ByteTokenizer(engine.cfg.model.vocab)
        self.label = label
        self.spec = spec_driver
        self._lock = threading.Lock()
        self._gpu_of = lambda e: expert_gpu(e, engine.cfg.model, engine.cfg.parallel)
        self.healthy = True
        # ROUTE_PIPELINE=1: every token's real routing drives the native predictor + prefetch scheduler; the turn's
        # x_summary then carries their hit rates (what an expert-prefetch scheme would have achieved on this turn)
        self.pipeline = None
        if os.environ.get("ROUTE_PIPELINE"):
            from ..routing.pipeline import RoutingPipeline
            m = engine.cfg.model
            self.pipeline = RoutingPipeline(m.n_layers, m.n_experts, m.top_k, n_gpus=max(engine.cfg.parallel.world, 1))

    def placement_fn(self):
        return self._gpu_of

    def _routes(self, routes, token_index: int):
        n_layers = max(1, len(routes))
        pick = routes if os.environ.get("X_TELEMETRY_ALL_LAYERS") else routes[token_index % n_layers: token_index % n_layers + 1]
        return [{"layer": r.layer, "expert_id": int(e), "gpu": int(self._gpu_of(int(e)))} for r in pick for e in r.experts]

    def stream(self, req: ChatRequest, topo: dict) -> Iterator[dict]:
        from ..runtime.sampler import SamplingParams
        prompt = self.tok.encode("\n".join(m.content for m in req.messages))
        m = self.engine.cfg.model
        room = self.engine.cfg.max_seq - len(prompt) - 1
        if room < 1:
            prompt = prompt[-(self.engine.cfg.max_seq // 2):]
            room = self.engine.cfg.max_seq - len(prompt) - 1
        n_new = max(1, min(req.max_tokens, room))
        with self._lock:
            self.engine.set_sampling(SamplingParams(temperature=0.0 if self.spec is not None else req.temperature, seed=0))
            self.engine.reset()
            proposed = accepted = 0
            step_s = []
            try:
                pre = self.engine.prefill(prompt)
                tokens = [pre.next_token]
                if self.spec is not None and hasattr(self.spec, "begin"):
                    self.spec.begin(prompt)
                routes = list(self.engine.model.last_routes) if self.engine.gpu is None else self.engine.gpu.last_routes()
                yield self._chunk(req, 0, tokens[0], 1e3 * pre.seconds, routes, 1, 1)
                while len(tokens) < n_new:
                    if self.spec is not None:
                        rnd = self.spec.step(tokens[-1])
                        proposed += rnd.n_proposed
                        accepted += rnd.n_accepted
                        per = 1e3 * rnd.seconds / max(1, len(rnd.tokens))
                        for t in rnd.tokens:
                            if len(tokens) >= n_new:
                                break
                            tokens.append(t)
                            step_s.append(per * 1e-3)
                            yield self._chunk(req, len(tokens) - 1, t, per, rnd.routes, rnd.n_proposed, rnd.n_accepted)
                    else:
                        st = self.engine.decode_step()
                        tokens.append(st.token_id)
                        step_s.append(st.seconds)
                        yield self._chunk(req, len(tokens) - 1, st.token_id, 1e3 * st.seconds, st.routes, 1, 1)
            except Exception as e:                      # surfaced in-stream; the server stays up
                self.healthy = False
                yield {"error": {"message": f"{type(e).__name__}: {e}", "type": "engine_error"}}
                return
        total = sum(step_s)
        rate = round(len(step_s) / total, 1) if total > 0 else 0.0
        world = self.engine.cfg.parallel.world
        dtype = {"fp8_block": "fp8", "bf16": "bf16"}.get(self.engine.cfg.quant.weights, "bf16")
        profile = B200X8 if world >= 8 else B200X1 if self.engine.device.type == "cuda" else H100X8
        extra = summary_fields(1000.0 / rate, rate, weight_dtype=dtype, collective_us=5.0, ctx=len(prompt),
                               profile=profile) if rate > 0 else {}
        yield {"x_summary": {"engine": self.label, "ttft_ms": round(1e3 * pre.seconds, 3), "decode_tok_per_s": rate,
                             "prefill_tokens": len(prompt), "completion_tokens": len(tokens),
                             "spec_enabled": self.spec is not None,
                             "spec_accept_rate": round(accepted / proposed, 3) if proposed else 0.0, **extra,
                             **({"route_prediction": self.pipeline.stats()} if self.pipeline is not None else {})}}

    def _chunk(self, req, i, token, t_ms, routes, proposed, accepted) -> dict:
        if self.pipeline is not None and routes:
            self.pipeline.on_token({r.layer: r.experts for r in routes})
        return {"id": "chatcmpl-b200", "object": "chat.completion.chunk", "model": req.model,
                "choices": [{"index": 0, "delta": {"content": self.tok.piece(int(token))}, "finish_reason": None}],
                "x_telemetry": {"token_index": i, "t_ms": round(t_ms, 4), "experts": self._routes(routes, i),
                                "spec": {"proposed": int(proposed), "accepted": int(accepted)}}}


def _vllm_healthy(url: Optional[str] = None) -> bool:
    try:
        urllib.request.urlopen(f"{url or VLLM_URL}/health", timeout=2)
        return True
    except Exception:
        return False


def _build_engine_backend() -> Backend:
    from ..runtime.engine import InferenceEngine
    model = os.environ.get("ENGINE_MODEL", "tiny")
    device = os.environ.get("ENGINE_DEVICE", "cpu")
    weights = os.environ.get("ENGINE_WEIGHTS", "fp32" if device == "cpu" else "fp8_block")
    # ENGINE_CHECKPOINT: a directory of Hugging Face safetensors shards (else random weights of the named architecture);
    # ENGINE_TOKENIZER: a Hugging Face tokenizer directory (else the reversible byte mapping)
    eng = InferenceEngine.build(model, weights=weights, kv=os.environ.get("ENGINE_KV") or None, device=device,
                                max_seq=int(os.environ.get("ENGINE_MAX_SEQ", "1024")),
                                checkpoint=os.environ.get("ENGINE_CHECKPOINT") or None)
    tok = None
    if os.environ.get("ENGINE_TOKENIZER"):
        from .tokenizer import HFTokenizer
        tok = HFTokenizer(os.environ["ENGINE_TOKENIZER"])
    return EngineBackend(eng, tokenizer=tok)


def get_backend() -> Backend:
    """``BACKEND=mock|engine|vllm``; unset: vLLM when its health probe answers, else the mock."""
    choice = os.environ.get("BACKEND", "").lower()
    if choice == "mock":
        return MockBackend()
    if choice == "engine":
        return _build_engine_backend()
    if choice == "vllm" or _vllm_healthy():
        if _vllm_healthy():
            return VLLMBackend()
    return MockBackend()
