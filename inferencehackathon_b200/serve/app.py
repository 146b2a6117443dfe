"""FastAPI application: ``GET /health``, ``GET /v1/models``, ``GET /v1/topology``, ``POST /v1/chat/completions``
(SSE chunks, then ``data: [DONE]``) - the reference's contract (server/main.py:11-56) - plus ``GET /metrics``: counters
of this server in the Prometheus text format, with the speculative-decoding counter names that
``spec_metrics.parse_spec_counters`` reads from a vLLM server (so the same scraper works against either)."""
from __future__ import annotations

import os
import time

from fastapi import FastAPI
from fastapi.middleware.cors import CORSMiddleware
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from .backends import Backend, EngineBackend, get_backend
from .schemas import ChatRequest, sse, sse_done
from .topology import build_topology


def create_app(backend: Backend = None) -> FastAPI:
    app = FastAPI(title="multi-gpu-inference-console")
    app.add_middleware(CORSMiddleware, allow_origins=["*"], allow_methods=["*"], allow_headers=["*"])
    state = {"backend": backend or get_backend(), "delay": float(os.environ.get("STREAM_DELAY", "0") or 0)}
    app.state.ihb = state
    counters = {"requests_total": 0, "generation_tokens_total": 0, "prompt_tokens_total": 0, "errors_total": 0,
                "ttft_seconds_sum": 0.0, "ttft_seconds_count": 0, "spec_decode_num_accepted_tokens_total": 0,
                "spec_decode_num_draft_tokens_total": 0, "spec_decode_num_drafts_total": 0}
    state["counters"] = counters

    def observe(chunk: dict) -> None:
        """Updates the counters from the frames the backend emits (telemetry per token, one summary per request)."""
        tel = chunk.get("x_telemetry")
        if tel:
            counters["generation_tokens_total"] += 1
            spec = tel.get("spec") or {}
            if spec.get("proposed"):
                counters["spec_decode_num_drafts_total"] += 1
                counters["spec_decode_num_draft_tokens_total"] += int(spec.get("proposed", 0))
                counters["spec_decode_num_accepted_tokens_total"] += int(spec.get("accepted", 0))
        summ = chunk.get("x_summary")
        if summ:
            counters["prompt_tokens_total"] += int(summ.get("prefill_tokens", 0) or 0)
            if summ.get("ttft_ms") is not None:
                counters["ttft_seconds_sum"] += float(summ["ttft_ms"]) / 1e3
                counters["ttft_seconds_count"] += 1
        if "error" in chunk:
            counters["errors_total"] += 1

    def topo() -> dict:
        b = state["backend"]
        if isinstance(b, EngineBackend):
            m = b.engine.cfg.model
            return build_topology(m.n_layers, m.n_experts, placement_fn=b.placement_fn())
        return build_topology()

    @app.get("/health")
    def health():
        b = state["backend"]
        return {"status": "ok" if getattr(b, "healthy", True) else "degraded", "backend": type(b).__name__}

    @app.get("/v1/models")
    def models():
        ids = ["qwen3-235b-a22b"]
        b = state["backend"]
        if isinstance(b, EngineBackend) and b.engine.cfg.model.name not in ids:
            ids.append(b.engine.cfg.model.name)
        return {"object": "list", "data": [{"id": i, "object": "model"} for i in ids]}

    @app.get("/v1/topology")
    def topology():
        return topo()

    @app.get("/metrics")
    def metrics():
        lines = []
        for k, v in counters.items():
            name = "ihb:" + k
            lines.append(f"# TYPE {name} counter")
            lines.append(f"{name} {float(v)}")
        b = state["backend"]
        lines.append("# TYPE ihb:backend_healthy gauge")
        lines.append(f"ihb:backend_healthy {1.0 if getattr(b, 'healthy', True) else 0.0}")
        return PlainTextResponse("\n".join(lines) + "\n", media_type="text/plain; version=0.0.4")

    @app.post("/v1/chat/completions")
    def chat(req: ChatRequest):
        t = topo()
        backend = state["backend"]
        counters["requests_total"] += 1
        if not req.stream:
            parts = []
            for c in backend.stream(req, t):
                observe(c)
                if "choices" in c:
                    parts.append(c["choices"][0]["delta"]["content"])
            text = "".join(parts)
            return JSONResponse({"id": "chatcmpl-b200", "object": "chat.completion", "model": req.model,
                                 "choices": [{"index": 0, "message": {"role": "assistant", "content": text},
                                              "finish_reason": "stop"}]})

        def gen():
            for chunk in backend.stream(req, t):
                observe(chunk)
                yield sse(chunk)
                if state["delay"]:
                    time.sleep(state["delay"])
            yield sse_done()

        return StreamingResponse(gen(), media_type="text/event-stream")

    return app
