"""FastAPI application: ``GET /health``, ``GET /v1/models``, ``GET /v1/topology``, ``POST /v1/chat/completions``
(SSE chunks, then ``data: [DONE]``) - the reference's contract (server/main.py:11-56)."""
from __future__ import annotations

import os
import time

from fastapi import FastAPI
from fastapi.middleware.cors import CORSMiddleware
from fastapi.responses import JSONResponse, StreamingResponse

from .backends import Backend, EngineBackend, get_backend
from .schemas import ChatRequest, sse, sse_done
from .topology import build_topology


def create_app(backend: Backend = None) -> FastAPI:
    app = FastAPI(title="multi-gpu-inference-console")
    app.add_middleware(CORSMiddleware, allow_origins=["*"], allow_methods=["*"], allow_headers=["*"])
    state = {"backend": backend or get_backend(), "delay": float(os.environ.get("STREAM_DELAY", "0") or 0)}
    app.state.ihb = state

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

    @app.post("/v1/chat/completions")
    def chat(req: ChatRequest):
        t = topo()
        backend = state["backend"]
        if not req.stream:
            text = "".join(c["choices"][0]["delta"]["content"] for c in backend.stream(req, t) if "choices" in c)
            return JSONResponse({"id": "chatcmpl-b200", "object": "chat.completion", "model": req.model,
                                 "choices": [{"index": 0, "message": {"role": "assistant", "content": text},
                                              "finish_reason": "stop"}]})

        def gen():
            for chunk in backend.stream(req, t):
                yield sse(chunk)
                if state["delay"]:
                    time.sleep(state["delay"])
            yield sse_done()

        return StreamingResponse(gen(), media_type="text/event-stream")

    return app
