"""Deterministic token stream for GPU-free demos and contract tests (reference: server/mock_engine.py:13-103).
Every content chunk carries ``x_telemetry`` (eight expert routes of layer ``token_index % num_layers``, speculative
counts); the final chunk is ``x_summary``."""
from __future__ import annotations

from typing import Iterator, List

from .optimization_telemetry import summary_fields
from .schemas import ChatRequest

_WORDS = ("Tensor-parallel decode on eight B200s folds every all-reduce into the GEMV that feeds it so that "
          "single-stream latency stays near the weight-read floor.").split()

# serving profiles a UI can race: per_tok_ms is the emitted rate, forward_tpot_ms / collective_us feed the breakdown
ENGINE_PROFILES = {
    "conifer": {"label": "Conifer", "ttft_ms": 34.0, "per_tok_ms": 8.61, "spec_enabled": True, "proposed": 8,
                "forward_tpot_ms": 8.61, "collective_us": 9.35, "weight_dtype": "fp8"},
    "vllm": {"label": "vLLM", "ttft_ms": 110.0, "per_tok_ms": 11.7, "spec_enabled": False, "proposed": 1,
             "forward_tpot_ms": 11.7, "collective_us": 17.0, "weight_dtype": "bf16"},
}


def engine_profile(name: str) -> dict:
    return ENGINE_PROFILES.get((name or "").lower(), ENGINE_PROFILES["conifer"])


def _experts_for(token_index: int, topo: dict, top_k: int = 8) -> List[dict]:
    layer = token_index % topo["num_layers"]
    n_e = topo["experts_per_layer"]
    row = topo["placement"][str(layer)]
    ids = [(7 * token_index + 13 * k) % n_e for k in range(min(top_k, n_e))]
    return [{"layer": layer, "expert_id": e, "gpu": row[str(e)]} for e in ids]


def mock_stream(req: ChatRequest, topo: dict) -> Iterator[dict]:
    prof = engine_profile(req.engine)
    n = max(1, req.max_tokens)
    spec = prof["spec_enabled"]
    acc_sum = prop_sum = 0
    for i in range(n):
        word = _WORDS[i % len(_WORDS)]
        proposed = prof["proposed"]
        accepted = (2 if i % 4 == 0 else 3) if spec else proposed
        acc_sum += accepted
        prop_sum += proposed
        yield {"id": "chatcmpl-mock", "object": "chat.completion.chunk", "model": req.model,
               "choices": [{"index": 0, "delta": {"content": word if i == 0 else " " + word}, "finish_reason": None}],
               "x_telemetry": {"token_index": i, "t_ms": prof["per_tok_ms"], "experts": _experts_for(i, topo),
                               "spec": {"proposed": proposed, "accepted": accepted}}}
    rate = round(1000.0 / prof["per_tok_ms"], 1)
    yield {"x_summary": {"engine": prof["label"], "ttft_ms": prof["ttft_ms"], "decode_tok_per_s": rate,
                         "prefill_tokens": sum(len(m.content.split()) for m in req.messages), "completion_tokens": n,
                         "spec_enabled": spec, "spec_accept_rate": round(acc_sum / prop_sum, 3),
                         **summary_fields(prof.get("forward_tpot_ms", prof["per_tok_ms"]), rate,
                                          weight_dtype=prof.get("weight_dtype", "bf16"),
                                          collective_us=prof.get("collective_us", 16.0))}}
