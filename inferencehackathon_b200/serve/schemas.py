"""Wire schema of the OpenAI-compatible endpoint (reference: server/schemas.py:5-26; the UI types in
ui/src/types.ts:1-38 are the consumer contract)."""
from __future__ import annotations

import json
from typing import List

from pydantic import BaseModel


class ChatMessage(BaseModel):
    role: str
    content: str = ""


class ChatRequest(BaseModel):
    model: str = "qwen3-235b-a22b"
    messages: List[ChatMessage]
    temperature: float = 0.7
    max_tokens: int = 256
    stream: bool = True
    engine: str = "conifer"      # non-standard: serving profile, lets a UI race two engines


def sse(data: dict) -> str:
    return f"data: {json.dumps(data)}\n\n"


def sse_done() -> str:
    return "data: [DONE]\n\n"


def sse_error(message: str, code: str = "engine_error") -> str:
    """Error frame sent in-stream when the engine fails after the response has started."""
    return sse({"error": {"message": message, "type": code}})
