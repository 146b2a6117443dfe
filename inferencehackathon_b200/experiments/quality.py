"""Greedy-output quality gates and the numerical check of block-fp8 weights.

``probe`` collects greedy completions of a fixed prompt set (from an ``InferenceEngine`` or from an OpenAI-compatible
endpoint), ``compare`` / ``compare_ids`` measure agreement between two such runs (exact-match rate and common-prefix
share, per prompt and overall), ``validate_fp8`` compares a block-fp8 matrix product with the unquantised one for one
matrix of each kind. Reference: tools/quality_probe.py, tools/quality_compare.py, tools/validate_fp8_quant.py.
"""
from __future__ import annotations

import argparse
import json
import urllib.request
from typing import Dict, List, Sequence

PROMPTS = [
    "Write a function that checks whether a string reads the same in both directions.",
    "Name the capital of Australia in one sentence.",
    "What separates a stack from a queue?",
    "Multiply 17 by 23 and show the steps.",
    "Begin a story about the keeper of a lighthouse.",
    "List the planets in order of distance from the sun.",
    "Write binary search with comments.",
    "What does status code 404 mean?",
    "Say 'I would like a coffee' in French.",
    "Define recursion with a one-line example.",
]


def prefix_agreement(a: Sequence, b: Sequence) -> float:
    """Longest common prefix as a share of the baseline length (words or token ids)."""
    if not len(a):
        return 1.0 if not len(b) else 0.0
    i = 0
    while i < len(a) and i < len(b) and a[i] == b[i]:
        i += 1
    return i / len(a)


def compare_ids(base: Sequence[Sequence[int]], cand: Sequence[Sequence[int]]) -> dict:
    per = [prefix_agreement(list(a), list(b)) for a, b in zip(base, cand)]
    exact = [list(a) == list(b) for a, b in zip(base, cand)]
    n = max(1, len(per))
    return {"n": len(per), "exact_match_rate": sum(exact) / n, "mean_prefix_agreement": sum(per) / n,
            "min_prefix_agreement": min(per) if per else 1.0}


def compare(base: Dict, cand: Dict, min_agreement: float = 0.8) -> dict:
    """Two ``probe`` outputs ({"outputs": [{"prompt", "text"}]}) -> word-level gate."""
    rows = []
    for a, b in zip(base["outputs"], cand["outputs"]):
        wa, wb = a["text"].split(), b["text"].split()
        rows.append({"prompt": a["prompt"][:40], "agreement": prefix_agreement(wa, wb), "exact": a["text"] == b["text"]})
    n = max(1, len(rows))
    mean = sum(r["agreement"] for r in rows) / n
    return {"per_prompt": rows, "mean_agreement": mean, "exact_match_rate": sum(r["exact"] for r in rows) / n,
            "passed": mean >= min_agreement}


def probe_http(base_url: str, model: str, max_tokens: int = 96, prompts: Sequence[str] = PROMPTS, timeout: float = 120.0) -> dict:
    outs = []
    for p in prompts:
        body = json.dumps({"model": model, "messages": [{"role": "user", "content": p}], "temperature": 0.0,
                           "max_tokens": max_tokens, "stream": False}).encode()
        req = urllib.request.Request(base_url.rstrip("/") + "/v1/chat/completions", data=body,
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=timeout) as r:
            d = json.loads(r.read())
        outs.append({"prompt": p, "text": d["choices"][0]["message"]["content"]})
    return {"endpoint": base_url, "model": model, "outputs": outs}


def probe_engine(engine, prompts: Sequence[Sequence[int]], new_tokens: int = 32) -> dict:
    return {"outputs": [{"prompt": list(p), "tokens": engine.generate(list(p), new_tokens).tokens} for p in prompts]}


def validate_fp8(hidden: int = 1024, inter: int = 512, vocab: int = 4096, seed: int = 0, tol: float = 0.05) -> List[dict]:
    """For one matrix of each kind (q / o projection, expert gate and down, head): relative error of
    ``fake-quantised activation x block-fp8 weight`` against the fp32 product."""
    import torch
    from ..models.quant import quant_block
    from ..models.qwen3_moe import fake_quant_act
    g = torch.Generator().manual_seed(seed)
    kinds = {"attn_q": (hidden, hidden), "attn_o": (hidden, hidden), "expert_gate": (inter, hidden),
             "expert_down": (hidden, inter), "lm_head": (vocab, hidden)}
    rows = []
    for name, (r, c) in kinds.items():
        w = torch.randn(r, c, generator=g) * (c ** -0.5)
        x = torch.randn(4, c, generator=g)
        ref = x @ w.t()
        qw = quant_block(w)
        got = fake_quant_act(x, "fp8") @ qw.dequant().t()
        rel = float((got - ref).norm() / ref.norm())
        cos = float(torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0))
        rows.append({"matrix": name, "shape": [r, c], "rel_error": rel, "cosine": cos, "ok": rel < tol})
    return rows


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m inferencehackathon_b200.experiments.quality")
    sub = p.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("probe"); s.add_argument("--base", required=True); s.add_argument("--model", default="qwen3-235b-a22b")
    s.add_argument("--tokens", type=int, default=96); s.add_argument("--out", required=True)
    s = sub.add_parser("compare"); s.add_argument("baseline"); s.add_argument("candidate"); s.add_argument("--out")
    sub.add_parser("validate-fp8")
    a = p.parse_args(argv)
    if a.cmd == "probe":
        r = probe_http(a.base, a.model, a.tokens)
        with open(a.out, "w") as f:
            json.dump(r, f, indent=1)
        print(f"{len(r['outputs'])} completions -> {a.out}")
    elif a.cmd == "compare":
        r = compare(json.load(open(a.baseline)), json.load(open(a.candidate)))
        print(json.dumps({k: v for k, v in r.items() if k != "per_prompt"}, indent=1))
        if a.out:
            with open(a.out, "w") as f:
                json.dump(r, f, indent=1)
        return 0 if r["passed"] else 1
    else:
        rows = validate_fp8()
        print(json.dumps(rows, indent=1))
        return 0 if all(r["ok"] for r in rows) else 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
