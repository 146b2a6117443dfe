"""Speculative decoding benchmark on one engine: plain greedy decoding against speculative rounds with (a) the n-gram
drafter on a prompt made of a repeated random block and (b) a random-init one-layer EAGLE-3-style head with tree
verify. Checks that the speculative output equals the plain one (greedy is lossless), then reports tokens per second,
accept length, acceptance rate, target forwards per token and the verify cost in decode-step units (tau / speedup).

    python -m inferencehackathon_b200.spec.bench --model tiny --device cpu --backend torch
    python -m inferencehackathon_b200.spec.bench --model qwen3-235b-a22b --layers 8 --weights fp8_block --device cuda:0

Prints one JSON line. Reference counterparts: kernels/spec_decode_loop.cu (measured forward x accept length with an
n-gram drafter, kernels/spec_loop_e2e.txt) and kernels/ngram_drafter_tau.py; the EAGLE-3 numbers there are anchored
on a published accept length, here the head is random-init, so its acceptance is near zero by construction and the
run shows the cost side (verify windows on the tensor cores) and the lossless rule.
"""
from __future__ import annotations

import argparse
import json
import time
from typing import List, Optional, Sequence

import torch

from ..runtime.engine import InferenceEngine
from . import driver as D
from .eagle_head import EagleHead, EagleHeadConfig, default_aux_layers
from .ngram import NGramDrafter


def repeated_prompt(vocab: int, block: int = 64, repeats: int = 16, seed: int = 0) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    blk = torch.randint(0, vocab, (block,), generator=g).tolist()
    return blk * repeats


def _sync(engine) -> None:
    if engine.device.type == "cuda":
        torch.cuda.synchronize(engine.device)


def run_plain(engine, prompt: Sequence[int], n: int) -> dict:
    engine.reset()
    _sync(engine)
    t0 = time.perf_counter()
    res = engine.generate(list(prompt), n)
    _sync(engine)
    dt = time.perf_counter() - t0
    return {"tokens": res.tokens, "seconds": dt, "decode_tok_s": res.decode_tok_per_s}


def run_spec(engine, source, prompt: Sequence[int], n: int, *, depth: int, width: int, tree=None, aux=(),
             floor_fraction: float = 0.86) -> dict:
    drv = D.SpecDriver(engine, source, depth=depth, width=width, tree=tree, aux_layers=aux, floor_fraction=floor_fraction)
    engine.reset()
    pre = engine.prefill(list(prompt))
    drv.begin(prompt)
    out = [pre.next_token]
    _sync(engine)
    t0 = time.perf_counter()
    rounds = 0
    while len(out) < n:
        rnd = drv.step(out[-1])
        rounds += 1
        out.extend(rnd.tokens[: n - len(out)])
    _sync(engine)
    dt = time.perf_counter() - t0
    tel = drv.telemetry
    return {"tokens": out, "seconds": dt, "decode_tok_s": (len(out) - 1) / dt if dt > 0 else 0.0, "rounds": rounds,
            "accept_length": tel.mean_accept_length(), "acceptance_rate": tel.acceptance_rate(),
            "mean_verify_depth": tel.mean_verify_depth(), "target_forwards": drv.runner.forwards,
            "forwards_per_token": drv.runner.forwards / max(1, len(out) - 1)}


def verify_forward_sweep(engine, prompt: Sequence[int], ms=(1, 4, 8, 16), reps: int = 10) -> dict:
    """Full-forward time of a verify window of M tokens, T(M), device-timed, for the M of a speculative round, beside
    the plain decode step: how flat the verify cost is in M decides what a drafter's accept length is worth
    (reference: the T(M) table of kernels/decode_step_tp8.cu:3154-3175; T(16) / T(1) = 1.003 for its GEMM path)."""
    if engine.device.type != "cuda":
        return {}
    engine.reset()
    pre = engine.prefill(list(prompt))
    dev = engine.device

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) * 1e3 / reps

    base = engine.seq_len
    out = {}
    toks = list(prompt[:max(ms)])
    for m in ms:
        out[f"T({m})_us"] = round(timed(lambda: engine.logits_for(toks[:m], commit=False)), 1)
    def step():
        engine.gpu.run_steps(1)
        engine.gpu.rollback(base)
    out["decode_step_us"] = round(timed(step), 1)
    engine.gpu.cur_token.fill_(pre.next_token)
    for m in ms:
        out[f"T({m})/T(1)"] = round(out[f"T({m})_us"] / out[f"T({ms[0]})_us"], 3)
    out["T(1)/decode_step"] = round(out[f"T({ms[0]})_us"] / out["decode_step_us"], 2)
    return out


def main(argv: Optional[Sequence[str]] = None) -> int:
    p = argparse.ArgumentParser(prog="python -m inferencehackathon_b200.spec.bench")
    p.add_argument("--model", default="tiny")
    p.add_argument("--layers", type=int, default=None)
    p.add_argument("--weights", default="fp32")
    p.add_argument("--device", default="cpu")
    p.add_argument("--backend", default="auto")
    p.add_argument("--block", type=int, default=64)
    p.add_argument("--repeats", type=int, default=16)
    p.add_argument("--new-tokens", type=int, default=64)
    p.add_argument("--depth", type=int, default=8)
    p.add_argument("--tree", default="4x4", help="depth x branch of the EAGLE tree")
    p.add_argument("--max-candidates", type=int, default=16, help="beam budget of the tree (candidates verified per round)")
    p.add_argument("--skip-eagle", action="store_true")
    p.add_argument("--tm-sweep", action="store_true", help="also time verify windows of 1, 4, 8, 16 tokens (GPU only)")
    a = p.parse_args(argv)
    n_prompt = a.block * a.repeats
    eng = InferenceEngine.build(a.model, weights=a.weights, device=a.device, backend=a.backend, n_layers=a.layers,
                                max_seq=n_prompt + a.new_tokens + 2 * a.max_candidates + 64)
    m = eng.cfg.model
    prompt = repeated_prompt(m.vocab, a.block, a.repeats)
    plain = run_plain(eng, prompt, a.new_tokens)
    out = {"model": m.name, "device": str(eng.device), "backend": eng.backend, "prompt_tokens": n_prompt,
           "new_tokens": a.new_tokens, "plain_tok_s": plain["decode_tok_s"]}
    ng = run_spec(eng, NGramDrafter(3, min_n=1), prompt, a.new_tokens, depth=a.depth, width=1, floor_fraction=1.0)
    out["ngram"] = {k: v for k, v in ng.items() if k != "tokens"}
    out["ngram"]["lossless"] = ng["tokens"] == plain["tokens"]
    out["ngram"]["speedup"] = ng["decode_tok_s"] / plain["decode_tok_s"] if plain["decode_tok_s"] else 0.0
    if out["ngram"]["speedup"] > 0:
        out["ngram"]["verify_cost_steps"] = out["ngram"]["accept_length"] / out["ngram"]["speedup"]
    if not a.skip_eagle:
        td, tb = (int(x) for x in a.tree.lower().split("x"))
        aux = default_aux_layers(m.n_layers)
        head = EagleHead(EagleHeadConfig(hidden=m.hidden, n_heads=max(1, m.n_q_heads // 2), n_kv_heads=max(1, m.n_kv_heads),
                                         head_dim=m.head_dim, draft_vocab=min(m.vocab, 32000), target_vocab=m.vocab),
                         eng.weights.embed)
        eg = run_spec(eng, head, prompt, a.new_tokens, depth=td, width=tb, tree=(td, tb, a.max_candidates), aux=aux)
        out["eagle_tree"] = {k: v for k, v in eg.items() if k != "tokens"}
        out["eagle_tree"]["lossless"] = eg["tokens"] == plain["tokens"]
        out["eagle_tree"]["speedup"] = eg["decode_tok_s"] / plain["decode_tok_s"] if plain["decode_tok_s"] else 0.0
    if a.tm_sweep:
        out["verify_forward"] = verify_forward_sweep(eng, prompt)
    print(json.dumps(out))
    return 0 if out["ngram"]["lossless"] and out.get("eagle_tree", {}).get("lossless", True) else 1


if __name__ == "__main__":
    raise SystemExit(main())
