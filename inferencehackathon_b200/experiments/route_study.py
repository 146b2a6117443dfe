"""Route statistics of a decode run on this engine's model: what an expert-prefetch or placement scheme would see.

Decoding is driven one token at a time, so every generated token yields one clean ``layer -> top-k experts`` vector
(plus the hidden state entering each router). From these the study reports
  * per-layer expert activation frequency and the hot-expert coverage curve (experts staged vs share of hits),
  * predictability: persistence (token t's experts at token t + 1, same layer), static-hot coverage, their union,
    layer-to-layer overlap, and the accuracy of applying layer L + 1's router to layer L's input (direct proxy),
  * per-token GPU load imbalance (busiest GPU among the chosen experts) under round-robin, co-activation-affinity
    placement and round-robin with the R hottest experts replicated everywhere,
  * the share of co-activation weight kept on one GPU by each placement.
Reference: tools/routing_analysis.py, tools/routing_predict.py (imbalance / predictability / coverage numbers),
tools/verify_route_prediction.py (direct proxy, layer-to-layer and token-to-token overlap).
"""
from __future__ import annotations

import argparse
import json
from collections import Counter, defaultdict
from typing import Dict, List, Sequence

import torch

from inferutil.routing import CoActGraph, greedy_partition, ingest_telemetry, placement_stats, round_robin_placement


def collect_routes(engine, prompts: Sequence[Sequence[int]], new_tokens: int = 32):
    """-> (routes[token][layer] = list of experts, router inputs[token][layer] = hidden state or None)."""
    model = engine.model
    routes: List[List[List[int]]] = []
    hiddens: List[List[torch.Tensor]] = []
    cur_h: Dict[int, torch.Tensor] = {}

    def tap(L, h, router_w, top_k, renorm):
        from ..models.qwen3_moe import route
        cur_h[L] = h[-1].detach().float().cpu()
        return route(h, router_w, top_k, renorm)

    prev = model.route_fn
    model.route_fn = tap
    try:
        for p in prompts:
            engine.reset()
            engine.prefill(list(p))
            for _ in range(new_tokens):
                cur_h.clear()
                engine.decode_step()
                per_layer = {r.layer: list(r.experts) for r in model.last_routes}
                n_layers = model.cfg.n_layers
                routes.append([per_layer.get(L, []) for L in range(n_layers)])
                hiddens.append([cur_h.get(L) for L in range(n_layers)])
    finally:
        model.route_fn = prev
    return routes, hiddens


def _imbalance(experts: Sequence[int], gpu_of, n_gpus: int, replicated=frozenset()) -> float:
    load = [0] * n_gpus
    for e in experts:
        if e in replicated:
            continue                                  # a replicated expert runs wherever load is lowest: counted below
        load[gpu_of(e)] += 1
    for e in experts:
        if e in replicated:
            load[load.index(min(load))] += 1
    return max(load) / (len(experts) / n_gpus) if experts else 1.0


def analyze(routes, hiddens, routers: Sequence[torch.Tensor], n_experts: int, top_k: int, n_gpus: int = 8,
            hot_k: int = 16, replicate: int = 4) -> dict:
    n_tok, n_layers = len(routes), len(routes[0]) if routes else 0
    freq = [Counter() for _ in range(n_layers)]
    for tok in routes:
        for L, ex in enumerate(tok):
            freq[L].update(ex)
    hot = [set(e for e, _ in freq[L].most_common(hot_k)) for L in range(n_layers)]
    rep = [frozenset(e for e, _ in freq[L].most_common(replicate)) for L in range(n_layers)]
    # predictability ---------------------------------------------------------------------------------------------
    pers = stat = comb = l2l = proxy = 0.0
    n_p = n_l = n_x = 0
    for t in range(n_tok):
        for L in range(n_layers):
            cur = set(routes[t][L])
            if not cur:
                continue
            if t + 1 < n_tok:
                nxt = set(routes[t + 1][L])
                pers += len(cur & nxt) / top_k
                stat += len(nxt & hot[L]) / top_k
                comb += len(nxt & (cur | hot[L])) / top_k
                n_p += 1
            if L + 1 < n_layers and routes[t][L + 1]:
                l2l += len(cur & set(routes[t][L + 1])) / top_k
                n_l += 1
                h = hiddens[t][L]
                if h is not None:
                    guess = torch.topk(h @ routers[L + 1].float().cpu().t(), top_k).indices.tolist()
                    proxy += len(set(guess) & set(routes[t][L + 1])) / top_k
                    n_x += 1
    # coverage curve ------------------------------------------------------------------------------------------------
    coverage = {}
    for k in (4, 8, 16, 32, 64):
        if k <= n_experts:
            hit = sum(sum(c for _, c in freq[L].most_common(k)) for L in range(n_layers))
            tot = sum(sum(freq[L].values()) for L in range(n_layers))
            coverage[k] = hit / tot if tot else 0.0
    # imbalance -------------------------------------------------------------------------------------------------------
    per_gpu = max(1, n_experts // n_gpus)
    imb_rr = imb_blk = imb_rep = 0.0
    n_i = 0
    for tok in routes:
        for L, ex in enumerate(tok):
            if not ex:
                continue
            imb_rr += _imbalance(ex, lambda e: e % n_gpus, n_gpus)
            imb_blk += _imbalance(ex, lambda e: min(n_gpus - 1, e // per_gpu), n_gpus)
            imb_rep += _imbalance(ex, lambda e: e % n_gpus, n_gpus, rep[L])
            n_i += 1
    return {"tokens": n_tok, "layers": n_layers, "random_baseline": top_k / n_experts,
            "persistence": pers / max(1, n_p), "static_hot": stat / max(1, n_p), "combined": comb / max(1, n_p),
            "layer_to_layer": l2l / max(1, n_l), "direct_proxy": proxy / max(1, n_x), "coverage": coverage,
            "imbalance": {"round_robin": imb_rr / max(1, n_i), "contiguous": imb_blk / max(1, n_i),
                          f"round_robin_plus_{replicate}_replicated": imb_rep / max(1, n_i)},
            "activation_frequency": [dict(freq[L].most_common(8)) for L in range(n_layers)]}


def placement_report(routes, n_experts: int, n_gpus: int = 8) -> dict:
    """Share of co-activation weight (within a layer and between neighbouring layers) that stays on one GPU:
    round-robin against the affinity placement grown from the same routes."""
    n_layers = len(routes[0]) if routes else 0
    g = CoActGraph(n_experts=n_experts, n_layers=n_layers)
    ingest_telemetry(g, ({"experts": [{"layer": L, "expert_id": e} for L in range(n_layers) for e in tok[L]]}
                         for tok in routes))
    return {"round_robin": placement_stats(g, round_robin_placement(n_gpus, n_experts, n_layers), "round_robin"),
            "affinity": placement_stats(g, greedy_partition(g, n_gpus, n_experts, n_layers), "affinity")}


def main(argv=None) -> int:
    from ..runtime.engine import InferenceEngine
    p = argparse.ArgumentParser(prog="python -m inferencehackathon_b200.experiments.route_study")
    p.add_argument("--model", default="small"); p.add_argument("--prompts", type=int, default=4)
    p.add_argument("--prompt-len", type=int, default=16); p.add_argument("--tokens", type=int, default=24)
    p.add_argument("--gpus", type=int, default=8); p.add_argument("--device", default="cpu"); p.add_argument("--out")
    a = p.parse_args(argv)
    eng = InferenceEngine.build(a.model, device=a.device, backend="torch", max_seq=a.prompt_len + a.tokens + 8)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, eng.cfg.model.vocab, (a.prompt_len,), generator=g).tolist() for _ in range(a.prompts)]
    routes, hid = collect_routes(eng, prompts, a.tokens)
    m = eng.cfg.model
    rep = analyze(routes, hid, [lw.router for lw in eng.weights.layers], m.n_experts, m.top_k, a.gpus)
    print(json.dumps({k: v for k, v in rep.items() if k != "activation_frequency"}, indent=1))
    if a.out:
        with open(a.out, "w") as f:
            json.dump(rep, f, indent=1)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
