"""Self-speculation viability curve: how well does a SHALLOW pass (the first ``d`` layers, then the model's own
final norm and head) predict the full model's next token? Self-speculation drafts with the target's first layers,
so its acceptance is about the top-1 agreement at that depth and its draft cost about ``k d / n_layers`` of a step.
Reference: tools/verify_self_speculation.py (agreement of top-1 and of top-1 within the full model's top-4, per depth).
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from ..models.qwen3_moe import rmsnorm


def agreement_curve(model, prompts: Sequence[Sequence[int]], depths: Sequence[int] = (), top_n: int = 4) -> List[dict]:
    """Per depth: share of positions whose shallow arg-max equals the full model's arg-max, share whose shallow
    arg-max lies in the full model's top-n, and the break-even accept length of a k = 2 draft at that depth."""
    cfg = model.cfg
    depths = list(depths) or sorted({max(1, cfg.n_layers * i // 8) for i in range(1, 8)})
    depths = [d for d in depths if 1 <= d < cfg.n_layers]
    taps = tuple(d - 1 for d in depths)                     # residual stream after layer d - 1 = first d layers
    hit = {d: 0 for d in depths}
    near = {d: 0 for d in depths}
    n = 0
    dev = model.w.embed.device
    for p in prompts:
        cache = model.new_cache(len(p) + 1)
        toks = torch.as_tensor(list(p), dtype=torch.long, device=dev)
        hidden = model.forward_hidden(toks, cache, record_routes=False, aux_layers=taps)
        full = model.logits(hidden)
        top1 = full.argmax(-1)
        topn = torch.topk(full, min(top_n, full.shape[-1]), -1).indices
        for d in depths:
            shallow = model.logits(rmsnorm(model.aux_taps[d - 1], model.w.final_norm, cfg.rms_eps)).argmax(-1)
            hit[d] += int((shallow == top1).sum())
            near[d] += int((shallow[:, None] == topn).any(-1).sum())
        n += toks.shape[0]
    rows = []
    for d in depths:
        a = hit[d] / max(1, n)
        k = 2
        draft = k * d / cfg.n_layers
        tau = sum(a ** i for i in range(k + 1))
        rows.append({"depth": d, "top1_agreement": a, "in_top%d" % top_n: near[d] / max(1, n),
                     "draft_cost_steps": draft, "tau_k2": tau, "speedup_k2": tau / (1.0 + draft)})
    return rows
