"""EAGLE-3-style one-layer draft head (PyTorch), usable as a candidate source of the speculative drivers.

Input of head position ``i`` is the pair (target feature of position ``i``, embedding of token ``i + 1``); it
predicts token ``i + 2``. The target feature is a projection of hidden states tapped at three depths of the target
(low / middle / high); for drafted positions, where no target feature exists yet, the head's own hidden state is fed
back. One pre-norm decoder layer (GQA attention with RoPE over the head's own KV cache, dense SwiGLU MLP) and a
reduced draft vocabulary with a draft-to-target id map.

Reference: the head the reference's engine drives through ``AuxModelRunner::forward_single_with_aux(ctx, tok,
aux_layers=[1, 46, 90])`` (engine/src/spec/eagle3_engine.rs:27-60) and engine/src/spec/draft_vocab.rs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..models.qwen3_moe import apply_rope, rmsnorm, rope_tables
from . import native as N
from .driver import Candidate


@dataclass
class EagleHeadConfig:
    hidden: int
    n_heads: int = 8
    n_kv_heads: int = 2
    head_dim: int = 64
    intermediate: int = 0            # 0: 2 x hidden
    draft_vocab: int = 32000
    target_vocab: int = 151936
    rope_theta: float = 1e6
    rms_eps: float = 1e-6
    n_taps: int = 3


def default_aux_layers(n_layers: int) -> Tuple[int, int, int]:
    """Low / middle / high taps, e.g. (1, 46, 90) for 94 layers."""
    return (min(1, n_layers - 1), n_layers // 2 - 1 if n_layers >= 4 else n_layers // 2, max(0, n_layers - 4) if n_layers >= 8 else n_layers - 1)


class EagleHead:
    """Random-init (``seed``) or loaded head. ``candidates(context, chain_so_far, width)`` implements the candidate
    source protocol; ``bind(runner)`` gives access to the target features recorded by the engine runner."""

    def __init__(self, cfg: EagleHeadConfig, embed: torch.Tensor, device=None, dtype=torch.float32, seed: int = 0,
                 d2t: Optional[torch.Tensor] = None):
        self.cfg = cfg
        dev = device or embed.device
        g = torch.Generator(device="cpu").manual_seed(seed)
        H, hd = cfg.hidden, cfg.head_dim
        inter = cfg.intermediate or 2 * H

        def w(*shape, std=0.02):
            return (torch.randn(*shape, generator=g) * std).to(device=dev, dtype=dtype)

        self.embed = embed                                   # shared with the target
        self.fc = w(H, cfg.n_taps * H)
        self.norm_e = torch.ones(H, device=dev, dtype=dtype)
        self.norm_g = torch.ones(H, device=dev, dtype=dtype)
        self.wq = w(cfg.n_heads * hd, 2 * H)
        self.wk = w(cfg.n_kv_heads * hd, 2 * H)
        self.wv = w(cfg.n_kv_heads * hd, 2 * H)
        self.wo = w(H, cfg.n_heads * hd)
        self.norm_mlp = torch.ones(H, device=dev, dtype=dtype)
        self.w_gu = w(2 * inter, H)
        self.w_d = w(H, inter)
        self.norm_out = torch.ones(H, device=dev, dtype=dtype)
        self.lm_head = w(cfg.draft_vocab, H)
        if d2t is None:                                      # evenly spread ids; a trained head ships its own map
            d2t = torch.arange(cfg.draft_vocab, dtype=torch.int64) * max(1, cfg.target_vocab // cfg.draft_vocab)
        self.d2t = d2t.to(torch.int32).cpu().numpy()
        self.device, self.dtype = dev, dtype
        self.runner = None
        self.expert_fn = None                                # optional: hidden state -> predicted expert ids
        self._reset_cache()

    def bind(self, runner) -> None:
        self.runner = runner
        self._reset_cache()

    def _reset_cache(self) -> None:
        self._k: List[torch.Tensor] = []                     # per committed head position: [n_kv, hd]
        self._v: List[torch.Tensor] = []
        self._pos0 = None                                    # absolute position of head cache entry 0
        self._hid: Dict[int, torch.Tensor] = {}              # absolute position -> head hidden state
        self._tokens: List[int] = []                         # token i + 1 paired with cache entry i
        self._states: Dict[Tuple[int, Tuple[int, ...]], tuple] = {}

    # one head position ------------------------------------------------------------------------------------------------
    def _layer(self, g: torch.Tensor, tok: int, pos: int, k_hist: List[torch.Tensor], v_hist: List[torch.Tensor]):
        c = self.cfg
        e = self.embed[tok].to(self.dtype)
        x = torch.cat([rmsnorm(e, self.norm_e, c.rms_eps), rmsnorm(g, self.norm_g, c.rms_eps)])
        q = (self.wq @ x).reshape(1, c.n_heads, c.head_dim)
        k = (self.wk @ x).reshape(1, c.n_kv_heads, c.head_dim)
        v = (self.wv @ x).reshape(c.n_kv_heads, c.head_dim)
        cos, sin = rope_tables(torch.tensor([pos], device=self.device), c.head_dim, c.rope_theta)
        q = apply_rope(q, cos, sin)[0]
        k = apply_rope(k, cos, sin)[0]
        K = torch.stack(k_hist + [k], dim=1)                 # [n_kv, S, hd]
        V = torch.stack(v_hist + [v], dim=1)
        grp = c.n_heads // c.n_kv_heads
        qf = q.reshape(c.n_kv_heads, grp, c.head_dim).float()
        p = torch.softmax(torch.einsum("kgd,ksd->kgs", qf, K.float()) * c.head_dim ** -0.5, dim=-1)
        a = torch.einsum("kgs,ksd->kgd", p, V.float()).reshape(-1).to(self.dtype)
        h = g + self.wo @ a
        m = rmsnorm(h, self.norm_mlp, c.rms_eps)
        gu = self.w_gu @ m
        inter = gu.shape[0] // 2
        h = h + self.w_d @ (torch.nn.functional.silu(gu[:inter]) * gu[inter:])
        return h, k, v

    def _logits(self, h: torch.Tensor) -> torch.Tensor:
        return self.lm_head @ rmsnorm(h, self.norm_out, self.cfg.rms_eps)

    # candidate source -------------------------------------------------------------------------------------------------
    def _sync(self, context: Sequence[int]) -> bool:
        """Brings the committed head cache up to head position ``n - 2`` (``n = len(context)``); returns False when
        the target feature of that position is not known yet."""
        feats = self.runner.features if self.runner is not None else {}
        n = len(context)
        last = n - 2
        if last < 0 or last not in feats:
            return False
        # drop cache entries beyond what is still valid (context rolled back or diverged)
        if self._pos0 is not None:
            keep = 0
            while keep < len(self._k) and self._pos0 + keep <= last and self._tokens[keep] == context[self._pos0 + keep + 1]:
                keep += 1
            if keep < len(self._k):
                del self._k[keep:], self._v[keep:], self._tokens[keep:]
                for p in [p for p in self._hid if p >= self._pos0 + keep]:
                    del self._hid[p]
        nxt = (self._pos0 + len(self._k)) if self._pos0 is not None and self._k else None
        if nxt is None or any(p not in feats for p in range(nxt, last + 1)):
            first = last
            while first - 1 in feats and first - 1 >= 0:
                first -= 1
            self._k, self._v, self._tokens, self._hid = [], [], [], {}
            self._pos0, nxt = first, first
        for p in range(nxt, last + 1):
            g = self.fc @ feats[p].to(self.dtype)
            h, k, v = self._layer(g, context[p + 1], p, self._k, self._v)
            self._k.append(k)
            self._v.append(v)
            self._tokens.append(int(context[p + 1]))
            self._hid[p] = h
        return True

    @torch.no_grad()
    def candidates(self, context: Sequence[int], chain_so_far: Sequence[int], width: int) -> List[Candidate]:
        ctx = list(context)
        if self.runner is None or not self._sync(ctx):
            return []
        key = (len(ctx), tuple(int(t) for t in chain_so_far))
        if not chain_so_far:
            self._states = {k: s for k, s in self._states.items() if k[0] == len(ctx)}
            h, ks, vs = self._hid[len(ctx) - 2], [], []
        else:
            st = self._states.get(key)
            if st is None:
                parent = self._states.get((len(ctx), key[1][:-1])) if len(chain_so_far) > 1 else (self._hid[len(ctx) - 2], [], [])
                if parent is None:
                    return []
                ph, pks, pvs = parent
                pos = len(ctx) - 2 + len(chain_so_far)
                h, k, v = self._layer(ph, int(chain_so_far[-1]), pos, self._k + pks, self._v + pvs)
                st = (h, pks + [k], pvs + [v])
                self._states[key] = st
            h, ks, vs = st
        if not chain_so_far:
            self._states[key] = (h, ks, vs)
        logits = self._logits(h).float().cpu().numpy()
        toks, lps = N.draft_top_candidates(logits, width, self.d2t)
        experts = list(self.expert_fn(h)) if self.expert_fn is not None else []
        return [Candidate(t, lp, experts) for t, lp in zip(toks, lps)]

    # weights ----------------------------------------------------------------------------------------------------------
    def state_dict(self) -> Dict[str, torch.Tensor]:
        names = ["fc", "norm_e", "norm_g", "wq", "wk", "wv", "wo", "norm_mlp", "w_gu", "w_d", "norm_out", "lm_head"]
        sd = {n: getattr(self, n) for n in names}
        sd["d2t"] = torch.from_numpy(self.d2t)
        return sd

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        for n, t in sd.items():
            if n == "d2t":
                self.d2t = t.to(torch.int32).cpu().numpy()
            else:
                setattr(self, n, t.to(device=self.device, dtype=self.dtype))
        self._reset_cache()
