"""Speculative-decoding drivers: draft -> one verify pass of the target -> lossless acceptance (C++).

Two layers:
  * the generic round logic over abstract ``ModelRunner`` / ``DrafterPool`` / ``CandidateSource`` objects
    (``SpecEngine``: several chain drafters; ``Eagle3Engine``: route-aware chain with adaptive verify depth, token
    trees, full decode loop with degenerate-round fallback);
  * ``EngineRunner`` / ``SpecDriver``: the same rounds on a real :class:`InferenceEngine`, reusing its KV cache
    (a verify window is ONE forward over ``[last token, drafts...]``; rejected rows are rolled back).

Reference: engine/src/spec/{types,model,engine,eagle3_engine,route_aware,route_aware_drafter,telemetry}.rs. Unlike
the reference's multi-drafter path every round verifies k + 1 rows, so the bonus token of a fully accepted round
is a real target sample, never a greedy stand-in.
"""
from __future__ import annotations

import json
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import native as N
from .native import ExpertUnion, SpecTree


# ---- plain data -------------------------------------------------------------------------------------------------------------
@dataclass
class Candidate:
    token: int
    draft_logprob: float
    experts: List[int] = field(default_factory=list)


@dataclass
class DraftProposal:
    drafter_id: int
    tokens: List[int]
    logprobs: List[float]


@dataclass
class AcceptedRun:
    accepted: List[int]
    bonus_token: int
    winning_drafter: Optional[int] = None
    accept_mask: Optional[np.ndarray] = None

    def n_accepted(self) -> int:
        return len(self.accepted)

    def all_tokens(self) -> List[int]:
        return list(self.accepted) + [self.bonus_token]


@dataclass
class RoundStats:
    n_accepted: int = 0
    n_proposed: int = 0
    winning_drafter: Optional[int] = None


@dataclass
class Eagle3RoundStats:
    n_accepted: int = 0
    n_drafted: int = 0
    verify_depth: int = 0
    union_size: int = 0


@dataclass
class DecodeStop:
    max_new_tokens: int
    eos_token: Optional[int] = None


class Rng:
    """Uniform source for the acceptance tests; seeded the same on every rank so tensor-parallel ranks agree."""

    def __init__(self, seed: int = 0):
        self._g = np.random.default_rng(seed)

    def next_f32(self) -> float:
        return float(self._g.random())

    def uniforms(self, n: int) -> np.ndarray:
        return self._g.random(n).astype(np.float32)


class FixedRng(Rng):
    def __init__(self, value: float):
        self.value = value

    def next_f32(self) -> float:
        return self.value

    def uniforms(self, n: int) -> np.ndarray:
        return np.full(n, self.value, np.float32)


# ---- abstract model / drafter interfaces ---------------------------------------------------------------------------------------
class ModelRunner:
    """Target model seen by the round logic. ``forward_single(context, token)`` returns the logits after
    ``context + [token]``. ``forward_batch`` returns ``[k + 1, vocab]``: row ``i`` follows
    ``context + draft[:i]`` (so row ``i`` scores ``draft[i]`` and row ``k`` is the bonus row); the default runs
    position by position, a real engine overrides it with one window forward."""

    def vocab_size(self) -> int:
        raise NotImplementedError

    def forward_single(self, context: Sequence[int], token: int) -> np.ndarray:
        raise NotImplementedError

    def forward_batch(self, context: Sequence[int], draft: Sequence[int]) -> np.ndarray:
        ctx = list(context)
        rows = []
        for i in range(len(draft) + 1):
            full = ctx + list(draft[:i])
            rows.append(self.forward_single(full[:-1], full[-1]))
        return np.stack(rows)

    def forward_tree(self, context: Sequence[int], tree: SpecTree) -> np.ndarray:
        """``[n_nodes, vocab]``: row ``i`` follows ``context + path(i)``; the default walks every path."""
        ctx = list(context)
        rows = []
        for i in range(tree.n_nodes):
            full = ctx + tree.path(i)
            rows.append(self.forward_single(full[:-1], full[-1]))
        return np.stack(rows)


class DrafterPool:
    def n_drafters(self) -> int:
        raise NotImplementedError

    def draft(self, context: Sequence[int], k: int) -> List[DraftProposal]:
        raise NotImplementedError


class ChainDrafterPool(DrafterPool):
    """Wraps objects with ``propose(context, k) -> tokens`` (point-mass drafters such as the n-gram lookup)."""

    def __init__(self, drafters: Sequence):
        self.drafters = list(drafters)

    def n_drafters(self) -> int:
        return len(self.drafters)

    def draft(self, context, k):
        out = []
        for i, d in enumerate(self.drafters):
            toks = list(d.propose(context, k))
            out.append(DraftProposal(i, toks, [0.0] * len(toks)))
        return out


# ---- multi-drafter engine ------------------------------------------------------------------------------------------------------
@dataclass
class SpecConfig:
    draft_len: int = 8
    vocab_size: int = 151936
    temperature: float = 0.0


class SpecEngine:
    """One round: every drafter proposes a chain, the target verifies each chain (k + 1 rows), the multi-drafter
    rule picks the longest lossless prefix. Reference: engine/src/spec/engine.rs:10-97."""

    def __init__(self, target: ModelRunner, drafters: DrafterPool, config: SpecConfig = SpecConfig()):
        self.target, self.drafters, self.config = target, drafters, config

    def step(self, context: Sequence[int], rng: Rng) -> Tuple[AcceptedRun, RoundStats]:
        k = self.config.draft_len
        props = [p for p in self.drafters.draft(context, k) if p.tokens]
        if not props:
            ctx = list(context)
            row = self.target.forward_single(ctx[:-1], ctx[-1])
            tok = _sample_row(row, self.config.temperature, rng.next_f32())
            return AcceptedRun([], tok), RoundStats(0, 0, None)
        kk = min(len(p.tokens) for p in props)
        toks = np.array([p.tokens[:kk] for p in props], np.int32)
        lps = np.array([p.logprobs[:kk] for p in props], np.float32)
        rows = np.stack([self.target.forward_batch(context, p.tokens[:kk]) for p in props])
        r = N.accept_multi(rows, toks, lps, rng.uniforms(len(props) * kk + 1), self.config.temperature)
        winner = props[r.winner].drafter_id if r.winner >= 0 else None
        run = AcceptedRun(r.tokens[:-1], r.tokens[-1], winner, r.accept_mask)
        return run, RoundStats(r.n_accepted, kk, winner)

    def decode(self, prompt: Sequence[int], stop: DecodeStop, rng: Rng) -> Tuple[List[int], "SpecTelemetry"]:
        ctx, out, tel = list(prompt), [], SpecTelemetry()
        while len(out) < stop.max_new_tokens:
            run, st = self.step(ctx, rng)
            tel.record(Eagle3RoundStats(st.n_accepted, st.n_proposed, st.n_proposed, 0))
            if _emit(run.all_tokens(), out, ctx, stop):
                break
        return out, tel


def _sample_row(row: np.ndarray, temperature: float, u: float) -> int:
    if temperature <= 0:
        return int(np.argmax(row))
    z = (row - row.max()) / temperature
    p = np.exp(z)
    c = np.cumsum(p / p.sum())
    return int(min(np.searchsorted(c, u, side="right"), len(row) - 1))


def _emit(tokens: Sequence[int], out: List[int], ctx: List[int], stop: DecodeStop) -> bool:
    for t in tokens:
        if len(out) >= stop.max_new_tokens:
            return True
        out.append(int(t))
        ctx.append(int(t))
        if stop.eos_token is not None and t == stop.eos_token:
            return True
    return len(out) >= stop.max_new_tokens


# ---- route-aware drafting --------------------------------------------------------------------------------------------------------
class RouteAwarePolicy:
    """Scores a candidate by ``draft_logprob + lambda * |experts ∩ union|``: drafts whose experts the verify pass
    already reads cost no extra weight traffic. ``lambda = 0`` is plain highest-probability drafting.
    Reference: engine/src/spec/route_aware.rs:37-157."""

    def __init__(self, lam: float = 0.0):
        self.lam = lam

    def select_one(self, cands: Sequence[Candidate], union: ExpertUnion) -> Optional[int]:
        if not cands:
            return None
        i = N.route_aware_select([c.draft_logprob for c in cands], [c.experts for c in cands], union, self.lam)
        union.update(cands[i].experts)
        return i


class RouteAwareDrafter:
    """Greedy chain from a candidate source (``candidates(context, chain_so_far, width) -> [Candidate]``).
    Reference: engine/src/spec/route_aware_drafter.rs:28-101."""

    def __init__(self, source, lam: float = 0.0):
        self.source = source
        self.policy = RouteAwarePolicy(lam)

    def draft_chain(self, context, depth: int, width: int) -> Tuple[DraftProposal, ExpertUnion]:
        prop, _, union = self._chain(context, depth, width)
        return prop, union

    def _chain(self, context, depth, width):
        toks, lps, experts = [], [], []
        union = ExpertUnion()
        for _ in range(depth):
            cands = self.source.candidates(context, toks, width)
            i = self.policy.select_one(cands, union)
            if i is None:
                break
            toks.append(int(cands[i].token))
            lps.append(float(cands[i].draft_logprob))
            experts.append(list(cands[i].experts))
        return DraftProposal(0, toks, lps), experts, union

    def draft_and_plan(self, context, depth: int, width: int, floor_fraction: float):
        prop, experts, _ = self._chain(context, depth, width)
        if not prop.tokens:
            return prop, experts, None
        probs = [float(min(1.0, max(0.0, np.exp(lp)))) for lp in prop.logprobs]
        return prop, experts, N.adaptive_verify_depth(probs, experts, floor_fraction)


# ---- EAGLE-3 style engine --------------------------------------------------------------------------------------------------------
@dataclass
class Eagle3Config:
    depth: int = 5
    width: int = 4
    vocab_size: int = 151936
    floor_fraction: float = 0.86
    temperature: float = 0.0


class Eagle3Engine:
    """Chain rounds with adaptive verify truncation (``step``), token-tree rounds (``step_tree``) and the decode
    loop with a plain-decode fallback for rounds in which the head proposes nothing.
    Reference: engine/src/spec/eagle3_engine.rs:27-297."""

    def __init__(self, drafter: RouteAwareDrafter, target: ModelRunner, config: Eagle3Config = Eagle3Config()):
        self.drafter, self.target, self.config = drafter, target, config

    def step(self, context: Sequence[int], rng: Rng) -> Tuple[AcceptedRun, Eagle3RoundStats]:
        cfg = self.config
        prop, _experts, plan = self.drafter.draft_and_plan(context, cfg.depth, cfg.width, cfg.floor_fraction)
        n_drafted = len(prop.tokens)
        depth = plan.depth if plan is not None else n_drafted
        union = plan.union_size if plan is not None else 0
        toks, lps = prop.tokens[:depth], prop.logprobs[:depth]
        if not toks:
            return AcceptedRun([], 0), Eagle3RoundStats(0, n_drafted, 0, union)
        rows = self.target.forward_batch(context, toks)            # depth + 1 rows: the last is the bonus row
        emitted, nacc = N.accept_chain(rows, toks, lps, rng.uniforms(depth + 1), cfg.temperature)
        return AcceptedRun(emitted[:-1], emitted[-1], 0), Eagle3RoundStats(nacc, n_drafted, depth, union)

    def step_tree(self, context: Sequence[int], depth: int, branch: int, rng: Rng, max_nodes: Optional[int] = None):
        ctx = list(context)
        root = ctx[-1] if ctx else 0

        def source(prefix, b):
            return [(c.token, c.draft_logprob) for c in self.drafter.source.candidates(ctx, prefix[len(ctx):], b)]

        tree = SpecTree.build_from_source(source, ctx, root, depth, branch, max_nodes)
        n_drafted = tree.n_nodes - 1
        if n_drafted == 0:
            return AcceptedRun([], self._fallback(ctx)), Eagle3RoundStats(0, 0, 0, 0)
        rows = self.target.forward_tree(ctx, tree)
        emitted, nodes = N.accept_tree(tree, rows, rng.uniforms(2 * tree.n_nodes + 2), self.config.temperature)
        return AcceptedRun(emitted[:-1], emitted[-1], 0), Eagle3RoundStats(len(nodes), n_drafted, len(nodes), n_drafted)

    def _fallback(self, ctx: List[int]) -> int:
        if not ctx:
            return 0
        return int(np.argmax(self.target.forward_single(ctx[:-1], ctx[-1])))

    def decode(self, prompt: Sequence[int], stop: DecodeStop, rng: Rng, tree: Optional[Tuple[int, int]] = None):
        ctx, out, tel = list(prompt), [], SpecTelemetry()
        while len(out) < stop.max_new_tokens:
            run, st = self.step_tree(ctx, tree[0], tree[1], rng) if tree else self.step(ctx, rng)
            tel.record(st)
            toks = run.all_tokens() if (st.n_drafted > 0 or tree) else [self._fallback(ctx)]
            if _emit(toks, out, ctx, stop):
                break
        return out, tel


# ---- telemetry -----------------------------------------------------------------------------------------------------------------
class SpecTelemetry:
    """Running acceptance statistics. ``mean_accept_length`` = accepted per round + 1 (the bonus token); union and
    depth average over rounds that drafted something. Reference: engine/src/spec/telemetry.rs:21-157."""

    def __init__(self):
        self.rounds = self.spec_rounds = 0
        self.total_accepted = self.total_drafted = self.total_verify_depth = self.total_union = 0

    def record(self, s: Eagle3RoundStats) -> None:
        self.rounds += 1
        self.total_accepted += s.n_accepted
        if s.n_drafted > 0:
            self.spec_rounds += 1
            self.total_drafted += s.n_drafted
            self.total_verify_depth += s.verify_depth
            self.total_union += s.union_size

    def mean_accept_length(self) -> float:
        return self.total_accepted / self.rounds + 1.0 if self.rounds else 0.0

    def mean_union(self) -> float:
        return self.total_union / self.spec_rounds if self.spec_rounds else 0.0

    def mean_verify_depth(self) -> float:
        return self.total_verify_depth / self.spec_rounds if self.spec_rounds else 0.0

    def acceptance_rate(self) -> float:
        return self.total_accepted / self.total_drafted if self.total_drafted else 0.0

    def snapshot(self) -> Dict:
        return {"rounds": self.rounds, "spec_rounds": self.spec_rounds,
                "mean_accept_length": self.mean_accept_length(), "mean_union": self.mean_union(),
                "mean_verify_depth": self.mean_verify_depth(), "acceptance_rate": self.acceptance_rate()}

    def to_sse_frame(self) -> str:
        return "data: " + json.dumps(self.snapshot()) + "\n\n"

    def projected_speedup(self, head_eager_cost: float, draft_graph_cost: float, depth: int, floor_fraction: float,
                          graphs: bool) -> float:
        if self.spec_rounds == 0:
            return 0.0
        first = min(0.99, max(0.05, self.acceptance_rate()))
        union = max(8, int(round(self.mean_union())))
        return N.predict_speedup(self.mean_accept_length(), first, depth, union, floor_fraction, head_eager_cost,
                                 draft_graph_cost, graphs)


# ---- a real engine behind the interfaces ---------------------------------------------------------------------------------------------
class EngineRunner(ModelRunner):
    """``ModelRunner`` over an :class:`InferenceEngine`. The interface is stateless (the context is passed every
    time) but the KV cache is reused: the runner remembers which tokens the cache holds, rolls back to the longest
    common prefix and feeds only what is missing, in the same window forward as the draft tokens."""

    def __init__(self, engine, aux_layers: Sequence[int] = ()):
        self.engine = engine
        self.aux_layers = tuple(aux_layers)
        self.kv: List[int] = []
        self.features: Dict[int, "object"] = {}      # absolute position -> concatenated aux hidden states
        self.forwards = 0
        self.seconds = 0.0
        engine.reset()

    def vocab_size(self) -> int:
        return self.engine.cfg.model.vocab

    def reset(self) -> None:
        self.engine.reset()
        self.kv = []
        self.features = {}

    def adopt(self, tokens: Sequence[int]) -> None:
        """Declare that the engine's cache already holds ``tokens`` (after an external prefill)."""
        self.kv = list(tokens)

    def _sync(self, need: List[int]) -> List[int]:
        lcp = 0
        m = min(len(self.kv), len(need))
        while lcp < m and self.kv[lcp] == need[lcp]:
            lcp += 1
        if lcp < len(self.kv):
            self.engine.rollback(lcp)
            self.kv = self.kv[:lcp]
            for p in [p for p in self.features if p >= lcp]:
                del self.features[p]
        return need[lcp:]

    def _forward(self, window: List[int], commit: bool, **kw):
        t0 = time.perf_counter()
        start = len(self.kv)
        logits = self.engine.logits_for(window, commit=commit, aux_layers=self.aux_layers, **kw)
        self.forwards += 1
        self.seconds += time.perf_counter() - t0
        taps = getattr(self.engine.model, "aux_taps", None) if self.aux_layers else None
        if taps and commit:
            import torch
            feat = torch.cat([taps[L] for L in self.aux_layers], dim=-1)
            for i in range(len(window)):
                self.features[start + i] = feat[i]
        if commit:
            self.kv += window
        return logits.float().cpu().numpy()

    def forward_single(self, context, token):
        return self.forward_batch(list(context) + [int(token)], [])[0]

    def forward_batch(self, context, draft):
        ctx = list(context)
        pending = self._sync(ctx[:-1])
        window = pending + [ctx[-1]] + [int(t) for t in draft]
        rows = self._forward(window, commit=True)
        return rows[len(pending):]

    def forward_tree(self, context, tree: SpecTree):
        import torch
        ctx = list(context)
        pending = self._sync(ctx[:-1])
        if pending:
            self._forward(pending, commit=True)
        base = len(self.kv)
        n = tree.n_nodes
        tokens = [ctx[-1]] + [int(t) for t in tree.tokens[1:]]
        dev = self.engine.device
        positions = torch.tensor([base + tree.depth(i) for i in range(n)], device=dev)
        mask = torch.zeros(n, n, dtype=torch.bool, device=dev)
        mask[:, 0] = True
        if n > 1:
            mask[1:, 1:] = torch.from_numpy(N.tree_mask(tree.parent)).to(dev)
        return self._forward(tokens, commit=False, tree_mask=mask, positions=positions)


@dataclass
class SpecRound:
    tokens: List[int]
    n_proposed: int
    n_accepted: int
    seconds: float
    routes: list


class SpecDriver:
    """Stateful speculative decoding on one engine, the hook the serving backend calls once per round:
    ``begin(prompt_tokens)`` after the prompt was prefilled, then ``step(last_token)`` returns the tokens of one
    round. ``mode``: ``"chain"`` (adaptive depth) or ``"tree"`` (``tree=(depth, branch)`` or
    ``(depth, branch, max_candidates)``)."""

    def __init__(self, engine, source, *, depth: int = 5, width: int = 4, lam: float = 0.0,
                 floor_fraction: float = 0.86, tree: Optional[Tuple[int, int]] = None, seed: int = 0,
                 aux_layers: Sequence[int] = (), temperature: float = 0.0):
        self.engine = engine
        self.runner = EngineRunner.__new__(EngineRunner)
        self.runner.engine, self.runner.aux_layers = engine, tuple(aux_layers)
        self.runner.kv, self.runner.features, self.runner.forwards, self.runner.seconds = [], {}, 0, 0.0
        cfg = Eagle3Config(depth, width, engine.cfg.model.vocab, floor_fraction, temperature)
        self.eagle = Eagle3Engine(RouteAwareDrafter(source, lam), self.runner, cfg)
        self.tree = tree
        self.rng = Rng(seed)
        self.context: List[int] = []
        self.telemetry = SpecTelemetry()
        self._last: Optional[int] = None
        if hasattr(source, "bind"):
            source.bind(self.runner)

    def begin(self, prompt_tokens: Sequence[int]) -> None:
        self.context = [int(t) for t in prompt_tokens]
        self.runner.adopt(self.context)
        self.runner.features = {}
        self.telemetry = SpecTelemetry()
        self._last = None

    def step(self, token: int) -> SpecRound:
        t0 = time.perf_counter()
        if self._last is None or token != self._last:       # the first token after the prompt comes from outside
            self.context.append(int(token))
        ctx = self.context
        if self.tree:
            run, st = self.eagle.step_tree(ctx, self.tree[0], self.tree[1], self.rng,
                                           self.tree[2] if len(self.tree) > 2 else None)
        else:
            run, st = self.eagle.step(ctx, self.rng)
        toks = run.all_tokens() if (st.n_drafted > 0 or self.tree) else [self.eagle._fallback(ctx)]
        self.telemetry.record(st)
        self.context = ctx + toks
        self._last = toks[-1]
        routes = list(getattr(self.engine.model, "last_routes", [])) if self.engine.gpu is None else []
        return SpecRound(toks, st.n_drafted, st.n_accepted, time.perf_counter() - t0, routes)

    def generate(self, prompt: Sequence[int], max_new_tokens: int, eos: Optional[int] = None) -> List[int]:
        """Prefill + speculative rounds; returns the generated tokens (the same sequence plain greedy decoding
        produces when ``temperature = 0``)."""
        self.engine.reset()
        pre = self.engine.prefill(list(prompt))
        self.begin(prompt)
        out = [pre.next_token]
        while len(out) < max_new_tokens and (eos is None or out[-1] != eos):
            rnd = self.step(out[-1])
            for t in rnd.tokens:
                if len(out) >= max_new_tokens:
                    break
                out.append(t)
                if eos is not None and t == eos:
                    break
        return out
