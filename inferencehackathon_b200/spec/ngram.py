"""Prompt-lookup n-gram drafter and its acceptance-length (tau) evaluation.

The drafter needs no model: it looks for the most recent earlier occurrence of the last ``n`` tokens and proposes
the ``k`` tokens that followed it. Reference: kernels/ngram_drafter_tau.py:37-98 (drafter + greedy tau over token
streams), kernels/make_corpora.py (token streams; here synthetic generators, there is no tokenizer download).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np


class NGramDrafter:
    """``propose(context, k)`` -> up to ``k`` tokens following the latest earlier match of the last ``n`` tokens;
    falls back to shorter n-grams down to ``min_n``. An incremental index (n-gram -> last end position) keeps a
    round O(k) instead of rescanning the context."""

    def __init__(self, n: int = 2, min_n: int = 1):
        assert n >= min_n >= 1
        self.n, self.min_n = n, min_n
        self._ctx: List[int] = []
        self._index: List[Dict[Tuple[int, ...], List[int]]] = [dict() for _ in range(n + 1)]

    def reset(self) -> None:
        self._ctx = []
        self._index = [dict() for _ in range(self.n + 1)]

    def _sync(self, context: Sequence[int]) -> None:
        c = self._ctx
        m = min(len(c), len(context))
        same = m
        for i in range(m):
            if c[i] != context[i]:
                same = i
                break
        if same < len(c):                      # context was rolled back: rebuild (rare)
            self.reset()
            c = self._ctx
            same = 0
        for i in range(same, len(context)):
            c.append(int(context[i]))
            end = len(c)                       # n-grams ending at position `end`
            for g in range(self.min_n, self.n + 1):
                if end >= g:
                    self._index[g].setdefault(tuple(c[end - g:end]), []).append(end)

    def propose(self, context: Sequence[int], k: int) -> List[int]:
        self._sync(context)
        c = self._ctx
        L = len(c)
        for g in range(min(self.n, L), self.min_n - 1, -1):
            ends = self._index[g].get(tuple(c[L - g:]))
            if not ends:
                continue
            # most recent occurrence that ends before the current suffix and has something after it
            for end in reversed(ends):
                if end < L:
                    return c[end:end + k]
        return []

    # candidate-source interface of the tree / route-aware drivers: a point-mass proposal
    def candidates(self, context: Sequence[int], chain_so_far: Sequence[int], width: int):
        from .driver import Candidate
        prop = self.propose(list(context) + list(chain_so_far), 1)
        return [Candidate(prop[0], 0.0, [])] if prop else []


@dataclass
class TauResult:
    k: int
    n: int
    tau: float
    rounds: int
    tokens: int


def ngram_tau(stream: Sequence[int], k: int, n: int, prompt_len: int = 64) -> TauResult:
    """Mean emitted tokens per round when the stream itself is the greedy target: each round accepts the longest
    matching prefix of the proposal plus one bonus token."""
    d = NGramDrafter(n)
    pos = min(prompt_len, len(stream))
    rounds = 0
    start = pos
    while pos < len(stream):
        prop = d.propose(stream[:pos], k)
        acc = 0
        while acc < len(prop) and pos + acc < len(stream) and prop[acc] == stream[pos + acc]:
            acc += 1
        pos += acc + 1
        rounds += 1
    emitted = min(pos, len(stream)) - start
    return TauResult(k, n, emitted / max(rounds, 1), rounds, emitted)


# ---- synthetic token streams ------------------------------------------------------------------------------------------------
def repeated_block_stream(block: int = 64, repeats: int = 16, vocab: int = 151936, seed: int = 0) -> List[int]:
    """A random block repeated: the best case of prompt lookup (every continuation was seen before)."""
    rng = np.random.default_rng(seed)
    return (rng.integers(0, vocab, block).tolist()) * repeats


def zipf_markov_stream(length: int = 4096, vocab: int = 4096, order_mix: float = 0.7, seed: int = 0) -> List[int]:
    """Text-like stream: with probability ``order_mix`` the next token is a fixed function of the previous one
    (a bigram habit), otherwise a Zipf draw. Gives tau between the random and the repeated extremes."""
    rng = np.random.default_rng(seed)
    habit = rng.integers(0, vocab, vocab)
    ranks = np.arange(1, vocab + 1, dtype=np.float64)
    pz = (1.0 / ranks) / (1.0 / ranks).sum()
    out = [int(rng.integers(0, vocab))]
    draws = rng.choice(vocab, size=length, p=pz)
    coin = rng.random(length)
    for i in range(1, length):
        out.append(int(habit[out[-1]]) if coin[i] < order_mix else int(draws[i]))
    return out


def main(argv: Optional[Sequence[str]] = None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description="n-gram drafter tau over synthetic token streams")
    ap.add_argument("--k", type=int, nargs="+", default=[3, 8, 16])
    ap.add_argument("--n", type=int, nargs="+", default=[1, 2, 3])
    ap.add_argument("--stream", choices=["repeat", "markov"], default="markov")
    ap.add_argument("--length", type=int, default=4096)
    a = ap.parse_args(argv)
    s = repeated_block_stream(64, max(2, a.length // 64)) if a.stream == "repeat" else zipf_markov_stream(a.length)
    for k in a.k:
        for n in a.n:
            r = ngram_tau(s, k, n)
            print(f"NGRAM_TAU_RESULT k={r.k} n={r.n} tau={r.tau:.3f} rounds={r.rounds}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
