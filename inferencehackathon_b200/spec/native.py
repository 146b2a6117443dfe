"""ctypes bindings of the speculative-decoding control plane (``libihb_ctrl.so``, ``csrc/ctrl/spec.cpp``).

Thin, array-in / array-out wrappers: numpy arrays cross the boundary, results come back as Python ints / lists.
Reference counterparts: engine/native/spec_accept.h, spec_accept_tree.h, tree_attn.h, draft_vocab.h,
sdpa_tree_ref.h and engine/src/spec/{accept,tree,tree_shape,adaptive_verify,projection,route_aware}.rs.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np

from ..ops import build as _build

_lib = None


def lib() -> C.CDLL:
    """Loads (building if stale) the control-plane library."""
    global _lib
    if _lib is None:
        path = os.environ.get("IHB_CTRL_LIB") or _build.build_ctrl()      # override: a sanitizer build of the library
        _lib = C.CDLL(path)
        _declare(_lib)
    return _lib


_f = C.POINTER(C.c_float)
_i = C.POINTER(C.c_int)
_u8 = C.POINTER(C.c_ubyte)
VERIFY_FN = C.CFUNCTYPE(None, C.c_void_p, _i, C.c_int, _f)


def _declare(L: C.CDLL) -> None:
    L.ihb_spec_accept.restype = C.c_int
    L.ihb_spec_accept.argtypes = [_f, C.c_int, C.c_int, _i, _f, _f, C.c_float, _i, _i]
    L.ihb_spec_accept_full.restype = C.c_int
    L.ihb_spec_accept_full.argtypes = [_f, C.c_int, C.c_int, _i, _f, _f, C.c_float, _i, _i]
    L.ihb_spec_accept_multi.restype = C.c_int
    L.ihb_spec_accept_multi.argtypes = [_f, C.c_int, C.c_int, C.c_int, _i, _f, _f, C.c_float, _i, _i, _i, _u8]
    L.ihb_spec_accept_tree.restype = C.c_int
    L.ihb_spec_accept_tree.argtypes = [C.c_int, _i, _i, _f, _f, C.c_int, _f, C.c_int, C.c_float, _i, _i, _i]
    L.ihb_tree_attn_build.restype = C.c_int
    L.ihb_tree_attn_build.argtypes = [C.c_int, _i, C.c_int, _i, _i, _i]
    L.ihb_tree_mask.restype = None
    L.ihb_tree_mask.argtypes = [C.c_int, _i, _u8]
    L.ihb_draft_top_candidates.restype = C.c_int
    L.ihb_draft_top_candidates.argtypes = [_i, _f, C.c_int, C.c_int, _i, _f]
    L.ihb_sdpa_tree_ref.restype = None
    L.ihb_sdpa_tree_ref.argtypes = [C.c_int, _i, C.c_int, C.c_int, C.c_int, C.c_int, _f, _f, _f, _f, _f, _f, _f,
                                    C.c_float, C.c_float, _f]
    L.ihb_spec_round.restype = C.c_int
    L.ihb_spec_round.argtypes = [_i, _f, C.c_int, C.c_int, C.c_int, VERIFY_FN, C.c_void_p, _f, C.c_float, _i, _i]
    L.ihb_verify_cost.restype = C.c_float
    L.ihb_verify_cost.argtypes = [C.c_uint, C.c_float, C.c_float]
    L.ihb_adaptive_verify_depth.restype = C.c_int
    L.ihb_adaptive_verify_depth.argtypes = [_f, C.c_int, _i, _i, C.c_float, C.c_float, _f, C.POINTER(C.c_uint), _f, _f]
    L.ihb_level_advance_prob.restype = C.c_float
    L.ihb_level_advance_prob.argtypes = [C.c_float, C.c_int]
    L.ihb_tree_expected_accepted.restype = C.c_float
    L.ihb_tree_expected_accepted.argtypes = [C.c_float, C.c_float, C.c_int, C.c_int]
    L.ihb_tree_nodes.restype = C.c_ulonglong
    L.ihb_tree_nodes.argtypes = [C.c_int, C.c_int]
    L.ihb_persistence.restype = C.c_float
    L.ihb_persistence.argtypes = [C.c_float, C.c_float, C.c_int]
    L.ihb_tree_shape_optimal.restype = C.c_float
    L.ihb_tree_shape_optimal.argtypes = [C.c_float, C.c_float, C.c_float, C.c_float, C.c_ulonglong, C.c_int, C.c_int,
                                         _i, _i, _f]
    L.ihb_predict_speedup.restype = C.c_float
    L.ihb_predict_speedup.argtypes = [C.c_float, C.c_float, C.c_int, C.c_uint, C.c_float, C.c_float, C.c_float, C.c_int]
    L.ihb_route_aware_select.restype = C.c_int
    L.ihb_route_aware_select.argtypes = [C.c_int, _f, _i, _i, _u8, C.c_float]


def _fa(x) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float32)


def _ia(x) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.int32)


def _pf(a: np.ndarray):
    return a.ctypes.data_as(_f)


def _pi(a: np.ndarray):
    return a.ctypes.data_as(_i)


# ---- acceptance ---------------------------------------------------------------------------------------------------------
def accept_chain(target_logits, draft_tokens, draft_logprobs, rng_u, temperature: float = 1.0) -> Tuple[List[int], int]:
    """Lossless chain acceptance. ``target_logits`` is ``[k + 1, vocab]``: row ``pos`` scores ``draft_tokens[pos]``
    (row 0 follows the last committed token) and row ``k`` is the real bonus distribution. Returns
    ``(emitted tokens, n_accepted)``; ``len(emitted) == n_accepted + 1``. ``temperature <= 0`` is greedy."""
    tl = _fa(target_logits)
    k = len(draft_tokens)
    assert tl.shape[0] == k + 1, "verify k + 1 rows: the last one is the bonus distribution"
    u = _fa(rng_u)
    assert u.size >= k + 1
    toks, lps = _ia(draft_tokens), _fa(draft_logprobs)
    out = np.zeros(k + 1, np.int32)
    nacc = C.c_int(0)
    n = lib().ihb_spec_accept(_pf(tl), tl.shape[1], k, _pi(toks), _pf(lps), _pf(u), temperature, _pi(out), C.byref(nacc))
    return out[:n].tolist(), nacc.value


def accept_chain_full(target_logits, draft_tokens, draft_probs, rng_u, temperature: float = 1.0) -> Tuple[List[int], int]:
    """Chain acceptance with the drafter's full per-position distributions ``draft_probs [k, vocab]``: the residual
    is ``max(0, p - q)`` over the whole vocabulary, exactly lossless for a sampling drafter. (``accept_chain`` knows
    only the drafted token's probability, as the reference does, and is exact for greedy targets and for
    deterministic drafters passed with log-probability 0.)"""
    tl, q = _fa(target_logits), _fa(draft_probs)
    k = len(draft_tokens)
    assert tl.shape[0] == k + 1 and q.shape == (k, tl.shape[1])
    u = _fa(rng_u)
    toks = _ia(draft_tokens)
    out = np.zeros(k + 1, np.int32)
    nacc = C.c_int(0)
    n = lib().ihb_spec_accept_full(_pf(tl), tl.shape[1], k, _pi(toks), _pf(q), _pf(u), temperature, _pi(out), C.byref(nacc))
    return out[:n].tolist(), nacc.value


@dataclass
class MultiAccept:
    tokens: List[int]
    n_accepted: int
    winner: int
    accept_mask: np.ndarray          # [n_drafters, k] which drafter's token was taken at each position


def accept_multi(target_logits, draft_tokens, draft_logprobs, rng_u, temperature: float = 1.0) -> MultiAccept:
    """``target_logits`` ``[n, k + 1, vocab]``, ``draft_tokens`` / ``draft_logprobs`` ``[n, k]``; ``rng_u`` needs
    ``n * k + 1`` uniforms."""
    tl = _fa(target_logits)
    toks, lps = _ia(draft_tokens), _fa(draft_logprobs)
    n, k = toks.shape
    assert tl.shape[:2] == (n, k + 1)
    u = _fa(rng_u)
    assert u.size >= n * k + 1
    out = np.zeros(k + 1, np.int32)
    mask = np.zeros((n, k), np.uint8)
    nacc, win = C.c_int(0), C.c_int(-1)
    m = lib().ihb_spec_accept_multi(_pf(tl), tl.shape[2], n, k, _pi(toks), _pf(lps), _pf(u), temperature, _pi(out),
                                    C.byref(nacc), C.byref(win), mask.ctypes.data_as(_u8))
    return MultiAccept(out[:m].tolist(), nacc.value, win.value, mask.astype(bool))


@dataclass
class SpecTree:
    """Token tree for one verify pass: node 0 is the root sentinel (the last committed token, ``parent[0] = 0``).
    Reference: engine/src/spec/tree.rs:29-86."""
    tokens: List[int]
    parent: List[int]
    draft_logprob: List[float]

    @property
    def n_nodes(self) -> int:
        return len(self.tokens)

    @classmethod
    def root(cls, token: int) -> "SpecTree":
        return cls([int(token)], [0], [0.0])

    def add(self, parent: int, token: int, logprob: float) -> int:
        self.tokens.append(int(token))
        self.parent.append(int(parent))
        self.draft_logprob.append(float(logprob))
        return len(self.tokens) - 1

    @classmethod
    def chain(cls, root_token: int, tokens: Sequence[int], logprobs: Sequence[float]) -> "SpecTree":
        t = cls.root(root_token)
        p = 0
        for tok, lp in zip(tokens, logprobs):
            p = t.add(p, tok, lp)
        return t

    @classmethod
    def build_from_source(cls, source, ctx: Sequence[int], root_token: int, depth: int, branch: int,
                          max_nodes: Optional[int] = None) -> "SpecTree":
        """Breadth-first expansion: ``source(prefix_tokens, branch)`` returns ``[(token, logprob), ...]`` for the
        continuation of ``ctx + path``. With ``max_nodes`` the tree is a beam: every level keeps only its
        ``max_nodes // depth`` best children by cumulative log-probability (e.g. 4 levels x 4 = 16 candidates)."""
        t = cls.root(root_token)
        frontier = [(0, 0.0)]
        keep = max(1, max_nodes // max(1, depth)) if max_nodes else None
        for _ in range(depth):
            cand = []
            for node, cum in frontier:
                for tok, lp in source(list(ctx) + t.path(node), branch):
                    cand.append((cum + float(lp), node, tok, lp))
            if keep is not None and len(cand) > keep:
                cand = sorted(cand, key=lambda c: -c[0])[:keep]
                cand.sort(key=lambda c: c[1])                      # children of one parent stay together
            frontier = [(t.add(node, tok, lp), cum) for cum, node, tok, lp in cand]
            if not frontier:
                break
        return t

    def path(self, node: int) -> List[int]:
        out = []
        while node != 0:
            out.append(self.tokens[node])
            node = self.parent[node]
        return out[::-1]

    def depth(self, node: int) -> int:
        d = 0
        while node != 0:
            node = self.parent[node]
            d += 1
        return d

    def children(self, node: int) -> List[int]:
        return [i for i in range(1, self.n_nodes) if self.parent[i] == node]


def accept_tree(tree: SpecTree, target_rows, rng_u, temperature: float = 1.0) -> Tuple[List[int], List[int]]:
    """SpecInfer-style lossless tree walk. ``target_rows[i]`` is the target's logits after node ``i``'s token.
    Returns ``(emitted tokens, accepted node ids)``; the last emitted token is the correction / bonus."""
    rows = _fa(target_rows)
    assert rows.shape[0] == tree.n_nodes
    u = _fa(rng_u)
    toks, par, lps = _ia(tree.tokens), _ia(tree.parent), _fa(tree.draft_logprob)
    out = np.zeros(tree.n_nodes + 1, np.int32)
    nodes = np.zeros(tree.n_nodes + 1, np.int32)
    nacc = C.c_int(0)
    n = lib().ihb_spec_accept_tree(tree.n_nodes, _pi(toks), _pi(par), _pf(lps), _pf(rows), rows.shape[1], _pf(u), u.size,
                                   temperature, _pi(out), _pi(nodes), C.byref(nacc))
    return out[:n].tolist(), nodes[:nacc.value].tolist()


def tree_attn_build(parent: Sequence[int], context_len: int) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """RoPE position per node (``ctx + depth - 1``) and CSR ancestor KV slots (root side first, self last; node
    ``i > 0`` lives in slot ``ctx + i - 1``). Reference: engine/native/tree_attn.h:25-63."""
    par = _ia(parent)
    n = par.size
    pos = np.zeros(n, np.int32)
    off = np.zeros(n + 1, np.int32)
    slots = np.zeros(n * n + 1, np.int32)
    w = lib().ihb_tree_attn_build(n, _pi(par), context_len, _pi(pos), _pi(off), _pi(slots))
    return pos, off, slots[:w].copy()


def tree_mask(parent: Sequence[int]) -> np.ndarray:
    """``[n - 1, n - 1]`` boolean visibility among draft nodes (query row ``i`` = node ``i + 1``)."""
    par = _ia(parent)
    n = par.size
    m = np.zeros((max(n - 1, 0), max(n - 1, 0)), np.uint8)
    if n > 1:
        lib().ihb_tree_mask(n, _pi(par), m.ctypes.data_as(_u8))
    return m.astype(bool)


def draft_top_candidates(draft_logits, m: int, d2t=None) -> Tuple[List[int], List[float]]:
    """Top-``m`` draft candidates as target-vocabulary ids with log-probabilities in the DRAFT vocabulary space
    (the acceptance ratio needs the drafter's own distribution). Reference: engine/native/draft_vocab.h:30-58."""
    dl = _fa(draft_logits).reshape(-1)
    mm = min(m, dl.size)
    toks = np.zeros(mm, np.int32)
    lps = np.zeros(mm, np.float32)
    map_ = _ia(d2t) if d2t is not None else None
    lib().ihb_draft_top_candidates(_pi(map_) if map_ is not None else None, _pf(dl), dl.size, mm, _pi(toks), _pf(lps))
    return toks.tolist(), lps.tolist()


def sdpa_tree_ref(parent, context_len, q, k_ctx, v_ctx, k_draft, v_draft, q_gamma, k_gamma, eps=1e-6, theta=1e6):
    """fp32 CPU oracle of tree-masked GQA attention (per-head RMSNorm + NeoX RoPE on q and the draft K rows).
    Shapes: q ``[n, n_q, hd]``, k_ctx / v_ctx ``[n_kv, ctx, hd]`` (already normed + roped), k_draft / v_draft
    ``[n, n_kv, hd]`` raw. Returns ``[n, n_q, hd]`` (row 0, the root, stays zero)."""
    par = _ia(parent)
    q, k_ctx, v_ctx, k_draft, v_draft = map(_fa, (q, k_ctx, v_ctx, k_draft, v_draft))
    qg, kg = _fa(q_gamma), _fa(k_gamma)
    n, n_q, hd = q.shape
    n_kv = k_draft.shape[1]
    out = np.zeros_like(q)
    lib().ihb_sdpa_tree_ref(n, _pi(par), context_len, n_q, n_kv, hd, _pf(q), _pf(k_ctx), _pf(v_ctx), _pf(k_draft),
                            _pf(v_draft), _pf(qg), _pf(kg), eps, theta, _pf(out))
    return out


def spec_round(draft_logits, vocab: int, verify, rng_u, d2t=None, temperature: float = 1.0) -> Tuple[List[int], int]:
    """One chain round on the host: greedy draft candidates from ``draft_logits [k, draft_vocab]`` ->
    ``verify(tokens) -> [k + 1, vocab]`` -> acceptance. Reference: engine/native/spec_round_ref.c:32-49."""
    dl = _fa(draft_logits)
    k, dv = dl.shape
    u = _fa(rng_u)

    def _cb(_ctx, toks_p, kk, rows_p):
        toks = [toks_p[i] for i in range(kk)]
        rows = _fa(verify(toks)).reshape(-1)
        C.memmove(rows_p, rows.ctypes.data, rows.nbytes)

    cb = VERIFY_FN(_cb)
    out = np.zeros(k + 1, np.int32)
    nacc = C.c_int(0)
    map_ = _ia(d2t) if d2t is not None else None
    n = lib().ihb_spec_round(_pi(map_) if map_ is not None else None, _pf(dl), dv, k, vocab, cb, None, _pf(u),
                             temperature, _pi(out), C.byref(nacc))
    return out[:n].tolist(), nacc.value


# ---- cost models --------------------------------------------------------------------------------------------------------
def verify_cost(union_size: int, floor_fraction: float = 0.86, top_k: float = 8.0) -> float:
    """Cost of a verify pass relative to one plain decode step: the floor part does not grow with the expert
    union, the rest scales as ``0.34 + 0.66 * union / top_k``. Reference: engine/src/spec/adaptive_verify.rs:23-40."""
    return float(lib().ihb_verify_cost(int(union_size), floor_fraction, top_k))


@dataclass
class VerifyPlan:
    depth: int
    emitted: float
    union_size: int
    cost: float
    value: float


def adaptive_verify_depth(accept_probs: Sequence[float], experts_per_pos: Sequence[Sequence[int]],
                          floor_fraction: float = 0.86, top_k: float = 8.0) -> VerifyPlan:
    """Depth that maximises expected emitted tokens per unit verify cost; ties keep the shallower depth."""
    k = len(accept_probs)
    off = np.zeros(k + 1, np.int32)
    ids: List[int] = []
    for i in range(k):
        ids.extend(experts_per_pos[i] if i < len(experts_per_pos) else [])
        off[i + 1] = len(ids)
    ida = _ia(ids if ids else [0])
    em, cost, val, uni = C.c_float(0), C.c_float(0), C.c_float(0), C.c_uint(0)
    d = lib().ihb_adaptive_verify_depth(_pf(_fa(accept_probs)), k, _pi(off), _pi(ida), floor_fraction, top_k,
                                        C.byref(em), C.byref(uni), C.byref(cost), C.byref(val))
    return VerifyPlan(d, em.value, uni.value, cost.value, val.value)


def level_advance_prob(p: float, branch: int) -> float:
    return float(lib().ihb_level_advance_prob(p, branch))


def tree_expected_accepted(first_pos: float, p: float, branch: int, depth: int) -> float:
    return float(lib().ihb_tree_expected_accepted(first_pos, p, branch, depth))


def tree_nodes(branch: int, depth: int) -> int:
    return int(lib().ihb_tree_nodes(branch, depth))


def persistence(mean_accept_len: float, first_pos: float, depth: int) -> float:
    """Per-position continuation probability reproducing a measured mean accept length (emitted tokens per
    round, bonus included). Reference: engine/src/spec/projection.rs:29-70."""
    return float(lib().ihb_persistence(mean_accept_len, first_pos, depth))


@dataclass
class TreeShape:
    branch: int
    depth: int
    emitted: float
    speedup: float


def tree_shape_optimal(mean_accept_len: float, first_pos: float, verify_flat_cost: float = 1.0,
                       head_level_cost: float = 0.05, node_budget: int = 64, max_branch: int = 8,
                       max_depth: int = 8) -> TreeShape:
    b, d, em = C.c_int(1), C.c_int(1), C.c_float(0)
    sp = lib().ihb_tree_shape_optimal(mean_accept_len, first_pos, verify_flat_cost, head_level_cost, node_budget,
                                      max_branch, max_depth, C.byref(b), C.byref(d), C.byref(em))
    return TreeShape(b.value, d.value, em.value, float(sp))


def predict_speedup(mean_accept_len: float, first_pos: float, depth: int, union_size: int,
                    floor_fraction: float = 0.86, head_eager_cost: float = 0.1, draft_graph_cost: float = 0.1,
                    graphs: bool = False) -> float:
    return float(lib().ihb_predict_speedup(mean_accept_len, first_pos, depth, union_size, floor_fraction,
                                           head_eager_cost, draft_graph_cost, int(graphs)))


class ExpertUnion:
    """Bit set of expert ids (up to 4096) that the round's verify pass already lights up."""

    def __init__(self, ids: Sequence[int] = ()):
        self.bits = np.zeros(512, np.uint8)
        for e in ids:
            self.add(e)

    def add(self, e: int) -> None:
        e &= 4095
        self.bits[e >> 3] |= np.uint8(1 << (e & 7))

    def update(self, ids: Sequence[int]) -> None:
        for e in ids:
            self.add(e)

    def __contains__(self, e: int) -> bool:
        e &= 4095
        return bool(self.bits[e >> 3] >> (e & 7) & 1)

    def __len__(self) -> int:
        return int(np.unpackbits(self.bits).sum())

    def overlap(self, ids: Sequence[int]) -> int:
        return sum(1 for e in ids if e in self)


def route_aware_select(draft_logprobs: Sequence[float], experts: Sequence[Sequence[int]], union: ExpertUnion,
                       lam: float) -> int:
    """Index of the candidate maximising ``logprob + lam * |experts ∩ union|``.
    Reference: engine/src/spec/route_aware.rs:37-157."""
    n = len(draft_logprobs)
    off = np.zeros(n + 1, np.int32)
    ids: List[int] = []
    for i in range(n):
        ids.extend(experts[i])
        off[i + 1] = len(ids)
    ida = _ia(ids if ids else [0])
    return int(lib().ihb_route_aware_select(n, _pf(_fa(draft_logprobs)), _pi(off), _pi(ida),
                                            union.bits.ctypes.data_as(_u8), lam))
