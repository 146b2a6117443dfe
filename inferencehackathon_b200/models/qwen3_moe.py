"""Functional Qwen3-MoE decoder in plain PyTorch: the numerical oracle for every CUDA kernel and the engine
behind the CPU/gloo configuration.

Math (all taken from the reference kernels' behaviour, not their code): RMSNorm eps 1e-6, per-head RMSNorm on Q
and K before RoPE (kernels/k1_attn_prologue.cu:524-604), NeoX rotate-half RoPE with theta 1e6, grouped-query
causal attention, router = softmax over all experts in fp32, top-k, renormalise the k weights to sum 1
(kernels/k4_router.cu:67-132), SwiGLU experts ``down(silu(gate x) * up x)`` (kernels/k5_experts.cu:91-149),
untied lm_head after a final RMSNorm (kernels/decode_step.cu:144-185).

Tensor parallelism follows kernels/decode_step_tp8.cu:18-41 (partial o_proj / down outputs summed over the TP
group); expert parallelism routes each token from its home rank to the ranks that own its experts and back.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch

from ..config import ModelConfig
from ..parallel.collectives import Collectives
from .weights import LayerWeights, ModelWeights


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return xf * inv * w.float()


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float) -> Tuple[torch.Tensor, torch.Tensor]:
    half = head_dim // 2
    inv_freq = theta ** (-torch.arange(0, half, dtype=torch.float32, device=positions.device) / half)
    ang = positions.float()[:, None] * inv_freq[None, :]
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """NeoX rotate-half on ``x[T, heads, hd]``: pairs (d, d + hd/2)."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def fake_quant_act(x: torch.Tensor, mode) -> torch.Tensor:
    """Round activations the way the tensor-core kernels store them: ``"fp8"`` = e4m3 with one scale per token
    per 128 channels, ``"bf16"``; ``None`` leaves them alone."""
    if mode is None:
        return x
    if mode == "bf16":
        return x.to(torch.bfloat16).float()
    K = x.shape[-1]
    Kp = (K + 127) // 128 * 128
    xp = torch.nn.functional.pad(x.float(), (0, Kp - K)).reshape(*x.shape[:-1], Kp // 128, 128)
    s = xp.abs().amax(dim=-1, keepdim=True).clamp_min(1e-12) / 448.0
    q = (xp / s).clamp(-448, 448).to(torch.float8_e4m3fn).float() * s
    return q.reshape(*x.shape[:-1], Kp)[..., :K]


def route(h: torch.Tensor, router_w: torch.Tensor, top_k: int, renorm: bool = True):
    """Router: fp32 softmax over all experts, top-k, optional renormalisation. Returns ``(idx, w, logits)``."""
    logits = h.float() @ router_w.float().t()
    probs = torch.softmax(logits, dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if renorm:
        w = w / w.sum(dim=-1, keepdim=True)
    return idx, w, logits


@dataclass
class RouteRecord:
    """Expert choice of one token in one layer (global expert ids and renormalised weights)."""
    layer: int
    experts: List[int]
    weights: List[float]


class TorchKV:
    """Contiguous KV cache ``[layers, kv_heads_local, max_seq, hd]`` for the PyTorch path. With
    ``dtype=torch.float8_e4m3fn`` rows are stored as e4m3 with one fp32 scale per (layer, head, position) (amax / 448)
    and dequantised on read; the reference stores e4m3 with static per-channel scales
    (kernels/k1_attn_prologue.cu:524-604, kernels/k2_flash_decode.cu:71-83)."""

    def __init__(self, n_layers: int, n_kv: int, max_seq: int, hd: int, dtype, device):
        self.k = torch.zeros(n_layers, n_kv, max_seq, hd, dtype=dtype, device=device)
        self.v = torch.zeros_like(self.k)
        self.fp8 = dtype == torch.float8_e4m3fn
        if self.fp8:
            self.k_scale = torch.ones(n_layers, n_kv, max_seq, 1, dtype=torch.float32, device=device)
            self.v_scale = torch.ones_like(self.k_scale)
        self.len = 0
        self.max_seq = max_seq

    def reset(self) -> None:
        self.len = 0

    def write(self, L: int, start: int, k: torch.Tensor, v: torch.Tensor) -> None:
        """k, v ``[nkv, T, hd]`` -> rows ``start .. start + T`` of layer ``L``."""
        T = k.shape[1]
        if not self.fp8:
            self.k[L, :, start:start + T] = k.to(self.k.dtype)
            self.v[L, :, start:start + T] = v.to(self.v.dtype)
            return
        for buf, sc, x in ((self.k, self.k_scale, k), (self.v, self.v_scale, v)):
            s = x.float().abs().amax(dim=-1, keepdim=True).clamp_min(1e-12) / 448.0
            buf[L, :, start:start + T] = (x.float() / s).clamp(-448, 448).to(torch.float8_e4m3fn)
            sc[L, :, start:start + T] = s

    def write_rows(self, L: int, rows: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
        """k, v ``[nkv, R, hd]`` -> the (not necessarily contiguous) rows ``rows[R]`` of layer ``L``."""
        if rows.numel() == 0:
            return
        if not self.fp8:
            self.k[L][:, rows] = k.to(self.k.dtype)
            self.v[L][:, rows] = v.to(self.v.dtype)
            return
        for buf, sc, x in ((self.k, self.k_scale, k), (self.v, self.v_scale, v)):
            s = x.float().abs().amax(dim=-1, keepdim=True).clamp_min(1e-12) / 448.0
            buf[L][:, rows] = (x.float() / s).clamp(-448, 448).to(torch.float8_e4m3fn)
            sc[L][:, rows] = s

    def read(self, L: int, n: int):
        """Rows ``0 .. n`` of layer ``L`` as (k, v) in a float type."""
        if not self.fp8:
            return self.k[L, :, :n], self.v[L, :, :n]
        return self.k[L, :, :n].float() * self.k_scale[L, :, :n], self.v[L, :, :n].float() * self.v_scale[L, :, :n]


def _attention(q: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor, positions: torch.Tensor,
               extra_mask: Optional[torch.Tensor]) -> torch.Tensor:
    """q[T, nq, hd]; kc/vc[nkv, S, hd] (S = cached length incl. the new tokens); causal w.r.t. ``positions``.

    ``extra_mask[T, T_new]`` (bool, True = visible) replaces causality among the new tokens for tree verify."""
    T, nq, hd = q.shape
    nkv, S, _ = kc.shape
    g = nq // nkv
    qf = q.float().reshape(T, nkv, g, hd).permute(1, 2, 0, 3)                     # [nkv, g, T, hd]
    scores = torch.einsum("kgtd,ksd->kgts", qf, kc.float()) * (hd ** -0.5)
    kpos = torch.arange(S, device=q.device)
    visible = kpos[None, :] <= positions[:, None]                                  # [T, S]
    if extra_mask is not None:
        t_new = extra_mask.shape[1]
        visible = visible.clone()
        visible[:, S - t_new:] = extra_mask
    scores = scores.masked_fill(~visible[None, None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    out = torch.einsum("kgts,ksd->kgtd", p, vc.float())
    return out.permute(2, 0, 1, 3).reshape(T, nq * hd)


def _attention_partial(q: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor, visible: torch.Tensor):
    """Attention of ``q[T, nh, hd]`` over SOME rows ``kc / vc [R, hd]`` of one KV head (``visible[T, R]``): the
    un-normalised output ``acc[T, nh, hd]`` with its running maximum ``m[T, nh]`` and denominator ``l[T, nh]``, i.e. the
    record a split-KV kernel writes per split. Rows a query does not see contribute nothing; a query that sees no row
    returns ``m = -inf, l = 0, acc = 0``."""
    T, nh, hd = q.shape
    if kc.shape[0] == 0:
        z = q.new_zeros(T, nh, dtype=torch.float32)
        return q.new_zeros(T, nh, hd, dtype=torch.float32), z - float("inf"), z
    scores = torch.einsum("thd,sd->ths", q.float(), kc.float()) * (hd ** -0.5)
    scores = scores.masked_fill(~visible[:, None, :], float("-inf"))
    m = scores.amax(-1)
    p = torch.exp(scores - torch.where(torch.isinf(m), torch.zeros_like(m), m)[..., None])
    p = torch.where(visible[:, None, :], p, torch.zeros_like(p))
    return torch.einsum("ths,sd->thd", p, vc.float()), m, p.sum(-1)


def _merge_partials(parts) -> torch.Tensor:
    """[(acc, m, l), ...] of disjoint row sets -> normalised attention output ``[T, nh, hd]`` (the merge a split-KV
    kernel does across its splits, here across the ranks that share a KV head)."""
    M = torch.stack([m for _, m, _ in parts]).amax(0)
    num = torch.zeros_like(parts[0][0])
    den = torch.zeros_like(parts[0][2])
    for acc, m, l in parts:
        f = torch.where(torch.isinf(m), torch.zeros_like(m), torch.exp(m - M))
        num = num + acc * f[..., None]
        den = den + l * f
    return num / den[..., None]


def _experts_local(h: torch.Tensor, lw: LayerWeights, idx: torch.Tensor, w: torch.Tensor, expert0: int,
                   n_local: int, act_mode=None) -> torch.Tensor:
    """Sum over the (token, slot) pairs whose expert is held locally; ``idx`` holds global expert ids."""
    out = torch.zeros(h.shape[0], lw.w_d.data.shape[-2], dtype=torch.float32, device=h.device)
    local = idx - expert0
    for e in torch.unique(local[(local >= 0) & (local < n_local)]).tolist():
        tok, slot = torch.nonzero(local == e, as_tuple=True)
        x = fake_quant_act(h[tok].float(), act_mode)
        wgu = lw.w_gu.select(e).dequant()
        I = wgu.shape[0] // 2
        gu = x @ wgu.t()
        a = fake_quant_act(torch.nn.functional.silu(gu[:, :I]) * gu[:, I:], act_mode)
        y = a @ lw.w_d.select(e).dequant().t()
        out.index_add_(0, tok, y * w[tok, slot].float()[:, None])
    return out


class Qwen3MoE:
    """One rank's model. ``forward`` runs ``T`` new tokens (prefill chunk, decode step or verify window)."""

    def __init__(self, weights: ModelWeights, comm: Optional[Collectives] = None, compute_dtype=torch.float32):
        self.w = weights
        self.cfg: ModelConfig = weights.cfg
        self.par = weights.par
        self.geom = weights.geom
        self.comm = comm if comm is not None else Collectives(weights.par)
        self.compute_dtype = compute_dtype
        self.last_routes: List[RouteRecord] = []
        self.aux_taps: dict = {}
        self.act_mode = None       # "fp8" / "bf16": round activations before every linear layer like the CUDA path
        # optional replacement of the router: (layer, h, router_w, top_k, renorm) -> (idx, w, logits); a dropped
        # expert keeps its slot with weight 0 (experiments: confidence-adaptive top-k)
        self.route_fn = None

    def _route(self, L: int, h: torch.Tensor, lw: LayerWeights):
        cfg = self.cfg
        if self.route_fn is not None:
            return self.route_fn(L, h, lw.router, cfg.top_k, cfg.norm_topk_prob)
        return route(h, lw.router, cfg.top_k, cfg.norm_topk_prob)

    def new_cache(self, max_seq: int, dtype=torch.float32, device=None) -> TorchKV:
        device = device if device is not None else self.w.embed.device
        share = self.par.kv_share
        rows = max_seq if share <= 1 else (max_seq + share - 1) // share      # a rank keeps every share-th row of its KV head
        kv = TorchKV(self.cfg.n_layers, self.geom.nkv_local, rows, self.cfg.head_dim, dtype, device)
        kv.max_seq = max_seq                                                 # positions it covers (``len`` counts positions)
        return kv

    # ---------------------------------------------------------------------------------------------------------
    def _moe(self, L: int, h: torch.Tensor, lw: LayerWeights, record: bool) -> torch.Tensor:
        cfg, par, geom = self.cfg, self.par, self.geom
        if par.ep == 1:
            idx, w, _ = self._route(L, h, lw)
            if record:
                self.last_routes.append(RouteRecord(L, idx[-1].tolist(), w[-1].tolist()))
            y = _experts_local(h, lw, idx, w, 0, cfg.n_experts, self.act_mode)
            return self.comm.all_reduce_tp(y)
        # expert parallel: home rank of token m is m % world -----------------------------------------------
        world, rank = par.world, par.rank
        T = h.shape[0]
        home = torch.arange(T, device=h.device) % world
        mine = torch.nonzero(home == rank, as_tuple=True)[0]
        idx, w, _ = self._route(L, h[mine], lw)
        n_el = geom.n_experts_local
        owner = idx // n_el                                                     # [Tm, k]
        flat_tok = mine[:, None].expand_as(idx).reshape(-1)
        flat_owner, flat_idx, flat_w = owner.reshape(-1), idx.reshape(-1), w.reshape(-1)
        order = torch.argsort(flat_owner, stable=True)
        send_counts = torch.bincount(flat_owner, minlength=world).tolist()
        # dispatch: hidden row, expert id and weight travel together (2 extra fp32 columns)
        payload = torch.cat([h[flat_tok[order]].float(), flat_idx[order, None].float(),
                             flat_w[order, None].float()], dim=1)
        # the peer-memory exchange holds at most `cap` rows per (source, destination): decided from T, which every rank knows
        fast = getattr(self.comm, "fast_a2a", None)
        allow = fast is not None and -(-T // world) * cfg.top_k <= fast.cap
        recv, recv_counts = self.comm.all_to_all_rows(payload, send_counts, allow)
        rh, ridx, rw = recv[:, :-2], recv[:, -2].long(), recv[:, -1]
        yo = torch.zeros(rh.shape[0], cfg.hidden, dtype=torch.float32, device=h.device)
        if rh.shape[0]:
            yo = _experts_local(rh, lw, ridx[:, None], rw[:, None], geom.expert0, n_el, self.act_mode)
        # combine: rows go back to their home rank in the order they came
        back, _ = self.comm.all_to_all_rows(yo, recv_counts, allow)
        y_mine = torch.zeros(mine.shape[0], cfg.hidden, dtype=torch.float32, device=h.device)
        if back.shape[0]:
            slot_of = torch.arange(mine.shape[0], device=h.device)[:, None].expand_as(idx).reshape(-1)[order]
            y_mine.index_add_(0, slot_of, back)
        # every rank needs every token for the next attention block
        y = torch.zeros(T, cfg.hidden, dtype=torch.float32, device=h.device)
        y[mine] = y_mine
        y = self.comm.all_reduce_world(y)
        if record:
            last_home = (T - 1) % world
            rec = torch.zeros(2 * cfg.top_k, dtype=torch.float32, device=h.device)
            if rank == last_home:
                rec[: cfg.top_k] = idx[-1].float()
                rec[cfg.top_k:] = w[-1].float()
            rec = self.comm.all_reduce_world(rec)
            self.last_routes.append(RouteRecord(L, rec[: cfg.top_k].long().tolist(), rec[cfg.top_k:].tolist()))
        return y

    def forward_hidden(self, tokens: torch.Tensor, cache: TorchKV, positions: Optional[torch.Tensor] = None,
                       tree_mask: Optional[torch.Tensor] = None, commit: bool = True,
                       record_routes: bool = True, aux_layers: Tuple[int, ...] = ()) -> torch.Tensor:
        """Runs the decoder stack over ``tokens[T]`` whose KV rows are written at ``cache.len ...``; returns the
        final-normed hidden states ``[T, H]``. ``commit=False`` leaves ``cache.len`` unchanged (verify window)."""
        cfg, geom = self.cfg, self.geom
        T = tokens.shape[0]
        start = cache.len
        if start + T > cache.max_seq:
            raise ValueError("KV cache overflow")
        if positions is None:
            positions = torch.arange(start, start + T, device=tokens.device)
        cos, sin = rope_tables(positions, cfg.head_dim, cfg.rope_theta)
        x = self.w.embed[tokens].float()
        self.last_routes = []
        self.aux_taps = {}
        hd = cfg.head_dim
        for L, lw in enumerate(self.w.layers):
            h = rmsnorm(x, lw.in_ln, cfg.rms_eps)
            qkv = fake_quant_act(h, self.act_mode) @ lw.wqkv.dequant().t()
            nq, nkv = geom.nq_local, geom.nkv_local
            q = qkv[:, : nq * hd].reshape(T, nq, hd)
            k = qkv[:, nq * hd: (nq + nkv) * hd].reshape(T, nkv, hd)
            v = qkv[:, (nq + nkv) * hd:].reshape(T, nkv, hd)
            q = apply_rope(rmsnorm(q, lw.q_norm, cfg.rms_eps), cos, sin)
            k = apply_rope(rmsnorm(k, lw.k_norm, cfg.rms_eps), cos, sin)
            if self.par.kv_share > 1:
                attn = self._attention_kv_split(L, q, k, v, cache, start, positions, tree_mask)
            else:
                cache.write(L, start, k.permute(1, 0, 2), v.permute(1, 0, 2))
                kc, vc = cache.read(L, start + T)
                attn = _attention(q, kc, vc, positions, tree_mask)
            o = fake_quant_act(attn, self.act_mode) @ lw.wo.dequant().t()
            x = x + self.comm.all_reduce_tp(o)
            h2 = rmsnorm(x, lw.post_ln, cfg.rms_eps)
            x = x + self._moe(L, h2, lw, record_routes)
            if L in aux_layers:
                self.aux_taps[L] = x.clone()
        if commit:
            cache.len = start + T
        return rmsnorm(x, self.w.final_norm, cfg.rms_eps)

    def _attention_kv_split(self, L: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cache: TorchKV, start: int,
                            positions: torch.Tensor, tree_mask: Optional[torch.Tensor]) -> torch.Tensor:
        """Context-parallel attention for the ranks that share one KV head (tp above the number of KV heads; the
        reference replicates the head's whole cache on them, kernels/decode_step_tp8.cu:153-160). Rank i of the group
        keeps cache rows r with r % kv_share == i, stored compactly at r // kv_share: 1 / kv_share of the head's KV bytes
        per rank. Per layer: the group gathers its query heads (every rank needs all of them for its rows), each rank
        attends over its own rows and produces un-normalised partials (acc, m, l), the group gathers the partials and
        every rank merges those of its own heads: the split-KV merge, across GPUs."""
        share = self.par.kv_share
        me = self.par.tp_rank % share
        T, nq, hd = q.shape
        slots = torch.arange(start, start + T, device=q.device)
        own_new = (slots % share) == me
        cache.write_rows(L, slots[own_new] // share, k[own_new].permute(1, 0, 2), v[own_new].permute(1, 0, 2))
        n_rows = (start + T - me + share - 1) // share if start + T > me else 0    # rows r < start + T with r % share == me
        kc, vc = cache.read(L, n_rows)
        own_slots = torch.arange(n_rows, device=q.device) * share + me
        visible = own_slots[None, :] <= positions[:, None]                         # as in _attention, on this rank's rows
        if tree_mask is not None:
            in_window = own_slots >= start
            visible = visible.clone()
            visible[:, in_window] = tree_mask[:, own_slots[in_window] - start]
        q_all = torch.cat(self.comm.all_gather_kv(q.float()), dim=1)               # [T, share * nq, hd], heads in rank order
        acc, m, l = _attention_partial(q_all, kc[0], vc[0], visible)
        packed = torch.cat([acc, m[..., None], l[..., None]], dim=-1)              # one record per (token, head)
        recs = self.comm.all_gather_kv(packed)
        mine = slice(me * nq, (me + 1) * nq)
        out = _merge_partials([(r[:, mine, :hd], r[:, mine, hd], r[:, mine, hd + 1]) for r in recs])
        return out.reshape(T, nq * hd)

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """Full-vocabulary logits ``[T, V]`` (gathered from the vocabulary shards)."""
        local = fake_quant_act(hidden.float(), self.act_mode) @ self.w.lm_head.dequant().t()
        return self.comm.gather_logits(local, self.cfg.vocab, self.geom.vocab_chunk)

    def greedy(self, hidden: torch.Tensor) -> torch.Tensor:
        local = fake_quant_act(hidden.float(), self.act_mode) @ self.w.lm_head.dequant().t()
        return self.comm.argmax_sharded(local, self.geom.vocab0)[1]

    def forward(self, tokens: torch.Tensor, cache: TorchKV, **kw) -> torch.Tensor:
        return self.logits(self.forward_hidden(tokens, cache, **kw))
