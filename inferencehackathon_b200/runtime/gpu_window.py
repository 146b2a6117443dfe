"""Multi-token forward on the GPU: prompt chunks (TTFT) and speculative-verify windows (chains and token trees).

Per layer: row RMSNorm + activation rows for the tensor cores -> tcgen05 GEMM (QKV) -> QK-norm / RoPE / KV append at
explicit positions -> window attention (causal or tree mask) -> tcgen05 GEMM (o_proj) -> all-reduce -> router ->
tokens sorted by expert -> GROUPED tcgen05 GEMMs (gate/up + SwiGLU, down) driven by a device-side group table (the
routing result never visits the host) -> weighted combine -> all-reduce. Windows are processed in passes of up to
1024 tokens; a dense GEMM is ONE launch over all token tiles of the pass, a grouped expert GEMM one launch per pass.

Block-scaled fp8 weights are multiplied as bf16 here (``IHB_WINDOW_BF16=1``, the default): a scale per 128 x 128
weight block and per token forces the fp8 kernel to fold every 128-deep K block into fp32 registers on the CUDA
cores, which is ~20x slower than the MMAs it serves; de-quantised bf16 copies of the weights (e4m3 x scale rounds to
bf16 with 0.2 % relative error, a thirtieth of the e4m3 grid itself) let a whole K range accumulate in tensor memory
and need no activation quantisation. The copies stay resident when they fit beside the model; otherwise a layer's
weights are de-quantised into a scratch buffer right before its GEMMs.

Tensor-, expert- and hybrid-parallel layouts run the same code: the attention heads a rank holds are tp-way shards
replicated world / tp times (o_proj partials are scaled by tp / world), a rank runs the (token, slot) pairs whose
expert it holds, and both partial results of a layer are summed over ALL ranks by the fused all-reduce + residual +
RMSNorm kernels (counted small-message kernel up to 64 tokens, two-shot above).

The contractions, the attention and the routing are this package's kernels (``ihb_tc_gemm``, ``ihb_window_attention``,
``ihb_norm_quant_rows``, ``ihb_qk_norm_rope_rows``, ``ihb_router_topk_rows``, ``ihb_moe_group_table``,
``ihb_moe_gather_rows``, ``ihb_moe_combine_rows``); PyTorch tensor ops remain for the embedding gather, position /
slot vectors and one residual add on a single GPU. Reference counterparts: kernels/prefill_attn.cu, kernels/prefill_moe.cu,
kernels/prefill_wgmma.cu (prefill) and kernels/spec_verify_forward_gemm.cu, engine/native/tc_verify_attn.cuh
(verify).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config import env_flag
from ..models.quant import QWeight
from ..ops import lib as K

CHUNK = 1024          # tokens per pass (the expert weights are read about once per pass)
TILE = 128            # token tile of one dense GEMM launch


class GpuWindow:
    def __init__(self, dec):
        self.d = dec
        m, w = dec.cfg.model, dec.w
        if w.layers and w.layers[0].wqkv.data.device.type == "meta":
            raise RuntimeError("the window path needs the plain row-major weights (persistent or streaming pipeline)")
        # GEMM operand type of this path: bf16 for bf16 models and (by default) for block-fp8 models as well
        self.bf16_copies = dec.fp8 and bool(env_flag("IHB_WINDOW_BF16", 1))
        self.fp8 = dec.fp8 and not self.bf16_copies
        # bf16 GEMM inputs come out of the fused all-reduce kernel; IHB_WINDOW_AR_BF16=0 rounds them in a launch of its own
        self.ar_bf16 = not self.fp8 and bool(env_flag("IHB_WINDOW_AR_BF16", 1))
        self.es = 1 if self.fp8 else 2
        dev = dec.device
        self._bf16 = {}                       # data_ptr of an fp8 weight -> its resident bf16 copy
        self._resident = False
        if self.bf16_copies:
            seen, need = set(), 0
            for lw in w.layers:
                for qw in (lw.wqkv, lw.wo, lw.w_gu, lw.w_d):
                    if qw.data.data_ptr() not in seen:
                        seen.add(qw.data.data_ptr())
                        need += qw.data.numel() * 2
            free = torch.cuda.mem_get_info(dev)[0]
            self._resident = need + (10 << 30) < free and not env_flag("IHB_WINDOW_BF16_SCRATCH", 0)
        self.sms = torch.cuda.get_device_properties(dev).multi_processor_count
        self.err = dec.err
        self._ws = {}
        self._views = {}
        self._args = {}                       # argument blocks of the GEMM launches, built once per (weight, tokens)
        self.n_gemm_launches = 0
        # several GPUs (tensor, expert or hybrid parallel): the two all-reduces of a layer run as this package's fused kernel
        # (reduce in the switch or over peer loads, residual add, RMSNorm of the next block) on a symmetric buffer of its
        # own; IHB_WINDOW_FUSED_AR=0 falls back to NCCL + separate norm. Building the buffer is a collective: every rank
        # builds its window together. Attention heads are split tp ways and replicated world / tp times, so the o_proj
        # partials are scaled by tp / world before the sum over all ranks (the decode kernel does the same); experts are
        # split ep ways: a rank runs the (token, slot) pairs whose expert it holds, the sum over ranks combines them.
        self.ar = None
        par = dec.cfg.parallel
        self.attn_scale = float(par.tp) / float(max(par.world, 1))
        if par.world > 1 and env_flag("IHB_WINDOW_FUSED_AR", 1):
            from ..parallel.symm import SymmetricComm
            small = 4 * K.ARC_MAX_ROWS * dec.H * 8           # slots of the counted small-message variant (its own region)
            self.ar = SymmetricComm(par, dev, slot_floats=2 * CHUNK * dec.H, extra_bytes=small)
            self.ar_epoch = torch.zeros(4, dtype=torch.int32, device=dev)
            self.ar_counter = torch.zeros(8, dtype=torch.int32, device=dev)
            self.ar_cm = self.ar.comm_block(self.ar_epoch)
            self.ar_cm_small = self.ar.comm_block(self.ar_epoch, slot_offset_bytes=self.ar.extra_off)
            self.ar_calls = torch.zeros(K.ARC_MAX_ROWS, dtype=torch.int32, device=dev)

    def _all_reduce(self, part: torch.Tensor, resid: torch.Tensor, gamma: Optional[torch.Tensor], tag: str,
                    want_fp32_norm: bool = True):
        """sum over ranks of ``part`` + ``resid`` -> (new residual stream, its RMSNorm * gamma in fp32 or None, the same
        rounded to bf16 as GEMM input or None). The bf16 copy comes out of the all-reduce kernel itself when the GEMMs
        of this path take bf16 activations: no separate rounding launch."""
        d = self.d
        T, H = part.shape
        if self.ar is None:
            x = resid + d.comm_ref.all_reduce_world(part.clone() if d.cfg.parallel.world > 1 else part)
            return x, None, None
        out = self._buf("ar_out_" + tag, (T, H), torch.float32)
        outn = self._buf("ar_norm_" + tag, (T, H), torch.float32) if (gamma is not None and (want_fp32_norm or not self.ar_bf16)) else None
        outb = self._buf("ar_bf16_" + tag, (T, H * 2), torch.uint8) if (gamma is not None and self.ar_bf16) else None
        if T <= K.ARC_MAX_ROWS and H <= 8192:
            # verify windows and short prompts: one one-way trip through the switch, no barrier (9 us instead of 33 us
            # for the two-shot kernel at 16 KB on two GPUs)
            K.allreduce_counted(self.ar_cm_small, part, out, self.ar_counter, self.ar_calls, self.err, resid=resid, gamma=gamma,
                                eps=d.cfg.model.rms_eps, out_norm=outn, out_norm_bf16=outb)
            return out, outn, outb
        K.allreduce_norm(self.ar_cm, part, out, self.ar_counter, self.err, resid=resid, gamma=gamma,
                         eps=d.cfg.model.rms_eps, out_norm=outn, algo=2, out_norm_bf16=outb)
        return out, outn, outb

    def routing(self):
        """Expert ids ``[layers, T, k]`` (int32) and weights of the last chunk that went through this path: every
        token's routing decision as the device router took it."""
        if getattr(self, "_last_route_shape", None) is None:
            raise RuntimeError("no window has run yet")
        return (self._buf("ti_all", self._last_route_shape, torch.int32), self._buf("tw_all", self._last_route_shape, torch.float32))

    @property
    def act_mode(self) -> str:
        """How this path rounds activations before a linear layer ("fp8": per token and 128 channels; "bf16")."""
        return "fp8" if self.fp8 else "bf16"

    # ---- small helpers ---------------------------------------------------------------------------------------------
    def _buf(self, name: str, shape, dtype) -> torch.Tensor:
        """Workspace tensor ``name`` of the given shape: the same storage (and the same view object) every time it is
        asked for with the same shape, so that argument blocks built once stay valid and the host does no tensor
        bookkeeping per launch."""
        key = (name, tuple(shape), dtype)
        v = self._views.get(key)
        if v is not None:
            return v
        t = self._ws.get(name)
        n = 1
        for s in shape:
            n *= s
        if t is None or t.numel() < n or t.dtype != dtype:
            t = torch.zeros(max(n, 1), dtype=dtype, device=self.d.device)
            self._ws[name] = t
            self._views = {k: w for k, w in self._views.items() if k[0] != name}      # views of the old storage
            self._args = {}                                                           # and blocks that point into it
        v = t[:n].view(*shape)
        self._views[key] = v
        return v

    def _quant(self, x: torch.Tensor, gamma: Optional[torch.Tensor], tag: str, want_norm: bool = False):
        """x [T, K] fp32 -> (xq [T, K] e4m3|bf16 bytes, xs [ceil(K / 128), T] or None, xn or None)."""
        T, Kd = x.shape
        xq = self._buf("q_" + tag, (T, Kd * self.es), torch.uint8)
        xs = self._buf("s_" + tag, ((Kd + 127) // 128, T), torch.float32) if self.fp8 else None
        xn = self._buf("n_" + tag, (T, Kd), torch.float32) if want_norm else None
        K.norm_quant_rows(x.contiguous(), gamma, self.d.cfg.model.rms_eps, xq, xs, self.fp8, xn)
        return xq, xs, xn

    def _w(self, qw, tag: str):
        """The weight a GEMM of this path multiplies: ``qw`` itself, or its bf16 copy (resident, or de-quantised now
        into the scratch buffer ``tag``)."""
        if not self.bf16_copies or qw.scale is None:
            return qw
        key = qw.data.data_ptr()
        hit = self._bf16.get(key)
        if hit is not None:
            return hit
        out = (torch.empty(qw.data.shape, dtype=torch.bfloat16, device=qw.data.device) if self._resident
               else self._buf("w_" + tag, tuple(qw.data.shape), torch.bfloat16))
        if qw.data.shape[-1] % 16 == 0 and qw.kb % 16 == 0 and qw.data.is_contiguous():
            K.dequant_bf16(qw, out)                                          # one pass: 1 byte read, 2 written per weight
        elif qw.data.dim() == 3:
            step = max(1, (256 << 20) // max(1, qw.data[0].numel()))       # fp32 temporaries of ~1 GB at most
            for e0 in range(0, qw.data.shape[0], step):
                out[e0:e0 + step] = qw.select(slice(e0, e0 + step)).dequant(torch.bfloat16)
        else:
            out.copy_(qw.dequant(torch.bfloat16))
        res = QWeight(out)
        if self._resident:
            self._bf16[key] = res
        return res

    def _k_split(self, tiles: int, nkb: int, T: int) -> int:
        """K split of a dense launch. Measured on B200 (bf16, 1280 x 4096 weights): with 64 or more token columns per
        tile a split costs more than it gains even when the tiles cover half the SMs (1024 tokens: 39 us unsplit, 55 us
        split in two, 90 us in four; 128 tokens split in fourteen: 104 us) because the finishing unit reads every
        member's 32-64 KB partial; with 16 or 32 columns the partials are small and the split that minimises
        waves x (K blocks per unit + 2) wins (the head GEMV of one token: 149 row tiles on 148 SMs)."""
        if T > 32:
            return 1
        best, best_cost = 1, None
        for ks in range(1, min(nkb, 16) + 1):
            waves = -(-tiles * ks // self.sms)
            cost = waves * (-(-nkb // ks) + (2 if ks > 1 else 0))
            if best_cost is None or cost < best_cost:
                best, best_cost = ks, cost
        return best

    def _linear(self, qw, xq, xs, T: int, tag: str) -> torch.Tensor:
        """[T, K] x W[rows, K]^T on the tensor cores."""
        wq = self._w(qw, tag)
        key = ("lin", wq.data.data_ptr(), xq.data_ptr(), T, tag)
        hit = self._args.get(key)
        if hit is None:
            a = K.IhbTcArgs()
            K.tc_fill_weight(a, wq)
            rows = a.rows
            out = self._buf("o_" + tag, (T, rows), torch.float32)
            a.X, a.mode, a.out_stride = xq.data_ptr(), K.TC_LINEAR, rows
            if xs is not None:
                a.xscale = xs.data_ptr()
            a.T_total, a.err = T, self.err.data_ptr()
            nkb = (a.K * self.es + 127) // 128
            a.T, a.tok0, a.out = T, 0, out.data_ptr()
            if T > TILE:
                a.tok_tile, a.tok_tiles = TILE, -(-T // TILE)
            tiles = ((rows + 127) // 128) * max(1, a.tok_tiles)
            a.ks = self._k_split(tiles, nkb, T)
            part = self._buf("part", (max(1, K.tc_partial_floats(a)),), torch.float32)
            ctr = self._buf("ctr", (max(tiles, 1),), torch.int32)
            a.partial, a.tile_counters = part.data_ptr(), ctr.data_ptr()
            hit = (a, out)
            self._args[key] = hit
        K.tc_gemm(hit[0], False)
        self.n_gemm_launches += 1
        return hit[1]

    def _grouped(self, qw, mode, rows: int, xq, xs, groups, n_groups, max_groups: int, nt: int, n_pairs: int, tag: str):
        wq = self._w(qw, tag)
        key = ("grp", wq.data.data_ptr(), xq.data_ptr(), n_pairs, nt, tag)
        hit = self._args.get(key)
        if hit is None:
            a = K.IhbTcArgs()
            K.tc_fill_weight(a, wq)
            a.rows = rows
            out = self._buf("g_" + tag, (n_pairs, rows), torch.float32)
            a.X, a.mode, a.out, a.out_stride = xq.data_ptr(), mode, out.data_ptr(), rows
            if xs is not None:
                a.xscale = xs.data_ptr()
            a.T, a.T_total, a.tok0, a.err = nt, n_pairs, 0, self.err.data_ptr()
            a.top_k, a.ks = 1, 1
            a.groups, a.n_groups, a.max_groups = groups.data_ptr(), n_groups.data_ptr(), max_groups
            hit = (a, out)
            self._args[key] = hit
        K.tc_gemm(hit[0], False)
        self.n_gemm_launches += 1
        return hit[1]

    @staticmethod
    def _group_table(flat_e: torch.Tensor, n_experts: int, nt: int):
        """Tokens sorted by expert -> (order, groups [G, 4] int32 = {expert, first row, rows, 0}, n_groups [1], G), with
        plain tensor ops: the oracle of ``moe_group_table_kernel`` (which the forward pass uses), checkable on the CPU.
        G is an upper bound that depends only on shapes."""
        pairs = flat_e.numel()
        order = torch.argsort(flat_e, stable=True)
        cnt = torch.bincount(flat_e, minlength=n_experts)
        offs = torch.cumsum(cnt, 0) - cnt
        ng = (cnt + nt - 1) // nt
        cum = torch.cumsum(ng, 0)
        gmax = n_experts + pairs // nt + 1
        j = torch.arange(gmax, device=flat_e.device)
        e_of = torch.searchsorted(cum, j, right=True).clamp_(max=n_experts - 1)
        k_in = j - (cum[e_of] - ng[e_of])
        valid = j < cum[-1]
        tok0 = torch.where(valid, offs[e_of] + k_in * nt, torch.zeros_like(j))
        ntok = torch.where(valid, (cnt[e_of] - k_in * nt).clamp(0, nt), torch.zeros_like(j))
        groups = torch.stack([e_of, tok0, ntok, torch.zeros_like(j)], 1).to(torch.int32).contiguous()
        return order, groups, cum[-1:].to(torch.int32).contiguous(), gmax

    # ---- one chunk of up to CHUNK tokens ----------------------------------------------------------------------------------
    def _chunk(self, tokens: torch.Tensor, base: int, positions: torch.Tensor, mask: Optional[torch.Tensor],
               aux_layers=()) -> torch.Tensor:
        d = self.d
        m, w = d.cfg.model, d.w
        T = tokens.shape[0]
        dev = d.device
        slots = (base + torch.arange(T, device=dev)).to(torch.int32)
        pos32 = positions.to(torch.int32).contiguous()
        x = w.embed[tokens].float().contiguous()
        nq, nkv, H, I, k = d.nq, d.nkv, d.H, d.I, m.top_k
        mask_u8 = mask.to(torch.uint8).contiguous() if mask is not None else None
        self.aux_taps = {}
        xn = xb = None                                           # RMSNorm(x) * in_ln (fp32 / bf16) when the last all-reduce produced it
        n_layers = len(w.layers)
        for L, lw in enumerate(w.layers):
            if xb is not None:
                xq, xs = xb, None                                # bf16 rows straight from the all-reduce kernel
            else:
                xq, xs, _ = self._quant(xn, None, "x") if xn is not None else self._quant(x, lw.in_ln, "x")
            qkv = self._linear(lw.wqkv, xq, xs, T, "qkv")
            ksc, vsc = d.kv_scales(L)                            # e4m3 cache rows: one scale per row, else None
            K.qk_norm_rope_rows(qkv, nq, nkv, lw.q_norm, lw.k_norm, m.rms_eps, d.cos, d.sin, pos32, slots,
                                d.k_cache[L], d.v_cache[L], d.max_seq, k_scale=ksc, v_scale=vsc)
            attn = self._buf("attn", (T, nq * 128), torch.float32)
            K.window_attention(qkv, d.k_cache[L], d.v_cache[L], nq, nkv, d.max_seq, base, mask_u8, attn,
                               scratch=self._buf("attn_part", (K.window_attention_scratch_floats(nq, nkv, T),), torch.float32),
                               k_scale=ksc, v_scale=vsc)
            aq, asc, _ = self._quant(attn, None, "a")
            o = self._linear(lw.wo, aq, asc, T, "wo")
            if self.attn_scale != 1.0:
                o.mul_(self.attn_scale)
            x, h2, hb = self._all_reduce(o, x, lw.post_ln, "a" + str(L & 1))          # the router reads h2 in fp32
            if hb is not None:
                hq, hs = hb, None
            elif h2 is not None:
                hq, hs, _ = self._quant(h2, None, "h")
            else:
                hq, hs, h2 = self._quant(x, lw.post_ln, "h", want_norm=True)
            # fused router (logits, softmax, top-k) and the expert group table: kernels of this package, on the device
            pairs = T * k
            E_l = lw.w_gu.data.shape[0]
            ti = self._buf("ti_all", (n_layers, T, k), torch.int32)[L]
            tw = self._buf("tw_all", (n_layers, T, k), torch.float32)[L]
            rlog = self._buf("router_logits", (T, m.n_experts), torch.float32) if (T <= 32 or T >= 256) else None
            K.router_topk_rows(h2, lw.router, k, bool(m.norm_topk_prob), ti, tw, logits=rlog)
            per = max(1, pairs // m.n_experts)
            nt = 16 if per <= 12 else 32 if per <= 28 else 64
            gmax = E_l + pairs // nt + 1
            order = self._buf("order", (pairs,), torch.int32)
            inv = self._buf("inv", (pairs,), torch.int32)
            groups = self._buf("groups", (gmax, 4), torch.int32)
            n_groups = self._buf("n_groups", (1,), torch.int32)
            K.moe_group_table(ti, w.geom.expert0, E_l, nt, order, inv, groups, n_groups)
            # grouped expert GEMMs over the (token, slot) pairs in expert order
            gq = self._buf("gq", (pairs, hq.shape[1]), torch.uint8)
            K.moe_gather_rows(hq, order, k, gq)
            gs = None
            if hs is not None:
                gs = hs[:, (order // k).long()].contiguous()
            act = self._grouped(lw.w_gu, K.TC_GATEUP, I, gq, gs, groups, n_groups, gmax, nt, pairs, "act")
            cq, cs, _ = self._quant(act, None, "c")
            yg = self._grouped(lw.w_d, K.TC_DOWN, H, cq, cs, groups, n_groups, gmax, nt, pairs, "y")
            if d.cfg.parallel.world > 1:
                y = self._buf("ycomb", (T, H), torch.float32)
                K.moe_combine_rows(yg, inv, tw, k, y)               # slot order: deterministic
                nxt = w.layers[L + 1].in_ln if L + 1 < n_layers else None
                x, xn, xb = self._all_reduce(y, x, nxt, "m" + str(L & 1), want_fp32_norm=False)
            else:
                xnew = self._buf("xres" + str(L & 1), (T, H), torch.float32)
                K.moe_combine_rows(yg, inv, tw, k, xnew, resid=x)
                x = xnew
            if L in aux_layers:
                self.aux_taps[L] = x.clone()
        self._last_route_shape = (n_layers, T, k)
        if n_layers:
            # routing telemetry of the window's last token, all layers in one copy
            d.sel_idx.copy_(self._buf("ti_all", (n_layers, T, k), torch.int32)[:, -1])
            d.sel_w.copy_(self._buf("tw_all", (n_layers, T, k), torch.float32)[:, -1])
        return x

    def _head(self, x: torch.Tensor) -> torch.Tensor:
        d = self.d
        w = d.w
        xq, xs, _ = self._quant(x, w.final_norm, "f")
        local = self._linear(w.lm_head, xq, xs, x.shape[0], "head")
        if d.cfg.parallel.world == 1:
            return local.clone()
        return d.comm_ref.gather_logits(local.clone(), d.cfg.model.vocab, w.geom.vocab_chunk)

    # ---- public -----------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, tokens, commit: bool = True, tree_mask=None, positions=None, last_only: bool = False,
                aux_layers=()) -> torch.Tensor:
        """Logits ``[T, V]`` (``last_only``: ``[1, V]``) of ``tokens`` appended after the cached context. Rows are
        written to the KV cache at ``seq_len ...``; ``commit=False`` leaves the sequence length unchanged."""
        d = self.d
        dev = d.device
        toks = torch.as_tensor(list(tokens) if not isinstance(tokens, torch.Tensor) else tokens, dtype=torch.long, device=dev)
        T = toks.shape[0]
        base = d.seq_len
        if base + T > d.max_seq:
            raise ValueError("KV cache overflow")
        if tree_mask is not None and T > TILE:
            raise ValueError(f"a masked window holds at most {TILE} tokens")
        pos = positions.to(dev) if positions is not None else base + torch.arange(T, device=dev)
        outs: List[torch.Tensor] = []
        for c0 in range(0, T, CHUNK):
            c1 = min(T, c0 + CHUNK)
            x = self._chunk(toks[c0:c1], base + c0, pos[c0:c1], tree_mask, aux_layers)
            if not last_only:
                outs.append(self._head(x))
            elif c1 == T:
                outs.append(self._head(x[-1:].contiguous()))
        if commit:
            d.pos.fill_(base + T)
        d.check_error()
        return torch.cat(outs, 0)
