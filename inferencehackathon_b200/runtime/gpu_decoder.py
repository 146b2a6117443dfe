"""Decode pipeline on the sm_100a kernels: seven launches per layer, the whole token under one CUDA graph.

Per layer: QKV GEMV -> QK-norm/RoPE/KV append -> split-KV flash decode -> o_proj GEMV fused with the
all-reduce, residual add and post-attention RMSNorm -> router GEMV with softmax/top-k tail -> expert gate/up
SwiGLU -> expert down projection fused with the all-reduce, residual add and the next layer's input RMSNorm.
The head GEMV ends with the argmax, writes the next token and advances the position counter on the device, so a
replayed graph needs no host input (the reference's graph replays a fixed dummy state,
kernels/k6_graph_capture.cu:33-64; its eager path issues ~1100 launches per token,
kernels/decode_step_tp8.cu:1193-1195).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional

import torch

from ..config import EngineConfig, env_flag
from ..models.qwen3_moe import RouteRecord, rope_tables
from ..models.weights import ModelWeights
from ..ops import lib as K


def _pick_ks(Kdim: int, celems: int) -> int:
    ks = 1
    while Kdim // ks // celems > 256 and ks < 8:
        ks *= 2
    return ks


class GpuDecoder:
    def __init__(self, cfg: EngineConfig, weights: ModelWeights, comm, device: torch.device):
        if device.type != "cuda":
            raise RuntimeError("the sm_100a decode path needs a CUDA device")
        K.load()
        self.cfg, self.w, self.device = cfg, weights, device
        m, g = cfg.model, weights.geom
        if m.head_dim != 128:
            raise ValueError("the CUDA attention kernels are built for head_dim 128")
        if weights.quant.weights not in ("bf16", "fp8_block"):
            raise ValueError("the CUDA path stores weights as bf16 or block-scaled fp8")
        self.H, self.nq, self.nkv, self.I = m.hidden, g.nq_local, g.nkv_local, g.inter_local
        self.max_seq = cfg.max_seq
        self.use_pdl = bool(env_flag("IHB_PDL", 1))
        self.use_tc = bool(env_flag("IHB_TC", 1))          # tensor-core linears (0: SIMT streaming GEMVs)
        # persistent whole-token kernel (tensor parallel only; expert parallel keeps the per-kernel pipeline)
        self.use_mega = bool(env_flag("IHB_MEGA", 1)) and m.n_experts <= 256
        # e4m3 KV cache with one scale per (layer, KV head, position): half the cache bytes per context token. The append
        # and attention kernels of the per-kernel pipeline and of the window path read it (the reference:
        # kernels/k1_attn_prologue.cu:524-604, kernels/k2_flash_decode.cu:71-83); the persistent kernel is built for
        # bf16 rows, so this mode runs the streaming per-kernel pipeline, whose weights the window path shares.
        self.kv_fp8 = cfg.quant.kv == "fp8"
        if self.kv_fp8:
            self.use_mega = False
            self.use_tc = False
        if cfg.parallel.kv_share > 1:
            raise ValueError("the CUDA pipelines keep all rows of a shared KV head on every rank; kv_seq_split is a "
                             "feature of the PyTorch path")
        if not self.use_mega and cfg.parallel.ep > 1 and cfg.parallel.world > 1:
            raise ValueError("expert parallelism on GPUs runs inside the persistent kernel; the per-kernel pipelines "
                             "(IHB_MEGA=0, kv='fp8') are tensor-parallel only")
        self.fp8 = weights.quant.weights == "fp8_block"
        self.use_graph = cfg.use_graph and bool(env_flag("IHB_GRAPH", 1))
        self.comm_ref = comm
        self.n_launches_per_step = 0
        dev = device
        f32 = dict(dtype=torch.float32, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        L = m.n_layers
        self.resid = torch.zeros(self.H, **f32)
        self.xn = torch.zeros(self.H, **f32)
        self.qkv = torch.zeros((self.nq + 2 * self.nkv) * 128, **f32)
        self.attn = torch.zeros(self.nq * 128, **f32)
        self.act = torch.zeros(m.top_k * self.I, **f32)
        self.router_logits = torch.zeros(L, m.n_experts, **f32)
        self.sel_idx = torch.zeros(L, m.top_k, **i32)
        self.sel_w = torch.zeros(L, m.top_k, **f32)
        # next token and device error word side by side: one device->host copy per step returns both
        self._tok_err = torch.zeros(2, **i32)
        self.cur_token = self._tok_err[0:1]
        self.pos = torch.zeros(1, **i32)
        self.n_forced = torch.zeros(1, **i32)
        self.forced = torch.zeros(self.max_seq + 1, **i32)
        self.token_ring = torch.zeros(self.max_seq + 1, **i32)
        self.counters = torch.zeros(8 + self.nq, dtype=torch.int32, device=dev)
        self.err = self._tok_err[1:2]
        self.epoch = torch.zeros(4, **i32)          # [0] all-reduce rounds, [1] arrival-counter rounds (persistent kernel)
        self.argmax_partial = torch.zeros(1024, dtype=torch.int64, device=dev)
        self.logits = torch.zeros(max(g.vocab_local, 1), **f32)
        kv_shape = (L, self.nkv, self.max_seq, 128)
        kv_t = torch.uint8 if self.kv_fp8 else torch.bfloat16
        self.k_cache = torch.zeros(kv_shape, dtype=kv_t, device=dev)
        self.v_cache = torch.zeros(kv_shape, dtype=kv_t, device=dev)
        self.k_scale = torch.zeros(kv_shape[:3], **f32) if self.kv_fp8 else None
        self.v_scale = torch.zeros(kv_shape[:3], **f32) if self.kv_fp8 else None
        cos, sin = rope_tables(torch.arange(self.max_seq, device=dev), 128, m.rope_theta)
        self.cos, self.sin = cos.contiguous(), sin.contiguous()
        q_per_kv = self.nq // self.nkv
        ngroups = max(1, q_per_kv // 8)
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        want = max(1, (2 * sms) // (self.nkv * ngroups))
        self.nsplit = env_flag("IHB_FD_SPLITS", max(1, min((self.max_seq + 127) // 128, want)))
        self.fd_scratch = torch.zeros(K.flash_decode_scratch_floats(self.nq, self.nsplit), **f32)
        celems = 16 if weights.quant.weights == "fp8_block" else 8
        self.ks_o = _pick_ks(self.nq * 128, celems)
        self._setup_comm()
        if self.use_mega:
            self._build_mega()
        elif self.use_tc:
            self._build_tc()
        else:
            self._build_args()
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._window = None
        self._ev0 = torch.cuda.Event(enable_timing=True)
        self._ev1 = torch.cuda.Event(enable_timing=True)
        # pinned staging for the per-step host<->device traffic of the public decode_step API
        self._tok_in = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._tok_out = torch.zeros(2, dtype=torch.int32).pin_memory()
        self.h2d_bytes_per_step = self._tok_in.numel() * 4
        self.d2h_bytes_per_step = self._tok_out.numel() * 4

    # communication block -------------------------------------------------------------------------------------
    def _setup_comm(self) -> None:
        par = self.cfg.parallel
        # the persistent kernel keeps 8 round parities of 64-bit slots: 16 floats per hidden channel
        nslots = max(2 * max(par.world, par.tp, 1) * max(self.ks_o, 2), 16) * self.H
        if par.world == 1:
            self.slots = torch.zeros(nslots, dtype=torch.float32, device=self.device)
            self.symm = None
        else:
            from ..parallel.symm import SymmetricComm
            self.symm = SymmetricComm(par, self.device, slot_floats=nslots)
            self.slots = self.symm.slots_local

    def _comm(self) -> K.IhbComm:
        if self.symm is None:
            return K.single_comm(self.slots, self.epoch)
        return self.symm.comm_block(self.epoch)

    # argument blocks -----------------------------------------------------------------------------------------
    def _gemv_args(self, qw, x, epi, **kw) -> K.IhbGemvArgs:
        a = K.IhbGemvArgs()
        K.fill_weight(a, qw)
        a.x = x.data_ptr()
        a.epi = epi
        a.ks = kw.pop("ks", 1)
        a.err = self.err.data_ptr()
        a.counter = kw.pop("counter").data_ptr() if "counter" in kw else None
        for k, v in kw.items():
            setattr(a, k, v.data_ptr() if isinstance(v, torch.Tensor) else v)
        return a

    def _build_args(self) -> None:
        m, w = self.cfg.model, self.w
        from ..models.quant import QWeight
        self.layer_args = []
        ctr = self.counters
        for L, lw in enumerate(w.layers):
            nxt_gamma = w.layers[L + 1].in_ln if L + 1 < len(w.layers) else w.final_norm
            qkv = self._gemv_args(lw.wqkv, self.xn, K.EPI_STORE, out=self.qkv)
            oproj = self._gemv_args(lw.wo, self.attn, K.EPI_AR_NORM, ks=self.ks_o, counter=ctr[0:1],
                                    resid=self.resid, gamma=lw.post_ln, xn_out=self.xn, eps=m.rms_eps)
            oproj.comm = self._comm()
            router = self._gemv_args(QWeight(lw.router), self.xn, K.EPI_ROUTER, counter=ctr[1:2],
                                     out=self.router_logits[L], top_k=m.top_k, renorm=int(m.norm_topk_prob),
                                     sel_idx=self.sel_idx[L], sel_w=self.sel_w[L])
            moe = K.IhbMoeArgs()
            moe.Wgu, moe.Wd = lw.w_gu.data.data_ptr(), lw.w_d.data.data_ptr()
            moe.wtype = K.wtype_of(lw.w_gu.data)
            moe.H, moe.I, moe.E_local = self.H, self.I, lw.w_gu.data.shape[0]
            moe.expert0, moe.top_k = w.geom.expert0, m.top_k
            if lw.w_gu.scale is not None:
                gsc, dsc = K.kernel_scale(lw.w_gu), K.kernel_scale(lw.w_d)
                moe.gu_scale, moe.d_scale = gsc.data_ptr(), dsc.data_ptr()
                moe.gu_rb, moe.gu_kb_shift, moe.gu_nkb = lw.w_gu.rb, K.kb_shift_of(lw.w_gu.kb), gsc.shape[-1]
                moe.d_rb, moe.d_kb_shift, moe.d_nkb = lw.w_d.rb, K.kb_shift_of(lw.w_d.kb), dsc.shape[-1]
            moe.x, moe.act = self.xn.data_ptr(), self.act.data_ptr()
            moe.sel_idx, moe.sel_w = self.sel_idx[L].data_ptr(), self.sel_w[L].data_ptr()
            moe.counter, moe.err = ctr[2:3].data_ptr(), self.err.data_ptr()
            moe.resid, moe.gamma, moe.xn_out, moe.eps = (self.resid.data_ptr(), nxt_gamma.data_ptr(),
                                                         self.xn.data_ptr(), m.rms_eps)
            moe.comm = self._comm()
            self.layer_args.append((qkv, oproj, router, moe, lw))
        self.head = self._gemv_args(w.lm_head, self.xn, K.EPI_ARGMAX, counter=ctr[3:4], out=self.logits,
                                    argmax_partial=self.argmax_partial, vocab0=w.geom.vocab0,
                                    cur_token=self.cur_token, pos=self.pos, token_ring=self.token_ring,
                                    token_ring_size=self.token_ring.numel(), forced=self.forced,
                                    n_forced=self.n_forced)
        self.head.comm = self._comm()

    # persistent whole-token kernel -------------------------------------------------------------------------------
    def _build_mega(self) -> None:
        """One cooperative launch per token: builds the device-side layer table and the argument block."""
        import ctypes as C
        from ..models.quant import QWeight
        m, w, dev = self.cfg.model, self.w, self.device
        f32 = dict(dtype=torch.float32, device=dev)
        layers = (K.IhbMegaLayer * len(w.layers))()
        # vectors handed from one phase to the next are {fp32 value, tag} pairs: two floats per element, zero = no tag
        self.mega_logits = torch.zeros(max(1, len(w.layers)), 2 * m.n_experts, **f32)
        self.mega_qkv = torch.zeros(2 * (self.nq + 2 * self.nkv) * 128, **f32)
        self.mega_attn = torch.zeros(2 * self.nq * 128, **f32)
        for L, lw in enumerate(w.layers):
            e = layers[L]
            e.wqkv, e.wo, e.wgu, e.wd = K.mat_of(lw.wqkv), K.mat_of(lw.wo), K.mat_of(lw.w_gu), K.mat_of(lw.w_d)
            e.router = lw.router.data_ptr()
            e.in_ln, e.post_ln = lw.in_ln.data_ptr(), lw.post_ln.data_ptr()
            e.q_norm, e.k_norm = lw.q_norm.data_ptr(), lw.k_norm.data_ptr()
            e.k_cache, e.v_cache = self.k_cache[L].data_ptr(), self.v_cache[L].data_ptr()
            e.router_logits = self.mega_logits[L].data_ptr()
            e.sel_idx, e.sel_w = self.sel_idx[L].data_ptr(), self.sel_w[L].data_ptr()
        if w.layers and w.layers[0].router.dtype != torch.bfloat16:
            raise ValueError("the persistent kernel reads the router matrix as bf16")
        raw = bytes(layers)
        self.mega_layers = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(dev)
        a = K.IhbMegaArgs()
        a.layers, a.n_layers = self.mega_layers.data_ptr(), len(w.layers)
        a.wtype = K.W_FP8 if self.fp8 else K.W_BF16
        a.H, a.nq, a.nkv, a.I, a.E = self.H, self.nq, self.nkv, self.I, m.n_experts
        a.top_k, a.renorm, a.max_seq = m.top_k, int(m.norm_topk_prob), self.max_seq
        par = self.cfg.parallel
        a.expert0, a.E_local = w.geom.expert0, w.geom.n_experts_local
        # the attention shard is computed identically on world / tp ranks: the sum over all ranks counts it that often
        a.attn_ar_scale = float(par.tp) / float(max(par.world, 1))
        a.cos_t, a.sin_t, a.eps = self.cos.data_ptr(), self.sin.data_ptr(), m.rms_eps
        a.embed, a.embed_is_bf16 = w.embed.data_ptr(), int(w.embed.dtype == torch.bfloat16)
        a.final_norm, a.lm_head, a.vocab0 = w.final_norm.data_ptr(), K.mat_of(w.lm_head), w.geom.vocab0
        a.logits = self.logits.data_ptr()
        a.cur_token, a.pos = self.cur_token.data_ptr(), self.pos.data_ptr()
        a.token_ring, a.token_ring_size = self.token_ring.data_ptr(), self.token_ring.numel()
        a.forced, a.n_forced = self.forced.data_ptr(), self.n_forced.data_ptr()
        ngrp = (self.nq // self.nkv + 7) // 8
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        a.max_split = env_flag("IHB_MEGA_SPLITS", max(1, min(64, sms // (self.nkv * ngrp))))
        self.mega_attn_part = torch.zeros(self.nq * a.max_split * 132, **f32)
        self.mega_act = torch.zeros(2 * m.top_k * 2 * self.I, **f32)
        self.mega_bar = torch.zeros(8 + self.nkv * ngrp, dtype=torch.int32, device=dev)
        a.qkv, a.attn_part, a.attn, a.act = (self.mega_qkv.data_ptr(), self.mega_attn_part.data_ptr(),
                                             self.mega_attn.data_ptr(), self.mega_act.data_ptr())
        # short contexts on few local heads: per-block partial records merged by the o_proj CTAs (IHB_MEGA_MERGE=0:
        # always the split-and-merge mode of long contexts)
        self.mega_attn_rec = torch.zeros(self.nq * 16 * 66, dtype=torch.int64, device=dev)
        if env_flag("IHB_MEGA_MERGE", 1):
            a.attn_rec = self.mega_attn_rec.data_ptr()
        a.argmax_partial, a.bar, a.err = self.argmax_partial.data_ptr(), self.mega_bar.data_ptr(), self.err.data_ptr()
        a.steps = 1
        # profiling aid on one GPU: every all-reduce slot receives k adds, the traffic of k ranks
        a.ar_loopback = env_flag("IHB_MEGA_LOOPBACK", 0) if par.world == 1 else 0
        # test aid: IHB_MEGA_DELAY="rank:cta:ns" makes one CTA of one rank lag before each all-reduce read
        spec = os.environ.get("IHB_MEGA_DELAY", "")
        if spec:
            r_, c_, ns_ = (int(x) for x in spec.split(":"))
            if r_ == par.rank:
                a.delay_cta, a.delay_ns = c_, ns_
        a.comm = self._comm()
        self.mega_prof = None
        if env_flag("IHB_MEGA_PROF", 0):
            self.mega_prof_n = 10 * len(w.layers) + 8
            self.mega_prof = torch.zeros(2 * self.mega_prof_n + 32 * len(w.layers), dtype=torch.int64, device=dev)
            a.prof, a.prof_n = self.mega_prof.data_ptr(), self.mega_prof_n
        self.mega = a
        self.mega_grid = min(env_flag("IHB_MEGA_GRID", sms), K.mega_max_grid(a), self.argmax_partial.numel())
        if self.mega_grid < 1:
            raise RuntimeError("the persistent decode kernel does not fit on this device")
        self.use_graph = False                   # one launch per token: nothing to capture
        self.n_launches_per_step = 1

    # tensor-core path -------------------------------------------------------------------------------------------
    def _tc_args(self, qw, tiled, x, xscale, mode, epi, rows=None, **kw) -> K.IhbTcDecArgs:
        a = K.IhbTcDecArgs()
        K.tc_dec_fill_weight(a, qw, tiled, rows)
        a.X, a.mode, a.epi, a.err = x.data_ptr(), mode, epi, self.err.data_ptr()
        a.S = env_flag("IHB_TD_S", 0)
        if self.fp8:
            a.xscale = xscale.data_ptr()
        for k, v in kw.items():
            setattr(a, k, v.data_ptr() if isinstance(v, torch.Tensor) else v)
        return a

    def _build_tc(self) -> None:
        """Re-tile every weight for the tensor-core decode kernels (the plain copies are released) and build the
        per-layer argument blocks."""
        m, w, dev = self.cfg.model, self.w, self.device
        from ..models.quant import QWeight
        es = 1 if self.fp8 else 2
        u8 = dict(dtype=torch.uint8, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        H, I, k = self.H, self.I, m.top_k
        nkb_i = (I * es + 127) // 128
        self.xq, self.xs = torch.zeros(H * es, **u8), torch.zeros(H // 128, **f32)
        self.attn_q, self.attn_s = torch.zeros(self.nq * 128 * es, **u8), torch.zeros(self.nq, **f32)
        self.act_q, self.act_s = torch.zeros(k * nkb_i * 128, **u8), torch.zeros(k * nkb_i, **f32)
        self.tile_ctr = torch.zeros(5, 4096, dtype=torch.int32, device=dev)
        # router GEMV: all eight warps of a CTA share one expert row (K split 8) when K allows
        self.router_ks = 8 if (H // 8) % 8 == 0 and H >= 1024 else 1
        self.router_partial = torch.zeros(8 * m.n_experts, **f32)
        tiled_of = {}

        def tiled(qw, reshape=None):
            key = id(qw)
            if key not in tiled_of:
                data = qw.data if reshape is None else qw.data.reshape(*reshape)
                shape = tuple(qw.data.shape)
                tiled_of[key] = K.tile_weight_v2(data)
                if qw.scale is not None:
                    K.kernel_scale(qw)
                # release the plain copy; keep a meta tensor for the shape/dtype queries of the argument builders
                qw.data = torch.empty(shape, dtype=qw.data.dtype, device="meta")
            return tiled_of[key]

        self.layer_args = []
        ctr = self.counters
        parts = 1
        for L, lw in enumerate(w.layers):
            nxt_gamma = w.layers[L + 1].in_ln if L + 1 < len(w.layers) else w.final_norm
            E_l = lw.w_gu.data.shape[0]
            t_qkv, t_o = tiled(lw.wqkv), tiled(lw.wo)
            t_gu, t_d = tiled(lw.w_gu, (E_l, 2, I, H)), tiled(lw.w_d)
            qkv = self._tc_args(lw.wqkv, t_qkv, self.xq, self.xs, K.TC_LINEAR, K.DEC_STORE, out=self.qkv,
                                tile_counters=self.tile_ctr[0])
            oproj = self._tc_args(lw.wo, t_o, self.attn_q, self.attn_s, K.TC_LINEAR, K.DEC_AR_NORM,
                                  tile_counters=self.tile_ctr[1], counter=ctr[0:1], resid=self.resid, gamma=lw.post_ln,
                                  xn_out=self.xn, eps=m.rms_eps, xq=self.xq, xs=self.xs)
            oproj.comm = self._comm()
            router = self._gemv_args(QWeight(lw.router), self.xn, K.EPI_ROUTER, counter=ctr[1:2], ks=self.router_ks,
                                     out=self.router_logits[L], top_k=m.top_k, renorm=int(m.norm_topk_prob),
                                     sel_idx=self.sel_idx[L], sel_w=self.sel_w[L],
                                     router_partial=self.router_partial)
            gu = self._tc_args(lw.w_gu, t_gu, self.xq, self.xs, K.TC_GATEUP, K.DEC_ACT, rows=I,
                               tile_counters=self.tile_ctr[2], expert0=w.geom.expert0, top_k=k,
                               sel_idx=self.sel_idx[L], sel_w=self.sel_w[L], act_q=self.act_q, act_s=self.act_s)
            gu.n_experts = E_l
            dn = self._tc_args(lw.w_d, t_d, self.act_q, self.act_s, K.TC_DOWN, K.DEC_AR_NORM,
                               tile_counters=self.tile_ctr[3], counter=ctr[2:3], expert0=w.geom.expert0, top_k=k,
                               sel_idx=self.sel_idx[L], sel_w=self.sel_w[L], resid=self.resid, gamma=nxt_gamma,
                               xn_out=self.xn, eps=m.rms_eps, xq=self.xq, xs=self.xs)
            dn.comm = self._comm()
            for a in (qkv, oproj, gu, dn):
                parts = max(parts, K.tc_dec_partial_floats(a))
            self.layer_args.append((qkv, oproj, router, gu, dn, lw))
        t_head = tiled(w.lm_head)
        self.head = self._tc_args(w.lm_head, t_head, self.xq, self.xs, K.TC_LINEAR, K.DEC_ARGMAX, out=self.logits,
                                  tile_counters=self.tile_ctr[4], counter=ctr[3:4], argmax_partial=self.argmax_partial,
                                  vocab0=w.geom.vocab0, cur_token=self.cur_token, pos=self.pos,
                                  token_ring=self.token_ring, token_ring_size=self.token_ring.numel(),
                                  forced=self.forced, n_forced=self.n_forced)
        self.head.comm = self._comm()
        parts = max(parts, K.tc_dec_partial_floats(self.head))
        self.tc_partial = torch.zeros(parts, **f32)
        for (qkv, oproj, router, gu, dn, lw) in self.layer_args:
            for a in (qkv, oproj, gu, dn):
                a.partial = self.tc_partial.data_ptr()
        self.head.partial = self.tc_partial.data_ptr()
        self._tiled = tiled_of

    def _enqueue_step_tc(self) -> None:
        m, w, pdl = self.cfg.model, self.w, self.use_pdl
        K.embed_norm(w.embed, self.cur_token, w.layers[0].in_ln, m.rms_eps, self.resid, self.xn, False,
                     self.xq, self.xs, self.fp8)
        fd_ctr = self.counters[8:]
        for L, (qkv, oproj, router, gu, dn, lw) in enumerate(self.layer_args):
            K.tc_decode(qkv, pdl)
            K.qk_norm_rope_kv(self.qkv, self.nq, self.nkv, lw.q_norm, lw.k_norm, m.rms_eps, self.cos, self.sin,
                              self.pos, self.k_cache[L], self.v_cache[L], self.max_seq, pdl)
            K.flash_decode(self.qkv, self.k_cache[L], self.v_cache[L], self.nq, self.nkv, self.max_seq, self.pos,
                           self.nsplit, self.fd_scratch, fd_ctr, self.attn, pdl, self.attn_q, self.attn_s, self.fp8)
            K.tc_decode(oproj, pdl)
            K.gemv(router, pdl)
            K.tc_decode(gu, pdl)
            K.tc_decode(dn, pdl)
        K.tc_decode(self.head, pdl)
        self.n_launches_per_step = 2 + 7 * len(self.layer_args)

    # one token -------------------------------------------------------------------------------------------------
    def _enqueue_step(self) -> None:
        if self.use_tc:
            return self._enqueue_step_tc()
        m, w, pdl = self.cfg.model, self.w, self.use_pdl
        n = 0
        K.embed_norm(w.embed, self.cur_token, w.layers[0].in_ln, m.rms_eps, self.resid, self.xn, False)
        n += 1
        fd_ctr = self.counters[8:]
        for L, (qkv, oproj, router, moe, lw) in enumerate(self.layer_args):
            K.gemv(qkv, pdl)
            ks, vs = self.kv_scales(L)
            K.qk_norm_rope_kv(self.qkv, self.nq, self.nkv, lw.q_norm, lw.k_norm, m.rms_eps, self.cos, self.sin,
                              self.pos, self.k_cache[L], self.v_cache[L], self.max_seq, pdl, k_scale=ks, v_scale=vs)
            K.flash_decode(self.qkv, self.k_cache[L], self.v_cache[L], self.nq, self.nkv, self.max_seq, self.pos,
                           self.nsplit, self.fd_scratch, fd_ctr, self.attn, pdl, k_scale=ks, v_scale=vs)
            K.gemv(oproj, pdl)
            K.gemv(router, pdl)
            K.moe_gateup(moe, pdl)
            K.moe_down(moe, pdl)
            n += 7
        K.gemv(self.head, pdl)
        self.n_launches_per_step = n + 1

    def _step(self) -> None:
        if self.use_mega:
            if self.mega_prof is not None:
                self.mega_prof[self.mega_prof_n: 2 * self.mega_prof_n].zero_()          # the latest-CTA stamps are atomic maxima
            K.mega_decode(self.mega, self.mega_grid)
            return
        if not self.use_graph:
            self._enqueue_step()
            return
        if self.graph is None:
            # warm up on a side stream (lazy module loading, attribute calls) and restore the state it advanced
            # (the collective epoch is NOT restored: the peers' arrival counters advanced with it)
            state = (self.pos.clone(), self.cur_token.clone())
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._enqueue_step()
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            self.pos.copy_(state[0]); self.cur_token.copy_(state[1])
            if self.symm is not None:
                self.symm.barrier_host()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._enqueue_step()
            self.pos.copy_(state[0]); self.cur_token.copy_(state[1])
            self.graph = g
        self.graph.replay()

    # public ------------------------------------------------------------------------------------------------------
    @property
    def seq_len(self) -> int:
        return int(self.pos.item())

    def reset(self) -> None:
        self.pos.zero_()
        self.n_forced.zero_()
        self.cur_token.zero_()

    def rollback(self, seq_len: int) -> None:
        self.pos.fill_(seq_len)

    def check_error(self) -> None:
        code = int(self.err.item())
        if code:
            self.err.zero_()
            if self.use_mega:
                self.mega_bar.zero_()          # the grid barrier counters are out of step after an abandoned wait
                if self.symm is None:
                    self.slots.zero_()         # so are the contribution counts of the all-reduce slots
            raise RuntimeError(f"device-side wait gave up: {K.ERR_NAMES.get(code, code)}")

    def prefill(self, toks: torch.Tensor, sampler, return_logits: bool):
        """Prompt processing by replaying the decode step once per prompt token with forced inputs (the
        tensor-core prefill path replaces this for long prompts)."""
        T = toks.shape[0]
        if self.seq_len + T > self.max_seq:
            raise ValueError("KV cache overflow")
        if T >= 2 and self.has_window() and env_flag("IHB_WINDOW_PREFILL", 1):
            # batched prompt processing on the tensor cores
            logits = self.window().forward(toks, commit=True, last_only=True)
            nxt = int(torch.argmax(logits[0])) if sampler.params.greedy else int(sampler.sample(logits[0]))
            self.cur_token.fill_(nxt)
            self.n_forced.zero_()
            return nxt, (logits if return_logits else None)
        start = self.seq_len
        self.forced[start:start + T] = toks.to(torch.int32)
        self.n_forced.fill_(start + T)
        self.cur_token.copy_(self.forced[start:start + 1])
        for _ in range(T):
            self._step()
        self.check_error()
        nxt = int(self.cur_token.item())
        logits = None
        if return_logits or not sampler.params.greedy:
            logits = self._full_logits()[None]
            if not sampler.params.greedy:
                nxt = int(sampler.sample(logits[0]))
                self.cur_token.fill_(nxt)
        return nxt, logits

    def _full_logits(self) -> torch.Tensor:
        local = self.logits[: self.w.geom.vocab_local].clone()
        if self.cfg.parallel.world == 1:
            return local
        return self.comm_ref.gather_logits(local[None], self.cfg.model.vocab, self.w.geom.vocab_chunk)[0]

    def decode_step(self, tok: int, sampler, timed: bool = True, want_routes: bool = True):
        """One token through the public path: the input token goes host->device from pinned memory, the step
        runs (graph replay), the produced token comes back device->host."""
        self._tok_in[0] = tok
        self._ev0.record()
        self.cur_token.copy_(self._tok_in, non_blocking=True)
        self._step()
        self._tok_out.copy_(self._tok_err, non_blocking=True)
        self._ev1.record()
        self._ev1.synchronize()
        seconds = self._ev0.elapsed_time(self._ev1) * 1e-3
        out = int(self._tok_out[0])
        if int(self._tok_out[1]):
            self.check_error()                       # a device-side wait gave up during this step: raises
        if not sampler.params.greedy:
            out = int(sampler.sample(self._full_logits()))
            self.cur_token.fill_(out)
        routes = self.last_routes() if want_routes else []
        return out, seconds, routes

    def _peek_token(self) -> int:
        return int(self.cur_token.item())

    def last_routes(self) -> List[RouteRecord]:
        idx, w = self.sel_idx.cpu(), self.sel_w.cpu()
        return [RouteRecord(L, idx[L].tolist(), w[L].tolist()) for L in range(idx.shape[0])]

    def mega_phase_us(self, which: str = "cta0") -> dict:
        """Per-phase device times (microseconds) of the last token; needs ``IHB_MEGA_PROF=1``. Phases per layer:
        qkv, attention, o_proj (+ all-reduce), norm + router, gate/up, down (+ all-reduce); then head and token
        update. ``which="cta0"``: CTA 0's own stamps; ``which="last"``: the latest stamp of any CTA per phase (the
        difference between the two tables is the spread between CTAs)."""
        if self.mega_prof is None:
            raise RuntimeError("set IHB_MEGA_PROF=1 before building the engine")
        t = self.mega_prof.cpu().numpy().astype("float64")
        if which == "last":
            t0 = t[0]
            t = t[self.mega_prof_n: 2 * self.mega_prof_n].copy()
            t[0] = t0
        else:
            t = t[: self.mega_prof_n]
        d = (t[1:] - t[:-1]) / 1e3
        L = len(self.w.layers)
        names = ["qkv", "attention", "o_proj_ar", "norm_router", "gate_up", "down_ar"]
        out = {n: float(d[i:6 * L:6].mean()) for i, n in enumerate(names)} if L else {}
        if L and which != "last":
            sub = t[6 * L + 4: 6 * L + 4 + 4 * L].reshape(L, 4)
            out["expert_select"] = float((sub[:, 1] - sub[:, 0]).mean() / 1e3)
            out["gate_up_gemv"] = float((sub[:, 2] - sub[:, 1]).mean() / 1e3)
        out["head"] = float(d[6 * L])
        out["token_update"] = float(d[6 * L + 1])
        out["total"] = float((t[6 * L + 2] - t[0]) / 1e3)
        if which != "last" and out["total"] > 0:
            out["sm_mhz"] = float(t[6 * L + 3] / out["total"])          # SM cycles of the launch / its duration
        return out

    def mega_detail_us(self) -> list:
        """Detail stamps of the last CTA (it runs the first attention work item), microseconds relative to the
        first stamp of each layer, averaged over layers 1..; needs ``IHB_MEGA_PROF=1``. Points: 0 item entered,
        1 q / k / v normed, 2 K / V rows in shared memory, 3 scores, 4 softmax + PV, 5 record stored, 6 merge
        staging entered, 8 {m, l} words seen, 9 records combined, 10 staged, 11 o_proj rows pushed, 12 all-reduce
        read + norm done, 13 router logit stored, 14 all logits seen, 15 experts selected, 16 / 17 gate-up GEMV
        starts / ends, 18 phase end, 19 barrier + slot clearing, 20 activations seen, 21 staged, 22 chunk table,
        23 down rows pushed; 25 previous layer's all-reduce read + norm done, 26 QKV rows stored (both precede
        point 0 of the same layer)."""
        if self.mega_prof is None:
            raise RuntimeError("set IHB_MEGA_PROF=1 before building the engine")
        L = len(self.w.layers)
        t = self.mega_prof.cpu().numpy().astype("float64")[2 * self.mega_prof_n:].reshape(L, 32)
        t = t[1:] if L > 1 else t
        rel = (t - t[:, :1]) / 1e3
        return [round(float(x), 2) for x in rel.mean(axis=0)[:30]]

    def op_table(self, reps: int = 20) -> list:
        """Per-kernel device times of the per-op pipelines (``IHB_MEGA=0``): every launch of one decode step is
        bracketed by CUDA events (so launches do not overlap), repeated ``reps`` times. Rows: kernel, launches per
        token, microseconds per launch, microseconds per token, share. The persistent kernel reports its phases
        through ``mega_phase_us`` instead. Reference: the in-binary profiler table of
        kernels/decode_step_tp8.cu:2631-2789. All ranks of a parallel run call this together."""
        if self.use_mega:
            raise RuntimeError("one launch per token: use mega_phase_us() (IHB_MEGA_PROF=1)")
        names = ["embed_norm", "gemv", "tc_decode", "qk_norm_rope_kv", "flash_decode", "moe_gateup", "moe_down"]
        orig = {n: getattr(K, n) for n in names if hasattr(K, n)}
        spans = []

        def wrap(name):
            def f(*a, **kw):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                orig[name](*a, **kw)
                e1.record()
                spans.append((name, e0, e1))
            return f

        state = (self.pos.clone(), self.cur_token.clone())
        try:
            for n in orig:
                setattr(K, n, wrap(n))
            for _ in range(reps):
                self._enqueue_step()
            torch.cuda.synchronize(self.device)
        finally:
            for n, fn in orig.items():
                setattr(K, n, fn)
            self.pos.copy_(state[0]); self.cur_token.copy_(state[1])
        agg = {}
        for name, e0, e1 in spans:
            t, c = agg.get(name, (0.0, 0))
            agg[name] = (t + e0.elapsed_time(e1) * 1e3, c + 1)
        total = sum(t for t, _ in agg.values()) / reps
        rows = [{"kernel": n, "launches_per_token": c // reps, "us_per_launch": t / c, "us_per_token": t / reps,
                 "share": (t / reps) / total if total else 0.0} for n, (t, c) in agg.items()]
        return sorted(rows, key=lambda r: -r["us_per_token"])

    def run_steps(self, n: int, per_launch: int = 1) -> None:
        """Enqueue ``n`` decode steps without any host synchronisation (benchmark loop). ``per_launch`` > 1 (persistent
        kernel, greedy decoding): one cooperative launch produces that many tokens in a row; the kernel feeds its own
        arg-max back and logs the tokens in the token ring."""
        if per_launch > 1 and self.use_mega:
            full, rem = divmod(n, per_launch)
            self.mega.steps = per_launch
            try:
                for _ in range(full):
                    self._step()
            finally:
                self.mega.steps = 1
            n = rem
        for _ in range(n):
            self._step()

    def decode_many(self, n: int, per_launch: int = 8) -> List[int]:
        """``n`` greedy tokens with one host synchronisation at the end; the tokens come from the device token ring."""
        if n > self.token_ring.numel():
            raise ValueError("more tokens than the token ring holds")
        pos0 = self.seq_len
        if pos0 + n > self.max_seq:
            raise ValueError("KV cache overflow")
        self.run_steps(n, per_launch)
        idx = (torch.arange(pos0, pos0 + n, device=self.device) % self.token_ring.numel()).long()
        toks = self.token_ring[idx].tolist()
        self.check_error()
        return toks

    def window(self):
        """Multi-token forward (prompt chunks, verify windows); needs the plain row-major weights, i.e. the
        persistent or the streaming pipeline (tensor-, expert- or hybrid-parallel)."""
        if self._window is None:
            from .gpu_window import GpuWindow
            self._window = GpuWindow(self)
        return self._window

    def kv_scales(self, L: int):
        """(k_scale, v_scale) ``[nkv, max_seq]`` of layer ``L`` for an e4m3 cache, (None, None) for a bf16 cache."""
        if not self.kv_fp8:
            return None, None
        return self.k_scale[L], self.v_scale[L]

    def has_window(self) -> bool:
        return (self.use_mega or not self.use_tc) and bool(env_flag("IHB_WINDOW", 1))

    def logits_for(self, tokens, commit=True, tree_mask=None, positions=None, aux_layers=()):
        """Logits ``[T, V]`` of a window of new tokens: one batched forward on the tensor cores."""
        if not self.has_window():
            raise NotImplementedError("window logits need the persistent or streaming pipeline (plain weight layout)")
        return self.window().forward(tokens, commit=commit, tree_mask=tree_mask, positions=positions,
                                     aux_layers=aux_layers)
