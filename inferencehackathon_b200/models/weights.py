"""Weight containers, sharding geometry, random initialisation and on-disk layouts.

Three sources feed the same per-rank :class:`ModelWeights`:

* a Hugging Face Qwen3-MoE state dict / safetensors directory (tensor names as listed in
  tools/conifer_weight_convert.py:68-96 of the reference),
* the converted per-rank engine layout ``rank{r}/layer{L}/{wqkv,wo,wgate,e{E}_wgu,e{E}_wd}.fp8/.scale`` ...
  (tools/conifer_weight_convert.py:8-19), written and read by :func:`save_engine_layout` /
  :func:`load_engine_layout`,
* random initialisation N(0, 0.02): either a full fp32 state dict on the host (small models, identical across
  parallel layouts) or streamed shard by shard on the device (models too large to materialise unsharded).

The tensor-parallel geometry is the reference's TP layout (kernels/decode_step_tp8.cu:18-41): query heads split
across ranks, KV heads split or replicated when there are fewer KV heads than ranks (here a rank keeps only the
KV heads its own query heads read), o_proj column slice, the expert intermediate dimension split inside every
expert, router replicated, lm_head vocabulary rows split.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import numpy as np
import torch

from ..config import ModelConfig, ParallelConfig, QuantConfig
from .quant import QWeight, quant_block, reblock_scales, store_weight


@dataclass(frozen=True)
class ShardGeometry:
    nq_local: int
    q_head0: int
    nkv_local: int
    kv_head0: int
    inter_local: int
    inter0: int
    expert0: int
    n_experts_local: int
    vocab0: int
    vocab_local: int
    vocab_chunk: int

    @property
    def q_per_kv_local(self) -> int:
        return self.nq_local // self.nkv_local


def shard_geometry(cfg: ModelConfig, par: ParallelConfig) -> ShardGeometry:
    par.validate(cfg)
    t, tp = par.tp_rank, par.tp
    nq_local = cfg.n_q_heads // tp
    q_head0 = t * nq_local
    if tp <= cfg.n_kv_heads:
        nkv_local = cfg.n_kv_heads // tp
        kv_head0 = t * nkv_local
    else:
        nkv_local = 1
        kv_head0 = (t * cfg.n_kv_heads) // tp
    if par.ep > 1:
        n_el = cfg.n_experts // par.ep
        expert0 = par.ep_rank * n_el
        inter_local, inter0 = cfg.moe_inter, 0
    else:
        n_el, expert0 = cfg.n_experts, 0
        inter_local = cfg.moe_inter // tp
        inter0 = t * inter_local
    chunk = math.ceil(cfg.vocab / par.world)
    vocab0 = min(cfg.vocab, par.rank * chunk)
    vocab_local = max(0, min(cfg.vocab, vocab0 + chunk) - vocab0)
    return ShardGeometry(nq_local, q_head0, nkv_local, kv_head0, inter_local, inter0, expert0, n_el,
                         vocab0, vocab_local, chunk)


@dataclass
class LayerWeights:
    in_ln: torch.Tensor
    post_ln: torch.Tensor
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    wqkv: QWeight          # [(nq_l + 2 nkv_l) * hd, H]   rows: Q heads, K heads, V heads
    wo: QWeight            # [H, nq_l * hd]
    router: torch.Tensor   # [E, H]  (never quantised: the router is quantisation-sensitive)
    w_gu: QWeight          # [E_l, 2 * I_l, H]             rows: gate then up
    w_d: QWeight           # [E_l, H, I_l]

    def to(self, device) -> "LayerWeights":
        return LayerWeights(self.in_ln.to(device), self.post_ln.to(device), self.q_norm.to(device),
                            self.k_norm.to(device), self.wqkv.to(device), self.wo.to(device),
                            self.router.to(device), self.w_gu.to(device), self.w_d.to(device))

    def nbytes(self) -> int:
        small = sum(t.numel() * t.element_size() for t in
                    (self.in_ln, self.post_ln, self.q_norm, self.k_norm, self.router))
        return small + self.wqkv.nbytes() + self.wo.nbytes() + self.w_gu.nbytes() + self.w_d.nbytes()


@dataclass
class ModelWeights:
    cfg: ModelConfig
    par: ParallelConfig
    quant: QuantConfig
    geom: ShardGeometry
    embed: torch.Tensor        # [V, H] replicated
    final_norm: torch.Tensor   # [H]
    lm_head: QWeight           # [V_local, H]
    layers: List[LayerWeights] = field(default_factory=list)

    def to(self, device) -> "ModelWeights":
        moved: Dict[int, LayerWeights] = {}
        layers = []
        for lw in self.layers:                      # keep aliasing of repeated layer objects
            if id(lw) not in moved:
                moved[id(lw)] = lw.to(device)
            layers.append(moved[id(lw)])
        return ModelWeights(self.cfg, self.par, self.quant, self.geom, self.embed.to(device),
                            self.final_norm.to(device), self.lm_head.to(device), layers)

    def nbytes(self) -> int:
        seen, n = set(), self.embed.numel() * self.embed.element_size() + self.lm_head.nbytes()
        for lw in self.layers:
            if id(lw) not in seen:
                seen.add(id(lw))
                n += lw.nbytes()
        return n


# --------------------------------------------------------------------------------------------------------------
# Hugging Face names
# --------------------------------------------------------------------------------------------------------------

def hf_layer_prefix(layer: int) -> str:
    return f"model.layers.{layer}."


def random_state_dict(cfg: ModelConfig, seed: int = 0, std: float = 0.02,
                      dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """Full unsharded random-init state dict with Hugging Face names (host memory; small models only)."""
    g = torch.Generator().manual_seed(seed)

    def rn(*shape):
        return (torch.randn(*shape, generator=g, dtype=torch.float32) * std).to(dtype)

    def ln(n):
        return (1.0 + 0.1 * torch.randn(n, generator=g, dtype=torch.float32)).to(dtype)

    H, hd = cfg.hidden, cfg.head_dim
    sd = {"model.embed_tokens.weight": rn(cfg.vocab, H), "model.norm.weight": ln(H)}
    if not cfg.tie_embeddings:
        sd["lm_head.weight"] = rn(cfg.vocab, H)
    for L in range(cfg.n_layers):
        p = hf_layer_prefix(L)
        sd[p + "input_layernorm.weight"] = ln(H)
        sd[p + "post_attention_layernorm.weight"] = ln(H)
        sd[p + "self_attn.q_proj.weight"] = rn(cfg.q_dim, H)
        sd[p + "self_attn.k_proj.weight"] = rn(cfg.kv_dim, H)
        sd[p + "self_attn.v_proj.weight"] = rn(cfg.kv_dim, H)
        sd[p + "self_attn.o_proj.weight"] = rn(H, cfg.q_dim)
        sd[p + "self_attn.q_norm.weight"] = ln(hd)
        sd[p + "self_attn.k_norm.weight"] = ln(hd)
        # a wider router spread than 0.02 so that expert choices are not all near-ties
        sd[p + "mlp.gate.weight"] = rn(cfg.n_experts, H) * 5.0
        for e in range(cfg.n_experts):
            ep = p + f"mlp.experts.{e}."
            sd[ep + "gate_proj.weight"] = rn(cfg.moe_inter, H)
            sd[ep + "up_proj.weight"] = rn(cfg.moe_inter, H)
            sd[ep + "down_proj.weight"] = rn(H, cfg.moe_inter)
    return sd


class DeviceRandomStateDict(dict):
    """The same full random-init state dict as :func:`random_state_dict` in spirit, for models too large to hold
    unsharded: a tensor is generated on ``device`` when it is asked for, from a seed derived from its NAME, and is not
    kept. Every rank and every parallel layout therefore slices the same full tensors, so a tensor-, expert- or
    hybrid-parallel engine holds exactly the weights of the one-GPU engine built from the same seed (which the
    per-rank streams of :func:`random_sharded_weights` do not give)."""

    def __init__(self, cfg: ModelConfig, seed: int = 0, device="cuda", std: float = 0.02):
        super().__init__()
        self.cfg, self.seed, self.device, self.std = cfg, seed, torch.device(device), std
        H, hd = cfg.hidden, cfg.head_dim
        spec = {"model.embed_tokens.weight": ((cfg.vocab, H), "w"), "model.norm.weight": ((H,), "ln")}
        if not cfg.tie_embeddings:
            spec["lm_head.weight"] = ((cfg.vocab, H), "w")
        for L in range(cfg.n_layers):
            p = hf_layer_prefix(L)
            spec[p + "input_layernorm.weight"] = ((H,), "ln")
            spec[p + "post_attention_layernorm.weight"] = ((H,), "ln")
            spec[p + "self_attn.q_proj.weight"] = ((cfg.q_dim, H), "w")
            spec[p + "self_attn.k_proj.weight"] = ((cfg.kv_dim, H), "w")
            spec[p + "self_attn.v_proj.weight"] = ((cfg.kv_dim, H), "w")
            spec[p + "self_attn.o_proj.weight"] = ((H, cfg.q_dim), "w")
            spec[p + "self_attn.q_norm.weight"] = ((hd,), "ln")
            spec[p + "self_attn.k_norm.weight"] = ((hd,), "ln")
            spec[p + "mlp.gate.weight"] = ((cfg.n_experts, H), "router")
            for e in range(cfg.n_experts):
                ep = p + f"mlp.experts.{e}."
                spec[ep + "gate_proj.weight"] = ((cfg.moe_inter, H), "w")
                spec[ep + "up_proj.weight"] = ((cfg.moe_inter, H), "w")
                spec[ep + "down_proj.weight"] = ((H, cfg.moe_inter), "w")
        self._spec = spec

    def __contains__(self, name) -> bool:
        return name in self._spec

    def __len__(self) -> int:
        return len(self._spec)

    def keys(self):
        return self._spec.keys()

    def __getitem__(self, name: str) -> torch.Tensor:
        import zlib
        shape, kind = self._spec[name]
        g = torch.Generator(device=self.device).manual_seed((zlib.crc32(name.encode()) << 20) ^ (self.seed * 1000003 + 17))
        t = torch.randn(*shape, device=self.device, dtype=torch.float32, generator=g)
        if kind == "ln":
            return 1.0 + 0.1 * t
        return t * (self.std * 5.0 if kind == "router" else self.std)


class _Getter:
    """Uniform tensor access over a dict or a safetensors directory; understands HF fp8 checkpoints."""

    def __init__(self, source):
        self._dict = None
        self._handles = {}
        self._index = None
        self._dir = None
        if isinstance(source, dict):
            self._dict = source
        else:
            from safetensors import safe_open  # lazy: only needed for on-disk checkpoints
            self._safe_open = safe_open
            self._dir = str(source)
            idx_path = os.path.join(self._dir, "model.safetensors.index.json")
            if os.path.exists(idx_path):
                with open(idx_path) as f:
                    self._index = json.load(f)["weight_map"]
            else:
                self._index = {}
                for fn in sorted(os.listdir(self._dir)):
                    if fn.endswith(".safetensors"):
                        with safe_open(os.path.join(self._dir, fn), framework="pt", device="cpu") as h:
                            for k in h.keys():
                                self._index[k] = fn

    def has(self, name: str) -> bool:
        return name in (self._dict if self._dict is not None else self._index)

    def get(self, name: str) -> torch.Tensor:
        if self._dict is not None:
            return self._dict[name]
        fn = self._index[name]
        if fn not in self._handles:
            self._handles[fn] = self._safe_open(os.path.join(self._dir, fn), framework="pt", device="cpu")
        return self._handles[fn].get_tensor(name)

    def weight(self, name: str):
        """Returns ``(tensor, scale_or_None)``; scale present for HF block-fp8 checkpoints."""
        w = self.get(name)
        sname = name + "_scale_inv"
        if self.has(sname):
            return w, self.get(sname).float()
        return w, None


def _store_slice(w, scale, row0, rows, k0, K, quant: QuantConfig) -> QWeight:
    """Shard ``[row0:row0+rows, k0:k0+K]`` of a 2-D weight and store it in the engine's format."""
    sub = w[row0:row0 + rows, k0:k0 + K]
    if scale is not None:                                   # already block-fp8 on disk: keep the bytes
        s, rb, kb = reblock_scales(scale, quant.block, quant.block, row0, rows, k0, K)
        if quant.weights == "fp8_block":
            return QWeight(sub.contiguous(), s, rb, kb)
        deq = QWeight(sub.contiguous(), s, rb, kb).dequant()
        return store_weight(deq, quant.weights)
    return store_weight(sub, quant.weights, quant.block, quant.block)


def _cat_q(parts: List[QWeight], dim: int = 0) -> QWeight:
    """Concatenate row-stacked QWeights that share block sizes (rows of each part a multiple of rb)."""
    if parts[0].scale is None:
        return QWeight(torch.cat([p.data for p in parts], dim=dim).contiguous())
    rb = parts[0].rb
    for p in parts:
        if p.rb != rb or p.kb != parts[0].kb:
            raise ValueError("parts with different block sizes")
    return QWeight(torch.cat([p.data for p in parts], dim=dim).contiguous(),
                   torch.cat([p.scale for p in parts], dim=dim).contiguous(), rb, parts[0].kb)


def _common_rb(sizes, block: int) -> int:
    g = block
    for s in sizes:
        g = math.gcd(g, s)
    return g


def shard_state_dict(source, cfg: ModelConfig, par: ParallelConfig, quant: QuantConfig,
                     device="cpu", small_dtype=torch.float32) -> ModelWeights:
    """Build one rank's :class:`ModelWeights` from a full HF-named state dict or safetensors directory."""
    raw = _Getter(source)
    geom = shard_geometry(cfg, par)
    hd, H = cfg.head_dim, cfg.hidden
    I, E = cfg.moe_inter, cfg.n_experts
    suffix_shape = {"q_proj.weight": (cfg.n_q_heads * hd, H), "k_proj.weight": (cfg.n_kv_heads * hd, H),
                    "v_proj.weight": (cfg.n_kv_heads * hd, H), "o_proj.weight": (H, cfg.n_q_heads * hd),
                    "gate_proj.weight": (I, H), "up_proj.weight": (I, H), "down_proj.weight": (H, I),
                    "mlp.gate.weight": (E, H), "input_layernorm.weight": (H,), "post_attention_layernorm.weight": (H,),
                    "q_norm.weight": (hd,), "k_norm.weight": (hd,), "model.norm.weight": (H,),
                    "model.embed_tokens.weight": (cfg.vocab, H), "lm_head.weight": (cfg.vocab, H)}

    def _check(name: str, t: torch.Tensor) -> torch.Tensor:
        # a checkpoint of another architecture fails here, with the tensor's name, not deep inside a concatenation
        for suffix, shape in suffix_shape.items():
            if name.endswith(suffix) and tuple(t.shape) != shape:
                raise ValueError(f"{name}: shape {tuple(t.shape)} in the checkpoint, {shape} for {cfg.name}")
        return t

    class _Checked:
        has = staticmethod(raw.has)

        @staticmethod
        def get(name):
            return _check(name, raw.get(name))

        @staticmethod
        def weight(name):
            w, sc = raw.weight(name)
            return _check(name, w), sc

    get = _Checked
    qr0, qrows = geom.q_head0 * hd, geom.nq_local * hd
    kr0, krows = geom.kv_head0 * hd, geom.nkv_local * hd
    # row-stacked tensors need one block height that divides every part (and shard offsets)
    qkv_rb = _common_rb([qrows, krows, qr0, kr0] if quant.weights == "fp8_block" else [quant.block], quant.block)
    gu_rb = _common_rb([geom.inter_local, geom.inter0] if quant.weights == "fp8_block" else [quant.block],
                       quant.block)
    emb_dtype = torch.float32 if quant.weights == "fp32" else torch.bfloat16

    def stack_rows(items, rb) -> QWeight:
        parts = []
        for (name, r0, rows) in items:
            w, s = get.weight(name)
            q = _store_slice(w, s, r0, rows, 0, w.shape[1], quant)
            if q.scale is not None and q.rb != rb:          # expand scale rows to the common height
                q = QWeight(q.data, q.scale.repeat_interleave(q.rb // rb, dim=-2)[: math.ceil(rows / rb)], rb, q.kb)
            parts.append(q)
        return _cat_q(parts)

    layers = []
    for L in range(cfg.n_layers):
        p = hf_layer_prefix(L)
        wqkv = stack_rows([(p + "self_attn.q_proj.weight", qr0, qrows),
                           (p + "self_attn.k_proj.weight", kr0, krows),
                           (p + "self_attn.v_proj.weight", kr0, krows)], qkv_rb)
        wo_w, wo_s = get.weight(p + "self_attn.o_proj.weight")
        wo = _store_slice(wo_w, wo_s, 0, H, qr0, qrows, quant)
        gus, ds = [], []
        for e in range(geom.expert0, geom.expert0 + geom.n_experts_local):
            ep = p + f"mlp.experts.{e}."
            gus.append(stack_rows([(ep + "gate_proj.weight", geom.inter0, geom.inter_local),
                                   (ep + "up_proj.weight", geom.inter0, geom.inter_local)], gu_rb))
            dw, dsc = get.weight(ep + "down_proj.weight")
            ds.append(_store_slice(dw, dsc, 0, H, geom.inter0, geom.inter_local, quant))
        w_gu = QWeight(torch.stack([g.data for g in gus]),
                       None if gus[0].scale is None else torch.stack([g.scale for g in gus]), gus[0].rb, gus[0].kb)
        w_d = QWeight(torch.stack([d.data for d in ds]),
                      None if ds[0].scale is None else torch.stack([d.scale for d in ds]), ds[0].rb, ds[0].kb)
        layers.append(LayerWeights(
            in_ln=get.get(p + "input_layernorm.weight").to(small_dtype),
            post_ln=get.get(p + "post_attention_layernorm.weight").to(small_dtype),
            q_norm=get.get(p + "self_attn.q_norm.weight").to(small_dtype),
            k_norm=get.get(p + "self_attn.k_norm.weight").to(small_dtype),
            wqkv=wqkv, wo=wo,
            router=get.get(p + "mlp.gate.weight").to(emb_dtype if emb_dtype == torch.float32 else torch.bfloat16),
            w_gu=w_gu, w_d=w_d).to(device))
    embed = get.get("model.embed_tokens.weight").to(emb_dtype)
    head_name = "lm_head.weight" if get.has("lm_head.weight") else "model.embed_tokens.weight"
    hw, hs = get.weight(head_name)
    lm_head = _store_slice(hw, hs, geom.vocab0, geom.vocab_local, 0, H, quant)
    return ModelWeights(cfg, par, quant, geom, embed.to(device), get.get("model.norm.weight").to(small_dtype).to(device),
                        lm_head.to(device), layers)


# --------------------------------------------------------------------------------------------------------------
# Streaming random initialisation on the device (large models)
# --------------------------------------------------------------------------------------------------------------

def _rand_weight(shape, quant: QuantConfig, device, gen, std=0.02, chunk_elems=1 << 27) -> QWeight:
    """Random N(0, std) weight of ``shape`` stored per ``quant`` without materialising more than
    ``chunk_elems`` fp32 elements at a time (chunks run over the leading dimension)."""
    shape = tuple(shape)
    lead = shape[0]
    per = int(np.prod(shape[1:]))
    step = max(1, min(lead, chunk_elems // max(per, 1)))
    if quant.weights == "fp8_block" and len(shape) == 2:
        step = max(quant.block, (step // quant.block) * quant.block)      # whole row blocks per chunk
    datas, scales = [], []
    for i in range(0, lead, step):
        n = min(step, lead - i)
        w = torch.randn((n,) + shape[1:], device=device, dtype=torch.float32, generator=gen) * std
        q = store_weight(w, quant.weights, quant.block, quant.block)
        datas.append(q.data)
        if q.scale is not None:
            scales.append(q.scale)
        del w
    data = datas[0] if len(datas) == 1 else torch.cat(datas, dim=0)
    scale = None
    if scales:
        scale = scales[0] if len(scales) == 1 else torch.cat(scales, dim=0)
    return QWeight(data, scale, quant.block, quant.block)


def random_sharded_weights(cfg: ModelConfig, par: ParallelConfig, quant: QuantConfig, device,
                           seed: int = 0, distinct_layers: int = 0,
                           progress: Optional[Callable[[int], None]] = None) -> ModelWeights:
    """Random-init one rank's shard directly on ``device``.

    Replicated tensors (embedding, norms, router) use a seed shared by all ranks so that every rank holds the
    same values; sharded tensors use a per-rank seed. With ``distinct_layers = D > 0`` only ``D`` layer weight
    sets are created and layer ``L`` uses set ``L % D``: the full depth is executed and every layer's weights
    still stream from HBM (``D`` sets are far larger than L2), which is how a model larger than the GPU memory
    is timed on one GPU.
    """
    geom = shard_geometry(cfg, par)
    dev = torch.device(device)
    g_rep = torch.Generator(device=dev).manual_seed(seed)
    g_loc = torch.Generator(device=dev).manual_seed(seed * 1000003 + 17 + par.rank)
    H, hd = cfg.hidden, cfg.head_dim
    emb_dtype = torch.float32 if quant.weights == "fp32" else torch.bfloat16

    def ln(n):
        return 1.0 + 0.1 * torch.randn(n, device=dev, dtype=torch.float32, generator=g_rep)

    embed = (torch.randn(cfg.vocab, H, device=dev, dtype=torch.float32, generator=g_rep) * 0.02).to(emb_dtype) \
        if cfg.vocab * H <= (1 << 28) else torch.cat([
            (torch.randn(min(1 << 15, cfg.vocab - i), H, device=dev, dtype=torch.float32, generator=g_rep) * 0.02)
            .to(emb_dtype) for i in range(0, cfg.vocab, 1 << 15)])
    n_sets = cfg.n_layers if distinct_layers <= 0 else min(distinct_layers, cfg.n_layers)
    sets = []
    qkv_rows = (geom.nq_local + 2 * geom.nkv_local) * hd
    for L in range(n_sets):
        router = (torch.randn(cfg.n_experts, H, device=dev, dtype=torch.float32, generator=g_rep) * 0.1).to(emb_dtype)
        sets.append(LayerWeights(
            in_ln=ln(H), post_ln=ln(H), q_norm=ln(hd), k_norm=ln(hd),
            wqkv=_rand_weight((qkv_rows, H), quant, dev, g_loc),
            wo=_rand_weight((H, geom.nq_local * hd), quant, dev, g_loc),
            router=router,
            w_gu=_rand_weight((geom.n_experts_local, 2 * geom.inter_local, H), quant, dev, g_loc),
            w_d=_rand_weight((geom.n_experts_local, H, geom.inter_local), quant, dev, g_loc)))
        if progress is not None:
            progress(L)
    layers = [sets[L % n_sets] for L in range(cfg.n_layers)]
    lm_head = _rand_weight((geom.vocab_local, H), quant, dev, g_loc)
    return ModelWeights(cfg, par, quant, geom, embed, ln(H), lm_head, layers)


# --------------------------------------------------------------------------------------------------------------
# Converted engine layout on disk
# --------------------------------------------------------------------------------------------------------------

def _dump(t: torch.Tensor, path: str) -> None:
    a = t.detach().cpu().contiguous()
    if a.dtype in (torch.bfloat16, torch.float8_e4m3fn):
        a = a.view(torch.uint8 if a.dtype == torch.float8_e4m3fn else torch.int16)
    a.numpy().tofile(path)


def _dump_q(w: QWeight, base: str) -> Dict:
    if w.scale is not None:
        _dump(w.data, base + ".fp8")
        _dump(w.scale, base + ".scale")
        return {"fmt": "fp8", "shape": list(w.data.shape), "rb": w.rb, "kb": w.kb, "sshape": list(w.scale.shape)}
    ext = ".bf16" if w.data.dtype == torch.bfloat16 else ".f32"
    _dump(w.data, base + ext)
    return {"fmt": ext[1:], "shape": list(w.data.shape)}


def save_engine_layout(w: ModelWeights, out_dir: str) -> str:
    """Write one rank's weights under ``out_dir/rank{r}/`` in the converted layout (file names as in
    tools/conifer_weight_convert.py:8-19; scales here are block scales and a ``manifest.json`` records shapes)."""
    rd = os.path.join(out_dir, f"rank{w.par.rank}")
    os.makedirs(rd, exist_ok=True)
    man: Dict = {"model": w.cfg.name, "tp": w.par.tp, "ep": w.par.ep, "world": w.par.world,
                 "quant": w.quant.weights, "layers": {}}
    _dump(w.embed, os.path.join(rd, "embed.bf16" if w.embed.dtype == torch.bfloat16 else "embed.f32"))
    man["embed"] = {"fmt": "bf16" if w.embed.dtype == torch.bfloat16 else "f32", "shape": list(w.embed.shape)}
    _dump(w.final_norm.float(), os.path.join(rd, "norm_final.f32"))
    man["lm_head"] = _dump_q(w.lm_head, os.path.join(rd, "lm_head"))
    for L, lw in enumerate(w.layers):
        ld = os.path.join(rd, f"layer{L}")
        os.makedirs(ld, exist_ok=True)
        for nm, t in (("in_ln", lw.in_ln), ("post_ln", lw.post_ln), ("q_norm", lw.q_norm), ("k_norm", lw.k_norm)):
            _dump(t.float(), os.path.join(ld, nm + ".f32"))
        ent = {"wqkv": _dump_q(lw.wqkv, os.path.join(ld, "wqkv")), "wo": _dump_q(lw.wo, os.path.join(ld, "wo"))}
        _dump(lw.router.float(), os.path.join(ld, "wgate.f32"))
        ent["wgate"] = {"fmt": "f32", "shape": list(lw.router.shape)}
        for e in range(lw.w_gu.data.shape[0]):
            E = w.geom.expert0 + e
            ent[f"e{E}_wgu"] = _dump_q(lw.w_gu.select(e), os.path.join(ld, f"e{E}_wgu"))
            ent[f"e{E}_wd"] = _dump_q(lw.w_d.select(e), os.path.join(ld, f"e{E}_wd"))
        man["layers"][str(L)] = ent
    with open(os.path.join(rd, "manifest.json"), "w") as f:
        json.dump(man, f)
    return rd


def _load(path_base: str, ent: Dict) -> QWeight:
    shape = ent["shape"]
    if ent["fmt"] == "fp8":
        q = torch.from_numpy(np.fromfile(path_base + ".fp8", dtype=np.uint8)).view(torch.float8_e4m3fn).reshape(shape)
        s = torch.from_numpy(np.fromfile(path_base + ".scale", dtype=np.float32)).reshape(ent["sshape"])
        return QWeight(q, s, ent["rb"], ent["kb"])
    if ent["fmt"] == "bf16":
        return QWeight(torch.from_numpy(np.fromfile(path_base + ".bf16", dtype=np.int16)).view(torch.bfloat16).reshape(shape))
    return QWeight(torch.from_numpy(np.fromfile(path_base + ".f32", dtype=np.float32)).reshape(shape))


def _next_pow2(n: int) -> int:
    p = 16
    while p < n:
        p *= 2
    return p


def _load_rowwise(path_base: str, rows: int, K: int) -> QWeight:
    """A matrix written by the reference's converter: e4m3 bytes ``[rows, K]`` and ONE fp32 scale per row. As a block
    scale that is a block of 1 row x the whole K range (the K block width is the next power of two, which the kernels'
    shift arithmetic needs and which changes nothing: there is one block along K)."""
    q = torch.from_numpy(np.fromfile(path_base + ".fp8", dtype=np.uint8)).view(torch.float8_e4m3fn).reshape(rows, K)
    s = torch.from_numpy(np.fromfile(path_base + ".scale", dtype=np.float32)).reshape(rows, 1)
    return QWeight(q, s.contiguous(), 1, _next_pow2(K))


def load_reference_layout(rd: str, cfg: ModelConfig, par: ParallelConfig, quant: QuantConfig, device="cpu") -> ModelWeights:
    """One rank directory written by the reference's own converter (tools/conifer_weight_convert.py:8-19,65-99):
    no manifest, tensor parallel only, per-ROW fp8 scales, the router as ``wgate.fp8`` + ``.scale``, and a QKV matrix
    that stacks this rank's query heads on ALL key and value heads (the reference replicates K / V on every rank).
    Shapes follow from the model and the rank; the K / V heads this rank attends with are cut out of the replicated
    rows; the router is de-quantised (this engine never multiplies a quantised router)."""
    if par.ep > 1:
        raise ValueError("the reference's converted layout is tensor parallel only")
    geom = shard_geometry(cfg, par)
    hd, H, tp = cfg.head_dim, cfg.hidden, par.tp
    nq_l = cfg.n_q_heads // tp
    I_l = cfg.moe_inter // tp
    voc_l = cfg.vocab // tp
    if cfg.vocab % tp or geom.vocab_local != voc_l:
        raise ValueError("the reference's layout shards the vocabulary evenly")

    def f32(path, n):
        return torch.from_numpy(np.fromfile(path, dtype=np.float32)).reshape(n)

    def store(qw: QWeight) -> QWeight:
        return qw if quant.weights == "fp8_block" else store_weight(qw.dequant(), quant.weights)

    epath = os.path.join(rd, "embed.bf16")
    if not os.path.exists(epath):                                  # the reference writes the table for rank 0 only
        epath = os.path.join(os.path.dirname(rd), "rank0", "embed.bf16")
    embed = torch.from_numpy(np.fromfile(epath, dtype=np.int16)).view(torch.bfloat16).reshape(cfg.vocab, H)
    layers = []
    for L in range(cfg.n_layers):
        ld = os.path.join(rd, f"layer{L}")
        full = _load_rowwise(os.path.join(ld, "wqkv"), (nq_l + 2 * cfg.n_kv_heads) * hd, H)
        k0 = nq_l * hd + geom.kv_head0 * hd
        v0 = nq_l * hd + cfg.n_kv_heads * hd + geom.kv_head0 * hd
        nkv = geom.nkv_local * hd
        rows = torch.cat([torch.arange(0, nq_l * hd), torch.arange(k0, k0 + nkv), torch.arange(v0, v0 + nkv)])
        wqkv = QWeight(full.data[rows].contiguous(), full.scale[rows].contiguous(), 1, full.kb)
        gate = _load_rowwise(os.path.join(ld, "wgate"), cfg.n_experts, H).dequant()
        gus = [_load_rowwise(os.path.join(ld, f"e{E}_wgu"), 2 * I_l, H) for E in range(cfg.n_experts)]
        dsl = [_load_rowwise(os.path.join(ld, f"e{E}_wd"), H, I_l) for E in range(cfg.n_experts)]
        stack = lambda qs: QWeight(torch.stack([q.data for q in qs]), torch.stack([q.scale for q in qs]), qs[0].rb, qs[0].kb)
        layers.append(LayerWeights(
            in_ln=f32(os.path.join(ld, "in_ln.f32"), H), post_ln=f32(os.path.join(ld, "post_ln.f32"), H),
            q_norm=f32(os.path.join(ld, "q_norm.f32"), hd), k_norm=f32(os.path.join(ld, "k_norm.f32"), hd),
            wqkv=store(wqkv), wo=store(_load_rowwise(os.path.join(ld, "wo"), H, nq_l * hd)),
            router=gate if quant.weights == "fp32" else gate.to(torch.bfloat16),
            w_gu=store(stack(gus)), w_d=store(stack(dsl))).to(device))
    lm = store(_load_rowwise(os.path.join(rd, "lm_head"), voc_l, H))
    small = torch.float32 if quant.weights == "fp32" else torch.bfloat16
    return ModelWeights(cfg, par, quant, geom, embed.to(small).to(device), f32(os.path.join(rd, "norm_final.f32"), H).to(device),
                        lm.to(device), layers)


def load_engine_layout(in_dir: str, cfg: ModelConfig, par: ParallelConfig, quant: QuantConfig,
                       device="cpu") -> ModelWeights:
    """One rank's weights from the converted on-disk layout: this package's (with ``manifest.json``), or, when the rank
    directory has no manifest, the reference converter's (see :func:`load_reference_layout`)."""
    rd = os.path.join(in_dir, f"rank{par.rank}")
    if not os.path.exists(os.path.join(rd, "manifest.json")):
        return load_reference_layout(rd, cfg, par, quant, device)
    with open(os.path.join(rd, "manifest.json")) as f:
        man = json.load(f)
    geom = shard_geometry(cfg, par)

    def f32(path, n):
        return torch.from_numpy(np.fromfile(path, dtype=np.float32)).reshape(n)

    embed = _load(os.path.join(rd, "embed"), man["embed"]).data
    layers = []
    for L in range(cfg.n_layers):
        ld = os.path.join(rd, f"layer{L}")
        ent = man["layers"][str(L)]
        gus = [_load(os.path.join(ld, f"e{E}_wgu"), ent[f"e{E}_wgu"])
               for E in range(geom.expert0, geom.expert0 + geom.n_experts_local)]
        dsl = [_load(os.path.join(ld, f"e{E}_wd"), ent[f"e{E}_wd"])
               for E in range(geom.expert0, geom.expert0 + geom.n_experts_local)]
        stack = lambda qs: QWeight(torch.stack([q.data for q in qs]),
                                   None if qs[0].scale is None else torch.stack([q.scale for q in qs]),
                                   qs[0].rb, qs[0].kb)
        router = f32(os.path.join(ld, "wgate.f32"), ent["wgate"]["shape"])
        layers.append(LayerWeights(
            in_ln=f32(os.path.join(ld, "in_ln.f32"), cfg.hidden), post_ln=f32(os.path.join(ld, "post_ln.f32"), cfg.hidden),
            q_norm=f32(os.path.join(ld, "q_norm.f32"), cfg.head_dim), k_norm=f32(os.path.join(ld, "k_norm.f32"), cfg.head_dim),
            wqkv=_load(os.path.join(ld, "wqkv"), ent["wqkv"]), wo=_load(os.path.join(ld, "wo"), ent["wo"]),
            router=router if quant.weights == "fp32" else router.to(torch.bfloat16),
            w_gu=stack(gus), w_d=stack(dsl)).to(device))
    return ModelWeights(cfg, par, quant, geom, embed.to(device), f32(os.path.join(rd, "norm_final.f32"), cfg.hidden).to(device),
                        _load(os.path.join(rd, "lm_head"), man["lm_head"]).to(device), layers)
