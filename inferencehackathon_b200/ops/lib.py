"""ctypes bindings of the sm_100a kernel library (``libihb_kernels.so``, built in-tree by :mod:`.build`).

The structures mirror ``csrc/kernels/api.h`` field by field. Launches go to ``torch.cuda.current_stream()`` so
that they are captured by ``torch.cuda.graph``. The library is required on a GPU machine: a missing or
unloadable ``.so`` raises instead of falling back to PyTorch ops.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from . import build as _build

MAX_RANKS = 8
W_FP8, W_BF16 = 0, 1
EPI_STORE, EPI_ROUTER, EPI_ARGMAX, EPI_AR_NORM = 0, 1, 2, 3

ERR_NAMES = {0: "none", 1: "pipeline full-barrier time-out", 2: "pipeline empty-barrier time-out",
             3: "peer barrier time-out", 4: "grid counter time-out", 5: "tensor-memory time-out", 6: "bad arguments"}

_vp = C.c_void_p


class IhbComm(C.Structure):
    _fields_ = [("nranks", C.c_int), ("rank", C.c_int),
                ("slots_local", _vp), ("slots_mc", _vp), ("slots_peer", _vp * MAX_RANKS),
                ("flag_local", _vp), ("flag_mc", _vp), ("flag_peer", _vp * MAX_RANKS),
                ("arg_slots_local", _vp), ("arg_slots_mc", _vp), ("arg_slots_peer", _vp * MAX_RANKS),
                ("epoch", _vp)]


class IhbA2AArgs(C.Structure):
    _fields_ = [("nranks", C.c_int), ("rank", C.c_int), ("row_floats", C.c_int), ("cap", C.c_int), ("round", C.c_uint),
                ("send", _vp), ("gather", _vp), ("offsets", _vp),
                ("recv_peer", _vp * MAX_RANKS), ("count_peer", _vp * MAX_RANKS), ("flag_peer", _vp * MAX_RANKS),
                ("flag_local", _vp), ("err", _vp)]


class IhbGemvArgs(C.Structure):
    _fields_ = [("W", _vp), ("wscale", _vp), ("wtype", C.c_int), ("rows", C.c_int), ("K", C.c_int),
                ("rb", C.c_int), ("kb_shift", C.c_int), ("nkb", C.c_int),
                ("x", _vp),
                ("R", C.c_int), ("S", C.c_int), ("grid", C.c_int), ("ks", C.c_int), ("epi", C.c_int),
                ("out", _vp), ("counter", _vp), ("err", _vp),
                ("top_k", C.c_int), ("renorm", C.c_int), ("sel_idx", _vp), ("sel_w", _vp), ("router_partial", _vp),
                ("argmax_partial", _vp), ("vocab0", C.c_int), ("cur_token", _vp), ("pos", _vp),
                ("token_ring", _vp), ("token_ring_size", C.c_int), ("forced", _vp), ("n_forced", _vp),
                ("resid", _vp), ("gamma", _vp), ("xn_out", _vp), ("eps", C.c_float),
                ("comm", IhbComm)]


class IhbMoeArgs(C.Structure):
    _fields_ = [("Wgu", _vp), ("gu_scale", _vp), ("Wd", _vp), ("d_scale", _vp), ("wtype", C.c_int),
                ("H", C.c_int), ("I", C.c_int), ("E_local", C.c_int), ("expert0", C.c_int), ("top_k", C.c_int),
                ("gu_rb", C.c_int), ("gu_kb_shift", C.c_int), ("gu_nkb", C.c_int),
                ("d_rb", C.c_int), ("d_kb_shift", C.c_int), ("d_nkb", C.c_int),
                ("x", _vp), ("sel_idx", _vp), ("sel_w", _vp), ("act", _vp),
                ("R_gu", C.c_int), ("R_d", C.c_int), ("S", C.c_int), ("grid", C.c_int),
                ("counter", _vp), ("err", _vp),
                ("resid", _vp), ("gamma", _vp), ("xn_out", _vp), ("eps", C.c_float),
                ("comm", IhbComm)]


TC_LINEAR, TC_GATEUP, TC_DOWN = 0, 1, 2
ARC_MAX_ROWS = 64          # IHB_ARC_MAX_ROWS: rows of the counted small-message all-reduce


class IhbTcArgs(C.Structure):
    _fields_ = [("W", _vp), ("wscale", _vp), ("wtype", C.c_int), ("rows", C.c_int), ("K", C.c_int),
                ("rb", C.c_int), ("nrb", C.c_int), ("nkb_stride", C.c_int),
                ("n_experts", C.c_int), ("expert0", C.c_int), ("top_k", C.c_int),
                ("X", _vp), ("xscale", _vp), ("T", C.c_int), ("T_total", C.c_int), ("tok0", C.c_int),
                ("mode", C.c_int), ("sel_idx", _vp), ("sel_w", _vp),
                ("out", _vp), ("out_stride", C.c_int), ("partial", _vp), ("tile_counters", _vp),
                ("ks", C.c_int), ("S", C.c_int), ("grid", C.c_int), ("n_units", C.c_int), ("err", _vp),
                ("tiled", C.c_int), ("x_rows1", C.c_int),
                ("groups", _vp), ("n_groups", _vp), ("max_groups", C.c_int),
                ("tok_tiles", C.c_int), ("tok_tile", C.c_int)]


DEC_STORE, DEC_AR_NORM, DEC_ARGMAX, DEC_ACT = 0, 1, 2, 3


class IhbTcDecArgs(C.Structure):
    _fields_ = [("W", _vp), ("wscale", _vp), ("wtype", C.c_int), ("rows", C.c_int), ("K", C.c_int),
                ("rb", C.c_int), ("nrb", C.c_int), ("nkb_stride", C.c_int),
                ("n_experts", C.c_int), ("expert0", C.c_int), ("top_k", C.c_int),
                ("X", _vp), ("xscale", _vp), ("mode", C.c_int), ("epi", C.c_int),
                ("sel_idx", _vp), ("sel_w", _vp), ("out", _vp), ("act_q", _vp), ("act_s", _vp),
                ("partial", _vp), ("tile_counters", _vp),
                ("ks", C.c_int), ("S", C.c_int), ("grid", C.c_int), ("n_units", C.c_int),
                ("counter", _vp), ("err", _vp),
                ("argmax_partial", _vp), ("vocab0", C.c_int), ("cur_token", _vp), ("pos", _vp),
                ("token_ring", _vp), ("token_ring_size", C.c_int), ("forced", _vp), ("n_forced", _vp),
                ("resid", _vp), ("gamma", _vp), ("xn_out", _vp), ("eps", C.c_float), ("xq", _vp), ("xs", _vp),
                ("comm", IhbComm)]


_lib: Optional[C.CDLL] = None


class IhbMat(C.Structure):
    _fields_ = [("W", _vp), ("wscale", _vp), ("rows", C.c_int), ("K", C.c_int),
                ("rb", C.c_int), ("kb_shift", C.c_int), ("nkb", C.c_int)]


class IhbMegaLayer(C.Structure):
    _fields_ = [("wqkv", IhbMat), ("wo", IhbMat), ("wgu", IhbMat), ("wd", IhbMat), ("router", _vp),
                ("in_ln", _vp), ("post_ln", _vp), ("q_norm", _vp), ("k_norm", _vp),
                ("k_cache", _vp), ("v_cache", _vp), ("router_logits", _vp), ("sel_idx", _vp), ("sel_w", _vp)]


class IhbMegaArgs(C.Structure):
    _fields_ = [("layers", _vp), ("n_layers", C.c_int), ("wtype", C.c_int),
                ("H", C.c_int), ("nq", C.c_int), ("nkv", C.c_int), ("I", C.c_int), ("E", C.c_int),
                ("top_k", C.c_int), ("renorm", C.c_int), ("expert0", C.c_int), ("E_local", C.c_int),
                ("attn_ar_scale", C.c_float), ("max_seq", C.c_int),
                ("cos_t", _vp), ("sin_t", _vp), ("eps", C.c_float),
                ("embed", _vp), ("embed_is_bf16", C.c_int), ("final_norm", _vp), ("lm_head", IhbMat),
                ("vocab0", C.c_int), ("logits", _vp), ("cur_token", _vp), ("pos", _vp), ("token_ring", _vp),
                ("token_ring_size", C.c_int), ("forced", _vp), ("n_forced", _vp),
                ("qkv", _vp), ("attn_part", _vp), ("attn", _vp), ("attn_rec", _vp), ("act", _vp), ("argmax_partial", _vp),
                ("bar", _vp), ("err", _vp), ("prof", _vp), ("prof_n", C.c_int), ("max_split", C.c_int), ("steps", C.c_int),
                ("ar_loopback", C.c_int), ("delay_cta", C.c_int), ("delay_ns", C.c_int), ("comm", IhbComm)]


def load(build_if_missing: bool = True) -> C.CDLL:
    """Load (building first if the sources changed and nvcc is present) the kernel library."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.KERNEL_LIB
    if build_if_missing:
        try:
            _build.build_kernels()
        except Exception:
            if not os.path.exists(path):
                raise
    if not os.path.exists(path):
        raise RuntimeError(f"kernel library {path} is missing: run `python -m inferencehackathon_b200.ops.build`")
    lib = C.CDLL(path)
    lib.ihb_gemv.argtypes = [C.POINTER(IhbGemvArgs), C.c_int, _vp]
    lib.ihb_moe_gateup.argtypes = [C.POINTER(IhbMoeArgs), C.c_int, _vp]
    lib.ihb_moe_down.argtypes = [C.POINTER(IhbMoeArgs), C.c_int, _vp]
    lib.ihb_embed_norm.argtypes = [_vp, C.c_int, _vp, C.c_int, _vp, C.c_float, _vp, _vp, _vp, _vp, C.c_int, C.c_int, _vp]
    lib.ihb_qk_norm_rope_kv.argtypes = [_vp, C.c_int, C.c_int, _vp, _vp, C.c_float, _vp, _vp, _vp, _vp, _vp,
                                        C.c_int, C.c_int, _vp]
    lib.ihb_flash_decode.argtypes = [_vp, _vp, _vp, C.c_int, C.c_int, C.c_int, _vp, C.c_int, _vp, _vp, _vp,
                                     _vp, _vp, C.c_int, C.c_int, _vp]
    lib.ihb_qk_norm_rope_kv8.argtypes = [_vp, C.c_int, C.c_int, _vp, _vp, C.c_float, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                         C.c_int, C.c_int, _vp]
    lib.ihb_flash_decode_kv8.argtypes = [_vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, _vp, C.c_int, _vp, _vp, _vp,
                                         _vp, _vp, C.c_int, C.c_int, _vp]
    lib.ihb_flash_decode_scratch_floats.argtypes = [C.c_int, C.c_int]
    lib.ihb_flash_decode_scratch_floats.restype = C.c_size_t
    lib.ihb_tc_gemm.argtypes = [C.POINTER(IhbTcArgs), C.c_int, _vp]
    lib.ihb_tc_gemm.restype = C.c_int
    lib.ihb_tc_partial_floats.argtypes = [C.POINTER(IhbTcArgs)]
    lib.ihb_tc_partial_floats.restype = C.c_size_t
    lib.ihb_tc_decode.argtypes = [C.POINTER(IhbTcDecArgs), C.c_int, _vp]
    lib.ihb_tc_decode.restype = C.c_int
    lib.ihb_tc_dec_partial_floats.argtypes = [C.POINTER(IhbTcDecArgs)]
    lib.ihb_tc_dec_partial_floats.restype = C.c_size_t
    lib.ihb_norm_quant_rows.argtypes = [_vp, _vp, C.c_float, C.c_int, C.c_int, _vp, _vp, _vp, C.c_int, _vp]
    lib.ihb_norm_quant_rows.restype = C.c_int
    lib.ihb_qk_norm_rope_rows.argtypes = [_vp, C.c_int, C.c_int, _vp, _vp, C.c_float, _vp, _vp, _vp, _vp, _vp, _vp,
                                          C.c_int, C.c_int, _vp]
    lib.ihb_qk_norm_rope_rows.restype = C.c_int
    lib.ihb_window_attention.argtypes = [_vp, C.c_int, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp, C.c_int, _vp,
                                         _vp]
    lib.ihb_window_attention.restype = C.c_int
    lib.ihb_qk_norm_rope_rows_kv8.argtypes = [_vp, C.c_int, C.c_int, _vp, _vp, C.c_float, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                              C.c_int, C.c_int, _vp]
    lib.ihb_qk_norm_rope_rows_kv8.restype = C.c_int
    lib.ihb_window_attention_kv8.argtypes = [_vp, C.c_int, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp,
                                             _vp, _vp, _vp]
    lib.ihb_window_attention_kv8.restype = C.c_int
    lib.ihb_window_attention_splits.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int]
    lib.ihb_window_attention_splits.restype = C.c_int
    lib.ihb_window_attention_scratch_floats.argtypes = [C.c_int, C.c_int, C.c_int]
    lib.ihb_window_attention_scratch_floats.restype = C.c_size_t
    lib.ihb_a2a_rows.argtypes = [C.POINTER(IhbA2AArgs), C.c_int, _vp]
    lib.ihb_a2a_rows.restype = C.c_int
    lib.ihb_allreduce_norm.argtypes = [C.POINTER(IhbComm), _vp, _vp, _vp, C.c_float, C.c_int, C.c_int, _vp, _vp, _vp, _vp, _vp,
                                       C.c_int, C.c_int, _vp]
    lib.ihb_allreduce_norm.restype = C.c_int
    lib.ihb_router_topk_rows.argtypes = [_vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp, _vp]
    lib.ihb_router_topk_rows.restype = C.c_int
    lib.ihb_clear_last_error.restype = C.c_int
    lib.ihb_moe_group_table.argtypes = [_vp, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp, _vp, C.c_int, _vp]
    lib.ihb_moe_group_table.restype = C.c_int
    lib.ihb_moe_gather_rows.argtypes = [_vp, _vp, C.c_int, C.c_int, C.c_int, _vp, _vp]
    lib.ihb_moe_gather_rows.restype = C.c_int
    lib.ihb_moe_combine_rows.argtypes = [_vp, _vp, _vp, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp]
    lib.ihb_moe_combine_rows.restype = C.c_int
    lib.ihb_allreduce_counted.argtypes = [C.POINTER(IhbComm), _vp, C.c_int, _vp, _vp, C.c_float, C.c_int, C.c_int, _vp, _vp, _vp, _vp,
                                          _vp, _vp, _vp]
    lib.ihb_allreduce_counted.restype = C.c_int
    lib.ihb_dequant_bf16.argtypes = [_vp, _vp, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp]
    lib.ihb_dequant_bf16.restype = C.c_int
    lib.ihb_mega_decode.argtypes = [C.POINTER(IhbMegaArgs), C.c_int, _vp]
    lib.ihb_mega_decode.restype = C.c_int
    lib.ihb_mega_max_grid.argtypes = [C.POINTER(IhbMegaArgs)]
    lib.ihb_mega_max_grid.restype = C.c_int
    for name in ("ihb_gemv", "ihb_moe_gateup", "ihb_moe_down", "ihb_embed_norm", "ihb_qk_norm_rope_kv",
                 "ihb_flash_decode", "ihb_qk_norm_rope_kv8", "ihb_flash_decode_kv8"):
        getattr(lib, name).restype = C.c_int
    _lib = lib
    return lib


def available() -> bool:
    return os.path.exists(_build.KERNEL_LIB)


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(code: int, what: str) -> None:
    if code != 0:
        _lib.ihb_clear_last_error()          # a refused launch must not be reported again by the next entry point
        raise RuntimeError(f"{what}: CUDA error {code}")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def wtype_of(t: torch.Tensor) -> int:
    if t.dtype == torch.float8_e4m3fn:
        return W_FP8
    if t.dtype == torch.bfloat16:
        return W_BF16
    raise TypeError(f"kernel weights must be float8_e4m3fn or bfloat16, got {t.dtype}")


def kb_shift_of(kb: int) -> int:
    s = kb.bit_length() - 1
    if (1 << s) != kb or kb < 16:
        raise ValueError("scale block width must be a power of two >= 16")
    return s


def single_comm(slots: torch.Tensor, epoch: torch.Tensor) -> IhbComm:
    """Comm block for one GPU: the partial lands in a local slot buffer and the tail only adds the residual."""
    cm = IhbComm()
    cm.nranks, cm.rank = 1, 0
    cm.slots_local = slots.data_ptr()
    cm.epoch = epoch.data_ptr()
    return cm


def kernel_scale(qw) -> torch.Tensor:
    """Block scales in the kernels' layout: each scale row padded to a multiple of 4 floats, because scale rows
    travel to shared memory by bulk copy (16-byte granules). Cached on the QWeight."""
    ks = getattr(qw, "_kscale", None)
    if ks is None:
        sc = qw.scale
        pad = (-sc.shape[-1]) % 4
        ks = torch.nn.functional.pad(sc, (0, pad)).contiguous() if pad else sc.contiguous()
        if ks.shape[-1] > 64:
            raise ValueError("at most 64 scale blocks along K")
        qw._kscale = ks
    return ks


def fill_weight(args, qw, prefix: str = "") -> None:
    """Set the weight fields of a GEMV argument block from a QWeight."""
    args.W = qw.data.data_ptr()
    args.wtype = wtype_of(qw.data)
    args.rows, args.K = qw.data.shape[-2], qw.data.shape[-1]
    if qw.scale is not None:
        ks = kernel_scale(qw)
        args.wscale = ks.data_ptr()
        args.rb, args.kb_shift, args.nkb = qw.rb, kb_shift_of(qw.kb), ks.shape[-1]


def gemv(args: IhbGemvArgs, use_pdl: bool = False) -> None:
    check(load().ihb_gemv(C.byref(args), int(use_pdl), stream_ptr()), "ihb_gemv")


def moe_gateup(args: IhbMoeArgs, use_pdl: bool = False) -> None:
    check(load().ihb_moe_gateup(C.byref(args), int(use_pdl), stream_ptr()), "ihb_moe_gateup")


def moe_down(args: IhbMoeArgs, use_pdl: bool = False) -> None:
    check(load().ihb_moe_down(C.byref(args), int(use_pdl), stream_ptr()), "ihb_moe_down")


def embed_norm(embed: torch.Tensor, token: torch.Tensor, gamma: torch.Tensor, eps: float, resid: torch.Tensor,
               xn: torch.Tensor, use_pdl: bool = False, xq: Optional[torch.Tensor] = None,
               xs: Optional[torch.Tensor] = None, xq_fp8: bool = True) -> None:
    check(load().ihb_embed_norm(embed.data_ptr(), int(embed.dtype == torch.bfloat16), token.data_ptr(),
                                embed.shape[1], gamma.data_ptr(), eps, resid.data_ptr(), xn.data_ptr(),
                                ptr(xq), ptr(xs), int(xq_fp8), int(use_pdl), stream_ptr()), "ihb_embed_norm")


def qk_norm_rope_kv(qkv: torch.Tensor, nq: int, nkv: int, q_gamma, k_gamma, eps: float, cos_t, sin_t, pos,
                    k_cache, v_cache, max_seq: int, use_pdl: bool = False,
                    k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None) -> None:
    """``k_scale`` / ``v_scale`` ``[nkv, max_seq]`` fp32: the caches are e4m3 bytes with one scale per row."""
    if k_scale is not None:
        check(load().ihb_qk_norm_rope_kv8(qkv.data_ptr(), nq, nkv, q_gamma.data_ptr(), k_gamma.data_ptr(), eps,
                                          cos_t.data_ptr(), sin_t.data_ptr(), pos.data_ptr(), k_cache.data_ptr(),
                                          v_cache.data_ptr(), k_scale.data_ptr(), v_scale.data_ptr(), max_seq, int(use_pdl),
                                          stream_ptr()), "ihb_qk_norm_rope_kv8")
        return
    check(load().ihb_qk_norm_rope_kv(qkv.data_ptr(), nq, nkv, q_gamma.data_ptr(), k_gamma.data_ptr(), eps,
                                     cos_t.data_ptr(), sin_t.data_ptr(), pos.data_ptr(), k_cache.data_ptr(),
                                     v_cache.data_ptr(), max_seq, int(use_pdl), stream_ptr()),
          "ihb_qk_norm_rope_kv")


def flash_decode_scratch_floats(nq: int, nsplit: int) -> int:
    return int(load().ihb_flash_decode_scratch_floats(nq, nsplit))


def flash_decode(q, k_cache, v_cache, nq: int, nkv: int, max_seq: int, pos, nsplit: int, scratch, counters, out,
                 use_pdl: bool = False, out_q: Optional[torch.Tensor] = None, out_s: Optional[torch.Tensor] = None,
                 out_fp8: bool = True, k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None) -> None:
    if k_scale is not None:                                     # e4m3 cache rows with a scale per row
        check(load().ihb_flash_decode_kv8(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), k_scale.data_ptr(),
                                          v_scale.data_ptr(), nq, nkv, max_seq, pos.data_ptr(), nsplit, scratch.data_ptr(),
                                          counters.data_ptr(), out.data_ptr(), ptr(out_q), ptr(out_s), int(out_fp8),
                                          int(use_pdl), stream_ptr()), "ihb_flash_decode_kv8")
        return
    check(load().ihb_flash_decode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), nq, nkv, max_seq,
                                  pos.data_ptr(), nsplit, scratch.data_ptr(), counters.data_ptr(), out.data_ptr(),
                                  ptr(out_q), ptr(out_s), int(out_fp8), int(use_pdl), stream_ptr()),
          "ihb_flash_decode")


def tc_gemm(args: IhbTcArgs, use_pdl: bool = False) -> None:
    check(load().ihb_tc_gemm(C.byref(args), int(use_pdl), stream_ptr()), "ihb_tc_gemm")


def tc_partial_floats(args: IhbTcArgs) -> int:
    return int(load().ihb_tc_partial_floats(C.byref(args)))


def tc_fill_weight(args: IhbTcArgs, qw) -> None:
    """Weight fields of a tensor-core GEMM block; ``qw.data`` is ``[rows, K]`` or ``[E, rows, K]``
    (gate/up weights: ``[E, 2 * I, K]`` with ``rows = I``, set by the caller)."""
    args.W = qw.data.data_ptr()
    args.wtype = wtype_of(qw.data)
    args.rows, args.K = qw.data.shape[-2], qw.data.shape[-1]
    args.n_experts = qw.data.shape[0] if qw.data.dim() == 3 else 1
    if qw.scale is not None:
        if qw.kb != 128:
            raise ValueError("the tensor-core path needs 128-wide K scale blocks")
        ks = kernel_scale(qw)
        args.wscale = ks.data_ptr()
        args.rb, args.nrb, args.nkb_stride = qw.rb, ks.shape[-2], ks.shape[-1]


def tile_weight(data: torch.Tensor) -> torch.Tensor:
    """Repack ``data[..., rows, K]`` (e4m3 or bf16) into the tensor-core kernels' HBM layout
    ``[..., k block, rows padded to 8, 128 B]`` with the 16-byte chunks of every row XOR-swizzled by
    ``row % 8``: a 128-row tile of one 128-byte K block is then one contiguous 16 KB run that a single bulk
    copy drops into shared memory in exactly the order the MMA's 128-byte-swizzle descriptor expects."""
    *lead, rows, K = data.shape
    raw = data.contiguous().view(torch.uint8).reshape(*lead, rows, -1)
    rowb = raw.shape[-1]
    nkb = (rowb + 127) // 128
    rows_p8 = (rows + 7) // 8 * 8
    raw = torch.nn.functional.pad(raw, (0, nkb * 128 - rowb, 0, rows_p8 - rows))
    v = raw.reshape(*lead, rows_p8 // 8, 8, nkb, 8, 16)                 # [.., grp, r, kb, chunk, 16]
    r = torch.arange(8, device=data.device)
    c = torch.arange(8, device=data.device)
    src_chunk = (c[None, :] ^ r[:, None])                                # dst chunk c of row r holds src chunk c ^ r
    idx = src_chunk[None, :, None, :, None].expand(v.shape[-5], 8, nkb, 8, 16)
    for _ in lead:
        idx = idx[None]
    v = torch.gather(v, -2, idx.expand(v.shape))
    out = v.permute(*range(len(lead)), len(lead) + 2, len(lead), len(lead) + 1, len(lead) + 3, len(lead) + 4)
    return out.contiguous().reshape(*lead, nkb, rows_p8, 128)


def tile_weight_v2(data: torch.Tensor) -> torch.Tensor:
    """Decode-path HBM layout: per matrix ``[row tile][k block][rows of the tile, padded to 8][128 B]`` (swizzled
    as in :func:`tile_weight`), flattened to ``[..., bytes]``. All K blocks of one 128-row tile are contiguous, so
    a stage of several K blocks is a single bulk copy."""
    v1 = tile_weight(data)                                   # [..., nkb, rows_p8, 128]
    rows_p8 = v1.shape[-2]
    lead = v1.shape[:-3]
    parts = []
    for r0 in range(0, rows_p8, 128):
        rt = min(128, rows_p8 - r0)
        parts.append(v1[..., :, r0:r0 + rt, :].reshape(*lead, -1))
    return torch.cat(parts, dim=-1).contiguous()


def act_row(x: torch.Tensor, fp8: bool):
    """Activation vector(s) ``x[..., K]`` (fp32) in the decode kernels' input format: plain rows padded to a
    multiple of 128 bytes, e4m3 with one scale per 128 channels (returns ``(bytes, scales)``) or bf16
    (``(bytes, None)``)."""
    K = x.shape[-1]
    if not fp8:
        raw = x.to(torch.bfloat16).contiguous().view(torch.uint8).reshape(*x.shape[:-1], -1)
        return torch.nn.functional.pad(raw, (0, (-raw.shape[-1]) % 128)).contiguous(), None
    Kp = (K + 127) // 128 * 128
    xp = torch.nn.functional.pad(x.float(), (0, Kp - K)).reshape(*x.shape[:-1], Kp // 128, 128)
    s = xp.abs().amax(dim=-1).clamp_min(1e-12) / 448.0
    q = (xp / s[..., None]).clamp(-448, 448).to(torch.float8_e4m3fn).reshape(*x.shape[:-1], Kp)
    return q.view(torch.uint8).contiguous(), s.contiguous()


def tc_dec_fill_weight(args: IhbTcDecArgs, qw, tiled: torch.Tensor, rows: Optional[int] = None) -> None:
    """Weight fields of a decode block: ``qw`` gives shapes and scales, ``tiled`` is ``tile_weight_v2`` of its data
    (gate/up: of ``data.reshape(E, 2, I, K)`` with ``rows = I``)."""
    args.W = tiled.data_ptr()
    args.wtype = wtype_of(qw.data)
    args.rows, args.K = (rows if rows is not None else qw.data.shape[-2]), qw.data.shape[-1]
    args.n_experts = qw.data.shape[0] if qw.data.dim() == 3 else 1
    if qw.scale is not None:
        if qw.kb != 128:
            raise ValueError("the tensor-core path needs 128-wide K scale blocks")
        ks = kernel_scale(qw)
        args.wscale = ks.data_ptr()
        args.rb, args.nrb, args.nkb_stride = qw.rb, ks.shape[-2], ks.shape[-1]


def tc_decode(args: IhbTcDecArgs, use_pdl: bool = False) -> None:
    check(load().ihb_tc_decode(C.byref(args), int(use_pdl), stream_ptr()), "ihb_tc_decode")


def tc_dec_partial_floats(args: IhbTcDecArgs) -> int:
    return int(load().ihb_tc_dec_partial_floats(C.byref(args)))


def mat_of(qw) -> IhbMat:
    """Describes a (stack of) plain row-major weight matrices to the persistent decode kernel."""
    m = IhbMat()
    m.W = qw.data.data_ptr()
    m.rows, m.K = qw.data.shape[-2], qw.data.shape[-1]
    if qw.scale is not None:
        ks = kernel_scale(qw)
        m.wscale = ks.data_ptr()
        m.rb, m.kb_shift, m.nkb = qw.rb, kb_shift_of(qw.kb) - 4, ks.shape[-1]     # shift counted in 16-element chunks
    return m


def mega_max_grid(args: IhbMegaArgs) -> int:
    return int(load().ihb_mega_max_grid(C.byref(args)))


def mega_decode(args: IhbMegaArgs, grid: int = 0) -> None:
    check(load().ihb_mega_decode(C.byref(args), grid, stream_ptr()), "ihb_mega_decode")


def norm_quant_rows(x: torch.Tensor, gamma: Optional[torch.Tensor], eps: float, xq: torch.Tensor,
                    xs: Optional[torch.Tensor], fp8: bool, xn: Optional[torch.Tensor] = None) -> None:
    """x ``[T, K]`` fp32 -> (optional RMSNorm) -> ``xq`` ``[T, K]`` e4m3 / bf16 and ``xs`` ``[K / 128, T]``."""
    T, Kd = x.shape
    check(load().ihb_norm_quant_rows(x.data_ptr(), ptr(gamma), eps, Kd, T, ptr(xn), xq.data_ptr(), ptr(xs), int(fp8),
                                     stream_ptr()), "ihb_norm_quant_rows")


def qk_norm_rope_rows(qkv: torch.Tensor, nq: int, nkv: int, q_gamma, k_gamma, eps: float, cos_t, sin_t, positions,
                      slots, k_cache, v_cache, max_seq: int,
                      k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None) -> None:
    if k_scale is not None:                                     # e4m3 cache rows with a scale per row
        check(load().ihb_qk_norm_rope_rows_kv8(qkv.data_ptr(), nq, nkv, q_gamma.data_ptr(), k_gamma.data_ptr(), eps,
                                               cos_t.data_ptr(), sin_t.data_ptr(), positions.data_ptr(), slots.data_ptr(),
                                               k_cache.data_ptr(), v_cache.data_ptr(), k_scale.data_ptr(), v_scale.data_ptr(),
                                               max_seq, qkv.shape[0], stream_ptr()), "ihb_qk_norm_rope_rows_kv8")
        return
    check(load().ihb_qk_norm_rope_rows(qkv.data_ptr(), nq, nkv, q_gamma.data_ptr(), k_gamma.data_ptr(), eps,
                                       cos_t.data_ptr(), sin_t.data_ptr(), positions.data_ptr(), slots.data_ptr(),
                                       k_cache.data_ptr(), v_cache.data_ptr(), max_seq, qkv.shape[0], stream_ptr()),
          "ihb_qk_norm_rope_rows")


def window_attention_scratch_floats(nq: int, nkv: int, T: int) -> int:
    return max(1, int(load().ihb_window_attention_scratch_floats(nq, nkv, T)))


def window_attention(qkv: torch.Tensor, k_cache, v_cache, nq: int, nkv: int, max_seq: int, base: int,
                     mask: Optional[torch.Tensor], out: torch.Tensor, mode: Optional[int] = None,
                     scratch: Optional[torch.Tensor] = None,
                     k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None) -> None:
    """``mode`` 0: tensor-core tiles, 1: per-token CUDA-core kernel; default from ``IHB_WINDOW_ATTN`` (0). ``scratch``
    (``window_attention_scratch_floats(nq, nkv, T)`` floats) lets short windows slice the keys over many CTAs.
    ``k_scale`` / ``v_scale``: the caches are e4m3 bytes with one scale per row (tensor-core tiles only)."""
    if mode is None:
        mode = int(os.environ.get("IHB_WINDOW_ATTN", "0"))
    if scratch is not None and scratch.numel() < window_attention_scratch_floats(nq, nkv, qkv.shape[0]):
        raise ValueError("window attention scratch too small")
    if k_scale is not None:
        check(load().ihb_window_attention_kv8(qkv.data_ptr(), qkv.shape[1], k_cache.data_ptr(), v_cache.data_ptr(),
                                              k_scale.data_ptr(), v_scale.data_ptr(), nq, nkv, max_seq, base, qkv.shape[0],
                                              ptr(mask), out.data_ptr(), ptr(scratch), stream_ptr()),
              "ihb_window_attention_kv8")
        return
    check(load().ihb_window_attention(qkv.data_ptr(), qkv.shape[1], k_cache.data_ptr(), v_cache.data_ptr(), nq, nkv,
                                      max_seq, base, qkv.shape[0], ptr(mask), out.data_ptr(), mode, ptr(scratch),
                                      stream_ptr()),
          "ihb_window_attention")


def router_topk_rows(h: torch.Tensor, router: torch.Tensor, top_k: int, renorm: bool, ti: torch.Tensor, tw: torch.Tensor,
                     logits: Optional[torch.Tensor] = None) -> None:
    """Fused router of a window: ``h [T, H]`` fp32, ``router [E, H]`` bf16 -> expert ids ``ti [T, k]`` int32 and weights
    ``tw [T, k]`` fp32 (softmax, top-k, optional renormalisation)."""
    T, H = h.shape
    check(load().ihb_router_topk_rows(h.data_ptr(), router.data_ptr(), T, H, router.shape[0], top_k, int(renorm), ptr(logits),
                                      ti.data_ptr(), tw.data_ptr(), stream_ptr()), "ihb_router_topk_rows")


def moe_group_table(ti: torch.Tensor, expert0: int, e_local: int, nt: int, order: torch.Tensor, inv: torch.Tensor,
                    groups: torch.Tensor, n_groups: torch.Tensor) -> None:
    check(load().ihb_moe_group_table(ti.data_ptr(), ti.numel(), expert0, e_local, nt, order.data_ptr(), inv.data_ptr(),
                                     groups.data_ptr(), n_groups.data_ptr(), groups.shape[0], stream_ptr()), "ihb_moe_group_table")


def moe_gather_rows(src: torch.Tensor, order: torch.Tensor, k: int, out: torch.Tensor) -> None:
    """``out[p] = src[order[p] // k]`` for rows of bytes (``src [T, row_bytes]`` uint8)."""
    check(load().ihb_moe_gather_rows(src.data_ptr(), order.data_ptr(), k, src.shape[1], order.numel(), out.data_ptr(),
                                     stream_ptr()), "ihb_moe_gather_rows")


def moe_combine_rows(yg: torch.Tensor, inv: torch.Tensor, tw: torch.Tensor, k: int, y: torch.Tensor,
                     resid: Optional[torch.Tensor] = None) -> None:
    T, H = y.shape
    check(load().ihb_moe_combine_rows(yg.data_ptr(), inv.data_ptr(), tw.data_ptr(), k, H, T, ptr(resid), y.data_ptr(),
                                      stream_ptr()), "ihb_moe_combine_rows")


def allreduce_counted(comm: IhbComm, x: torch.Tensor, out: torch.Tensor, counter: torch.Tensor, call_counter: torch.Tensor,
                      err: torch.Tensor, resid: Optional[torch.Tensor] = None, gamma: Optional[torch.Tensor] = None,
                      eps: float = 1e-6, out_norm: Optional[torch.Tensor] = None,
                      out_norm_bf16: Optional[torch.Tensor] = None) -> None:
    """Latency-optimal fused all-reduce (+ residual + RMSNorm) of ``x [T, H]`` (fp32 or bf16), ``T <= 64``: counted
    fixed-point slots, one one-way trip, no barrier (``csrc/kernels/allreduce.cu::ar_counted_kernel``). ``call_counter``:
    ``ARC_MAX_ROWS`` int32 zeros owned by the slot region (``4 * ARC_MAX_ROWS * H`` 64-bit words, zeroed); ``counter`` is
    unused (kept for signature symmetry). T may change from call to call."""
    T, H = x.shape
    check(load().ihb_allreduce_counted(C.byref(comm), x.data_ptr(), int(x.dtype == torch.bfloat16), ptr(resid), ptr(gamma), eps,
                                       T, H, out.data_ptr(), ptr(out_norm), ptr(out_norm_bf16), counter.data_ptr(), call_counter.data_ptr(),
                                       err.data_ptr(), stream_ptr()), "ihb_allreduce_counted")


def dequant_bf16(qw, out: torch.Tensor) -> None:
    """bf16 copy of a block-scaled e4m3 :class:`QWeight` (``data [..., rows, K]``, ``scale [..., nrb, nkb]``)."""
    rows, Kd = qw.data.shape[-2], qw.data.shape[-1]
    nmat = qw.data.numel() // (rows * Kd)
    sc = qw.scale.contiguous()
    check(load().ihb_dequant_bf16(qw.data.data_ptr(), sc.data_ptr(), nmat, rows, Kd, qw.rb, qw.kb, sc.shape[-2], sc.shape[-1],
                                  out.data_ptr(), stream_ptr()), "ihb_dequant_bf16")


def a2a_rows(args: IhbA2AArgs, grid: int = 32) -> None:
    """One all-to-all exchange of rows over peer memory (see ``csrc/kernels/a2a.cu``)."""
    check(load().ihb_a2a_rows(C.byref(args), grid, stream_ptr()), "ihb_a2a_rows")


def allreduce_norm(comm: IhbComm, x: torch.Tensor, out: torch.Tensor, counter: torch.Tensor, err: torch.Tensor,
                   resid: Optional[torch.Tensor] = None, gamma: Optional[torch.Tensor] = None, eps: float = 1e-6,
                   out_norm: Optional[torch.Tensor] = None, algo: int = 0, grid: int = 0,
                   out_norm_bf16: Optional[torch.Tensor] = None) -> None:
    """Fused all-reduce (+ residual + RMSNorm) of ``x [T, H]`` fp32 over the symmetric buffer described by ``comm``."""
    T, H = x.shape
    check(load().ihb_allreduce_norm(C.byref(comm), x.data_ptr(), ptr(resid), ptr(gamma), eps, T, H, out.data_ptr(),
                                    ptr(out_norm), ptr(out_norm_bf16), counter.data_ptr(), err.data_ptr(), algo, grid, stream_ptr()),
          "ihb_allreduce_norm")
