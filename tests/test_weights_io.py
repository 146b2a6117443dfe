"""Weight input / output on CPU: a Hugging Face style safetensors directory, this package's converted layout (save,
load, the convert command) and a directory in the exact format of the reference's converter
(tools/conifer_weight_convert.py: per-row fp8 scales, no manifest, K / V replicated in the QKV matrix)."""
import os

import numpy as np
import pytest
import torch

from inferencehackathon_b200.config import ParallelConfig, QuantConfig, get_model_config
from inferencehackathon_b200.models.qwen3_moe import Qwen3MoE
from inferencehackathon_b200.models.weights import (load_engine_layout, random_state_dict, save_engine_layout,
                                                    shard_state_dict)
from inferencehackathon_b200.parallel.collectives import Collectives


def _logits(w, toks):
    par = w.par
    m = Qwen3MoE(w, Collectives(ParallelConfig(tp=1, ep=1, rank=0, world=1)) if par.world == 1 else None)
    cache = m.new_cache(64, torch.float32, "cpu")
    return m.forward(torch.tensor(toks), cache)


def _same(a, b):
    assert a.data.dtype == b.data.dtype and torch.equal(a.data.view(torch.uint8), b.data.view(torch.uint8))
    assert (a.scale is None) == (b.scale is None)
    if a.scale is not None:
        assert torch.equal(a.scale, b.scale) and (a.rb, a.kb) == (b.rb, b.kb)


@pytest.mark.parametrize("weights", ["fp32", "fp8_block"])
def test_converted_layout_round_trip(tmp_path, weights):
    cfg = get_model_config("tiny")
    q = QuantConfig(weights=weights, kv="fp32")
    for rank in range(2):
        par = ParallelConfig(tp=2, ep=1, rank=rank, world=2)
        w = shard_state_dict(random_state_dict(cfg, 0), cfg, par, q)
        save_engine_layout(w, str(tmp_path))
        back = load_engine_layout(str(tmp_path), cfg, par, q)
        assert torch.equal(back.embed.float(), w.embed.float()) and torch.equal(back.final_norm, w.final_norm)
        _same(back.lm_head, w.lm_head)
        for a, b in zip(back.layers, w.layers):
            for nm in ("wqkv", "wo", "w_gu", "w_d"):
                _same(getattr(a, nm), getattr(b, nm))
            assert torch.equal(a.router.float(), b.router.float())
            for nm in ("in_ln", "post_ln", "q_norm", "k_norm"):
                assert torch.equal(getattr(a, nm), getattr(b, nm))


def test_safetensors_directory_and_convert_command(tmp_path):
    from safetensors.torch import save_file
    from inferencehackathon_b200.models import convert
    cfg = get_model_config("tiny")
    sd = random_state_dict(cfg, 3)
    src = tmp_path / "hf"
    src.mkdir()
    names = sorted(sd)
    half = len(names) // 2                                       # two shard files, no index: the loader scans them
    save_file({k: sd[k].contiguous() for k in names[:half]}, str(src / "model-00001-of-00002.safetensors"))
    save_file({k: sd[k].contiguous() for k in names[half:]}, str(src / "model-00002-of-00002.safetensors"))
    one = ParallelConfig(tp=1, ep=1, rank=0, world=1)
    q = QuantConfig(weights="fp32", kv="fp32")
    from_dir = shard_state_dict(str(src), cfg, one, q)
    from_dict = shard_state_dict(sd, cfg, one, q)
    toks = [1, 5, 9, 2, 7]
    assert torch.equal(_logits(from_dir, toks), _logits(from_dict, toks))
    # the command writes one directory per rank, which loads back to the same shards
    dst = tmp_path / "out"
    assert convert.main(["--src", str(src), "--dst", str(dst), "--model", "tiny", "--tp", "2", "--weights", "fp32"]) == 0
    for rank in range(2):
        par = ParallelConfig(tp=2, ep=1, rank=rank, world=2)
        back = load_engine_layout(str(dst / f"rank{rank:02d}"), cfg, par, q)
        want = shard_state_dict(sd, cfg, par, q)
        for a, b in zip(back.layers, want.layers):
            _same(a.wqkv, b.wqkv); _same(a.w_gu, b.w_gu); _same(a.w_d, b.w_d); _same(a.wo, b.wo)


def _rowwise(w):
    w = w.float()
    scale = w.abs().amax(dim=1).clamp_min(1e-8) / 448.0
    q = (w / scale[:, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q, scale.float()


def _write_reference_format(sd, cfg, tp, out):
    """The file set of tools/conifer_weight_convert.py for a model of any size (the tool itself hard-codes the
    235B shapes): per-row scales, K / V of all heads in every rank's wqkv, router as fp8, embed on rank 0 only."""
    hd, H = cfg.head_dim, cfg.hidden
    qr, ir, vr = cfg.n_q_heads * hd // tp, cfg.moe_inter // tp, cfg.vocab // tp
    expect = {}
    for r in range(tp):
        rd = os.path.join(out, f"rank{r}")
        os.makedirs(rd)
        if r == 0:
            sd["model.embed_tokens.weight"].to(torch.bfloat16).view(torch.int16).numpy().tofile(os.path.join(rd, "embed.bf16"))
        sd["model.norm.weight"].float().numpy().tofile(os.path.join(rd, "norm_final.f32"))

        def put(path, w, key):
            q, s = _rowwise(w.contiguous())
            q.view(torch.uint8).numpy().tofile(path + ".fp8")
            s.numpy().tofile(path + ".scale")
            expect[(r, key)] = q.float() * s[:, None]

        put(os.path.join(rd, "lm_head"), sd["lm_head.weight"][r * vr:(r + 1) * vr], "lm_head")
        for L in range(cfg.n_layers):
            ld = os.path.join(rd, f"layer{L}")
            os.makedirs(ld)
            p = f"model.layers.{L}."
            for nm, fn in (("input_layernorm", "in_ln"), ("post_attention_layernorm", "post_ln"),
                           ("self_attn.q_norm", "q_norm"), ("self_attn.k_norm", "k_norm")):
                sd[p + nm + ".weight"].float().numpy().tofile(os.path.join(ld, fn + ".f32"))
            wqkv = torch.cat([sd[p + "self_attn.q_proj.weight"][r * qr:(r + 1) * qr], sd[p + "self_attn.k_proj.weight"],
                              sd[p + "self_attn.v_proj.weight"]], 0)
            put(os.path.join(ld, "wqkv"), wqkv, (L, "wqkv"))
            put(os.path.join(ld, "wo"), sd[p + "self_attn.o_proj.weight"][:, r * qr:(r + 1) * qr], (L, "wo"))
            put(os.path.join(ld, "wgate"), sd[p + "mlp.gate.weight"], (L, "wgate"))
            for E in range(cfg.n_experts):
                ep = p + f"mlp.experts.{E}."
                wgu = torch.cat([sd[ep + "gate_proj.weight"][r * ir:(r + 1) * ir], sd[ep + "up_proj.weight"][r * ir:(r + 1) * ir]], 0)
                put(os.path.join(ld, f"e{E}_wgu"), wgu, (L, f"e{E}_wgu"))
                put(os.path.join(ld, f"e{E}_wd"), sd[ep + "down_proj.weight"][:, r * ir:(r + 1) * ir], (L, f"e{E}_wd"))
    return expect


def test_directory_written_by_the_reference_converter_loads(tmp_path):
    cfg = get_model_config("tiny")
    sd = random_state_dict(cfg, 1)
    tp = 2
    expect = _write_reference_format(sd, cfg, tp, str(tmp_path))
    q = QuantConfig(weights="fp8_block", kv="fp32")
    hd = cfg.head_dim
    for r in range(tp):
        par = ParallelConfig(tp=tp, ep=1, rank=r, world=tp)
        w = load_engine_layout(str(tmp_path), cfg, par, q)
        g = w.geom
        assert torch.equal(w.lm_head.dequant(), expect[(r, "lm_head")])
        for L, lw in enumerate(w.layers):
            full = expect[(r, (L, "wqkv"))]
            nq = g.nq_local * hd
            k0 = nq + g.kv_head0 * hd
            v0 = nq + cfg.n_kv_heads * hd + g.kv_head0 * hd
            want = torch.cat([full[:nq], full[k0:k0 + g.nkv_local * hd], full[v0:v0 + g.nkv_local * hd]], 0)
            assert lw.wqkv.data.shape[0] == (g.nq_local + 2 * g.nkv_local) * hd
            assert torch.equal(lw.wqkv.dequant(), want)
            assert torch.equal(lw.wo.dequant(), expect[(r, (L, "wo"))])
            assert torch.allclose(lw.router.float(), expect[(r, (L, "wgate"))], atol=0, rtol=1e-2)      # stored as bf16
            for E in range(cfg.n_experts):
                assert torch.equal(lw.w_gu.select(E).dequant(), expect[(r, (L, f"e{E}_wgu"))])
                assert torch.equal(lw.w_d.select(E).dequant(), expect[(r, (L, f"e{E}_wd"))])
    # and the loaded shards are a usable model: next to the fp32 model of the same state dict, within the e4m3 grid
    one = ParallelConfig(tp=1, ep=1, rank=0, world=1)
    exp1 = _write_reference_format(sd, cfg, 1, str(tmp_path / "tp1"))
    w1 = load_engine_layout(str(tmp_path / "tp1"), cfg, one, q)
    ref = shard_state_dict(sd, cfg, one, QuantConfig(weights="fp32", kv="fp32"))
    toks = [3, 1, 4, 1, 5, 9, 2, 6]
    a, b = _logits(w1, toks), _logits(ref, toks)
    assert torch.isfinite(a).all()
    assert float((a - b).abs().max()) < 0.15 * float(b.abs().max())


def test_device_random_state_dict_gives_every_layout_the_same_model():
    """Tensors generated on demand from a seed derived from their name: a tensor-parallel and an expert-parallel shard
    are slices of the one-rank model (what the benchmark's distributed correctness gate relies on)."""
    import torch
    from inferencehackathon_b200.config import ParallelConfig, QuantConfig, get_model_config
    from inferencehackathon_b200.models.weights import DeviceRandomStateDict, shard_state_dict
    m = get_model_config("small", 2)
    sd = DeviceRandomStateDict(m, 0, "cpu")
    assert "model.layers.1.mlp.experts.3.up_proj.weight" in sd and "nope" not in sd
    assert torch.equal(sd["model.norm.weight"], sd["model.norm.weight"])           # regenerated, same numbers
    q = QuantConfig(weights="bf16", kv="bf16")
    full = shard_state_dict(sd, m, ParallelConfig(tp=1, ep=1, rank=0, world=1), q, device="cpu")
    hd = m.head_dim
    for par in (ParallelConfig(tp=2, ep=1, rank=1, world=2), ParallelConfig(tp=1, ep=2, rank=1, world=2)):
        sh = shard_state_dict(sd, m, par, q, device="cpu")
        g = sh.geom
        f, s = full.layers[1], sh.layers[1]
        assert torch.equal(s.wqkv.data[: g.nq_local * hd], f.wqkv.data[g.q_head0 * hd:(g.q_head0 + g.nq_local) * hd])
        assert torch.equal(s.w_gu.data[0][: g.inter_local], f.w_gu.data[g.expert0][g.inter0: g.inter0 + g.inter_local])
        assert torch.equal(s.w_d.data[0], f.w_d.data[g.expert0][:, g.inter0: g.inter0 + g.inter_local])
        assert torch.equal(s.router, f.router)
        assert torch.equal(sh.lm_head.data, full.lm_head.data[g.vocab0: g.vocab0 + g.vocab_local])


def test_window_attention_scratch_always_covers_the_slices_it_is_asked_for():
    """Host-side sizing of the key-sliced window attention (no GPU needed): for every shape the scratch size the
    library reports must hold one 132-float record per (token, head, slice) for the slice count it will launch, and
    the slice count never exceeds the number of 64-key blocks or the library's limit."""
    from inferencehackathon_b200.ops import lib
    L = lib.load()
    for nq, nkv in [(8, 1), (8, 2), (16, 2), (64, 4), (4, 1), (32, 4), (1, 1)]:
        for T in [1, 4, 8, 16, 17, 64, 128, 257, 600, 1024]:
            need = int(L.ihb_window_attention_scratch_floats(nq, nkv, T))
            for base in [0, 1, 63, 64, 500, 4096, 32768]:
                s = int(L.ihb_window_attention_splits(nq, nkv, base, T))
                assert 1 <= s <= 32
                assert s <= (base + T + 63) // 64
                assert s == 1 or need >= T * nq * s * 132, (nq, nkv, T, base, s, need)


def test_k_split_rule_of_the_window_gemms():
    from inferencehackathon_b200.runtime.gpu_window import GpuWindow

    class _W:
        sms = 148
    assert GpuWindow._k_split(_W, 80, 64, 1024) == 1          # wide token tiles are never split
    assert GpuWindow._k_split(_W, 10, 64, 128) == 1
    assert GpuWindow._k_split(_W, 149, 64, 1) > 1             # the one-token head: 149 tiles on 148 SMs
    assert GpuWindow._k_split(_W, 1187, 64, 8) == 1           # many tiles: no split
    for tiles, nkb, T in [(10, 64, 8), (72, 64, 16), (32, 16, 8), (1, 3, 1)]:
        ks = GpuWindow._k_split(_W, tiles, nkb, T)
        assert 1 <= ks <= min(nkb, 16)


# ---- property-based checks ------------------------------------------------------------------------------------------------------------
from hypothesis import given, settings, strategies as st   # noqa: E402


@settings(max_examples=60, deadline=None)
@given(st.integers(1, 70), st.integers(1, 90), st.sampled_from([8, 16, 32]), st.sampled_from([8, 16, 32]), st.integers(0, 2 ** 31 - 1))
def test_block_quantisation_round_trip_and_sub_matrix_scales(rows, K, rb, kb, seed):
    """Any matrix size (not a multiple of the block), any block shape: de-quantised values are within half an e4m3 step of
    the input relative to the block's largest value, and the scales of any block-aligned-or-not sub-matrix, re-blocked by
    ``reblock_scales``, de-quantise that sub-matrix to the same numbers as the full matrix does."""
    from inferencehackathon_b200.models.quant import dequant_block, quant_block, reblock_scales
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, K, generator=g) * torch.rand(1, generator=g) * 10
    qw = quant_block(w, rb, kb)
    deq = dequant_block(qw.data, qw.scale, rb, kb)
    assert deq.shape == w.shape
    amax_blocks = qw.scale.repeat_interleave(rb, 0)[:rows].repeat_interleave(kb, 1)[:, :K] * 448.0
    assert float(((deq - w).abs() / amax_blocks).max()) <= 2 ** -4 + 1e-6          # e4m3: 3 mantissa bits
    r0 = int(torch.randint(0, rows, (1,), generator=g))
    k0 = int(torch.randint(0, K, (1,), generator=g))
    nr = int(torch.randint(1, rows - r0 + 1, (1,), generator=g))
    nk = int(torch.randint(1, K - k0 + 1, (1,), generator=g))
    sub, rb2, kb2 = reblock_scales(qw.scale, rb, kb, r0, nr, k0, nk)
    assert rb % rb2 == 0 and kb % kb2 == 0
    deq_sub = dequant_block(qw.data[r0:r0 + nr, k0:k0 + nk], sub, rb2, kb2)
    assert torch.equal(deq_sub, deq[r0:r0 + nr, k0:k0 + nk])


@settings(max_examples=80, deadline=None)
@given(st.sampled_from(["tiny", "small", "qwen3-30b-a3b", "qwen3-235b-a22b"]), st.sampled_from([1, 2, 4, 8]),
       st.sampled_from(["tp", "ep", "hybrid"]), st.sampled_from([1, 2, 4]))
def test_shards_of_all_ranks_tile_every_dimension_exactly_once(model, world, plan, attn_tp):
    """For every valid layout: the ranks' query heads, expert-intermediate columns / experts and vocabulary rows
    partition their ranges (no gap, no overlap), and every KV head is held by the ranks whose query heads use it."""
    from inferencehackathon_b200.models.weights import shard_geometry
    cfg = get_model_config(model)
    tp, ep = {"tp": (world, 1), "ep": (1, world), "hybrid": (min(attn_tp, world), world)}[plan]
    if world == 1:
        tp, ep = 1, 1
    try:
        geoms = [shard_geometry(cfg, ParallelConfig(tp=tp, ep=ep, rank=r, world=world)) for r in range(world)]
    except ValueError:
        return                                                              # a layout the model's shapes do not allow
    vocab = sorted((g.vocab0, g.vocab0 + g.vocab_local) for g in geoms)
    assert vocab[0][0] == 0 and all(a[1] == b[0] for a, b in zip(vocab, vocab[1:])) and vocab[-1][1] == cfg.vocab
    groups = world // tp                                                    # attention is replicated across tp groups
    heads = sorted((g.q_head0, g.q_head0 + g.nq_local) for g in geoms)
    for h in range(cfg.n_q_heads):
        assert sum(1 for a, b in heads if a <= h < b) == groups
    q_per_kv = cfg.n_q_heads // cfg.n_kv_heads
    for g in geoms:
        used = {h // q_per_kv for h in range(g.q_head0, g.q_head0 + g.nq_local)}
        assert used <= set(range(g.kv_head0, g.kv_head0 + g.nkv_local))
    if ep > 1:
        ex = sorted((g.expert0, g.expert0 + g.n_experts_local) for g in geoms)
        assert ex[0][0] == 0 and all(a[1] == b[0] for a, b in zip(ex, ex[1:])) and ex[-1][1] == cfg.n_experts
        assert all(g.inter_local == cfg.moe_inter and g.inter0 == 0 for g in geoms)
    else:
        cols = sorted((g.inter0, g.inter0 + g.inter_local) for g in geoms)
        assert cols[0][0] == 0 and all(a[1] == b[0] for a, b in zip(cols, cols[1:])) and cols[-1][1] == cfg.moe_inter
        assert all(g.n_experts_local == cfg.n_experts for g in geoms)


def test_checkpoint_of_another_shape_is_refused_with_the_tensors_name():
    cfg = get_model_config("tiny")
    sd = random_state_dict(cfg, 0)
    one, q = ParallelConfig(), QuantConfig(weights="fp32", kv="fp32")
    name = "model.layers.1.mlp.experts.3.up_proj.weight"
    bad = dict(sd)
    bad[name] = bad[name][:, :-1]
    with pytest.raises(ValueError, match="experts.3.up_proj.weight.*shape"):
        shard_state_dict(bad, cfg, one, q)
    bad = dict(sd)
    bad["model.layers.0.self_attn.q_norm.weight"] = torch.ones(cfg.head_dim * 2)
    with pytest.raises(ValueError, match="q_norm"):
        shard_state_dict(bad, cfg, one, q)
    missing = dict(sd)
    del missing[name]
    with pytest.raises(KeyError, match="up_proj"):
        shard_state_dict(missing, cfg, one, q)
