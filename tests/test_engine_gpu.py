"""End-to-end: the CUDA decode pipeline against the PyTorch reference model on the same weights (B200)."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

from inferencehackathon_b200 import SMALL
from inferencehackathon_b200.runtime.engine import InferenceEngine


def _prompt(n=24):
    return torch.randint(0, SMALL.vocab, (n,), generator=torch.Generator().manual_seed(3)).tolist()


@pytest.mark.parametrize("weights", ["bf16", "fp8_block"])
@pytest.mark.parametrize("pipeline,graph", [("mega", False), ("mega_wide", False), ("tc", False), ("tc", True), ("simt", True)])
def test_cuda_decode_matches_torch_reference(weights, pipeline, graph, monkeypatch):
    """``mega``: the persistent whole-token kernel (``mega_wide``: its build for large shares, forced onto the small
    model); ``tc``: tensor-core linears, one kernel per op; ``simt``: the streaming GEMV kernels."""
    monkeypatch.setenv("IHB_MEGA_WIDE", "1" if pipeline == "mega_wide" else "0")
    if pipeline == "mega_wide":
        pipeline = "mega"
    monkeypatch.setenv("IHB_MEGA", "1" if pipeline == "mega" else "0")
    monkeypatch.setenv("IHB_TC", "0" if pipeline == "simt" else "1")
    dev = "cuda:0"
    ref = InferenceEngine.build("small", weights=weights, device=dev, backend="torch", max_seq=256)
    eng = InferenceEngine.build("small", weights=weights, device=dev, backend="cuda", max_seq=256, use_graph=graph)
    assert eng.gpu.use_mega == (pipeline == "mega")
    tc_mode = "fp8" if weights == "fp8_block" else "bf16"
    # the oracle rounds activations the way the kernels store them: per-token fp8 / bf16 in the tensor-core GEMMs
    # (per-op pipeline, and the batched prompt pass of the other pipelines), fp16 in the CUDA-core GEMVs
    decode_mode = tc_mode if (eng.gpu.use_tc and not eng.gpu.use_mega) else None
    ref.model.act_mode = eng.gpu.window().act_mode if eng.gpu.has_window() else decode_mode
    pr = ref.prefill(_prompt(), return_logits=True)
    pe = eng.prefill(_prompt(), return_logits=True)
    scale = float(pr.logits.abs().max())
    assert float((pr.logits[0] - pe.logits[0]).abs().max()) < 0.02 * scale
    ref.reset(); eng.reset()
    ref.model.act_mode = decode_mode
    a = ref.generate(_prompt(), 24)
    # teacher forcing: the CUDA engine is fed the reference's tokens, so one near-tie cannot derail the comparison
    pe = eng.prefill(_prompt())
    got = [pe.next_token]
    routes_first = None
    for t in a.tokens[:-1]:
        st = eng.decode_step(t)
        got.append(st.token_id)
        if routes_first is None:
            routes_first = st.routes
    agree = sum(int(x == y) for x, y in zip(a.tokens, got))
    assert agree >= (22 if weights == "bf16" else 17), (a.tokens, got)
    # routing telemetry of the first decoded token comes from the device router
    ra = [sorted(r.experts) for r in a.routes[1]]
    rb = [sorted(r.experts) for r in routes_first]
    same = sum(int(x == y) for x, y in zip(ra, rb))
    assert same >= len(ra) - 1
    eng.gpu.check_error()


@pytest.mark.parametrize("weights", ["bf16", "fp8_block"])
def test_e4m3_kv_cache_on_the_cuda_path_matches_the_pytorch_cache(weights):
    """``kv="fp8"``: the window path and the per-kernel decode pipeline append e4m3 rows with a scale per position and
    attend over them; the oracle is the PyTorch model with its own e4m3 cache of the same scheme."""
    dev = "cuda:0"
    ref = InferenceEngine.build("small", weights=weights, kv="fp8", device=dev, backend="torch", max_seq=256)
    eng = InferenceEngine.build("small", weights=weights, kv="fp8", device=dev, backend="cuda", max_seq=256)
    assert eng.gpu.kv_fp8 and not eng.gpu.use_mega and eng.gpu.has_window()
    assert eng.gpu.k_cache.dtype == torch.uint8 and eng.gpu.k_scale.shape == eng.gpu.k_cache.shape[:3]
    ref.model.act_mode = eng.gpu.window().act_mode
    pr = ref.prefill(_prompt(), return_logits=True)
    pe = eng.prefill(_prompt(), return_logits=True)
    scale = float(pr.logits.abs().max())
    assert float((pr.logits[0] - pe.logits[0]).abs().max()) < 0.04 * scale
    # the rows the prompt pass wrote decode to the oracle's rows (layer 0: same inputs on both sides)
    n = len(_prompt())
    k_ref, v_ref = ref.cache.read(0, n)
    k_eng = eng.gpu.k_cache[0, :, :n].view(torch.float8_e4m3fn).float() * eng.gpu.k_scale[0, :, :n, None]
    v_eng = eng.gpu.v_cache[0, :, :n].view(torch.float8_e4m3fn).float() * eng.gpu.v_scale[0, :, :n, None]
    assert float((k_eng - k_ref.float()).abs().max()) < 0.14 * float(k_ref.float().abs().max())
    assert float((v_eng - v_ref.float()).abs().max()) < 0.14 * float(v_ref.float().abs().max())
    ref.reset(); eng.reset()
    ref.model.act_mode = None
    a = ref.generate(_prompt(), 24)
    pe = eng.prefill(_prompt())
    got = [pe.next_token]
    for t in a.tokens[:-1]:                      # teacher forcing, as in the bf16-cache test
        got.append(eng.decode_step(t).token_id)
    agree = sum(int(x == y) for x, y in zip(a.tokens, got))
    assert agree >= (20 if weights == "bf16" else 15), (a.tokens, got)
    eng.gpu.check_error()


@pytest.mark.parametrize("mega", ["0", "1"])
def test_graph_replay_is_deterministic(mega, monkeypatch):
    monkeypatch.setenv("IHB_MEGA", mega)
    eng = InferenceEngine.build("small", weights="fp8_block", device="cuda:0", backend="cuda", max_seq=256)
    a = eng.generate(_prompt(), 16).tokens
    b = eng.generate(_prompt(), 16).tokens
    assert a == b


def test_poisoned_error_word_ends_the_waits_and_the_engine_falls_back():
    """A nonzero device error word makes every bounded wait of the persistent kernel give up at once (no hang, no
    fault); the step reports it, the engine continues on the reference path with the same tokens."""
    dev = "cuda:0"
    ref = InferenceEngine.build("small", weights="bf16", device=dev, backend="torch", max_seq=256)
    eng = InferenceEngine.build("small", weights="bf16", device=dev, backend="cuda", max_seq=256)
    ref.model.act_mode = "bf16"
    prompt = _prompt(20)
    want = ref.generate(prompt, 10).tokens
    pe = eng.prefill(prompt)
    got = [pe.next_token]
    for i in range(9):
        if i == 3:
            eng.gpu.err.fill_(7)                   # host-set poison: the kernel's barriers check this word
        got.append(eng.decode_step().token_id)
    assert eng.healthy is False and eng.gpu is None and len(eng.failures) == 1
    agree = sum(int(a == b) for a, b in zip(want, got))
    assert agree >= 8, (want, got)


@pytest.mark.parametrize("tc", ["1", "0"])
def test_per_kernel_table_of_the_per_op_pipelines(tc, monkeypatch):
    """Every launch of a step is timed on the device; the table leaves the decode state untouched."""
    monkeypatch.setenv("IHB_MEGA", "0")
    monkeypatch.setenv("IHB_TC", tc)
    eng = InferenceEngine.build("small", weights="fp8_block", device="cuda:0", backend="cuda", max_seq=128)
    prompt = _prompt(16)
    first = eng.generate(prompt, 4).tokens
    rows = eng.gpu.op_table(3)
    per_token = sum(r["launches_per_token"] for r in rows)
    assert per_token == eng.gpu.n_launches_per_step
    assert all(r["us_per_launch"] > 0 for r in rows) and abs(sum(r["share"] for r in rows) - 1.0) < 1e-6
    assert eng.generate(prompt, 4).tokens == first


@pytest.mark.parametrize("ctx", [1500, 2600])
def test_persistent_kernel_at_longer_contexts(ctx, monkeypatch):
    """Both attention schemes of the persistent kernel against the PyTorch model: up to 16 blocks of 128 positions
    the partial records are merged by the o_proj CTAs (ctx 1500: 12 blocks); beyond that the split scheme with a
    last-arriver merge runs (ctx 2600: 21 blocks). The prompt goes through the batched window path; the decoded
    tokens are compared under teacher forcing."""
    monkeypatch.setenv("IHB_MEGA", "1")
    dev = "cuda:0"
    g = torch.Generator().manual_seed(ctx)
    prompt = torch.randint(0, SMALL.vocab, (ctx,), generator=g).tolist()
    ref = InferenceEngine.build("small", weights="bf16", device=dev, backend="torch", max_seq=ctx + 64)
    eng = InferenceEngine.build("small", weights="bf16", device=dev, backend="cuda", max_seq=ctx + 64)
    assert eng.gpu.use_mega
    a = ref.generate(prompt, 12)
    pe = eng.prefill(prompt)
    got = [pe.next_token]
    for t in a.tokens[:-1]:
        got.append(eng.decode_step(t, want_routes=False).token_id)
    eng.gpu.check_error()
    agree = sum(int(x == y) for x, y in zip(a.tokens[1:], got[1:]))          # the decoded tokens (not the prompt pass)
    assert agree >= 9, (a.tokens, got)


@pytest.mark.parametrize("weights", ["bf16", "fp8_block"])
def test_one_rank_of_tp8_of_the_large_architecture_against_pytorch(weights):
    """The weights the benchmark's distributed correctness gate builds at 8 GPUs (two layers of Qwen3-235B-A22B, every
    tensor generated whole from a name-derived seed and sliced: 8 query heads on a replicated KV head, 192 columns of
    every expert, block-fp8 gate/up shards with 64-row scale blocks), run as a one-rank model: the persistent kernel
    and the PyTorch model must agree on the logits after a prompt fed token by token."""
    from inferencehackathon_b200.config import EngineConfig, ParallelConfig, QuantConfig, get_model_config
    from inferencehackathon_b200.models.weights import DeviceRandomStateDict, shard_state_dict
    from inferencehackathon_b200.parallel.collectives import Collectives
    dev = torch.device("cuda", 0)
    mcfg = get_model_config("qwen3-235b-a22b", 2)
    q = QuantConfig(weights=weights, kv="bf16")
    w = shard_state_dict(DeviceRandomStateDict(mcfg, 0, dev), mcfg, ParallelConfig(tp=8, ep=1, rank=3, world=8), q, device=dev)
    if weights == "fp8_block":
        assert w.layers[0].w_gu.rb == 64 and w.layers[0].w_gu.data.shape[-2] == 2 * 192
    one = ParallelConfig(tp=1, ep=1, rank=0, world=1)
    prompt = torch.randint(0, mcfg.vocab, (12,), generator=torch.Generator().manual_seed(5)).tolist()
    outs = {}
    for backend in ("torch", "cuda"):
        cfg = EngineConfig(model=mcfg, parallel=one, quant=q, max_seq=64, seed=0, backend=backend)
        eng = InferenceEngine(cfg, w, Collectives(one), dev)
        if backend == "cuda":
            os.environ["IHB_WINDOW_PREFILL"] = "0"
        try:
            outs[backend] = eng.prefill(prompt, return_logits=True).logits[0].float()
        finally:
            os.environ.pop("IHB_WINDOW_PREFILL", None)
        if backend == "cuda":
            eng.gpu.check_error()
    scale = float(outs["torch"].abs().max())
    assert float((outs["torch"] - outs["cuda"]).abs().max()) < 0.02 * scale


@pytest.mark.parametrize("per_launch", [1, 4, 5])
def test_several_tokens_per_launch_give_the_tokens_of_single_steps(per_launch, monkeypatch):
    """``decode_many``: the persistent kernel loops over tokens inside one cooperative launch (feeding its own arg-max
    back, logging tokens in the device ring); the result must be the token sequence of one launch per token."""
    monkeypatch.setenv("IHB_MEGA", "1")
    dev = "cuda:0"
    a = InferenceEngine.build("small", weights="fp8_block", device=dev, backend="cuda", max_seq=256)
    b = InferenceEngine.build("small", weights="fp8_block", device=dev, backend="cuda", max_seq=256)
    pa, pb = a.prefill(_prompt()), b.prefill(_prompt())
    assert pa.next_token == pb.next_token
    single = [a.decode_step(want_routes=False).token_id for _ in range(13)]
    many = b.decode_many(13, per_launch=per_launch)
    assert many == single
    # both engines continue identically afterwards (position, token and history bookkeeping)
    assert a.decode_step(want_routes=False).token_id == b.decode_step(want_routes=False).token_id
    assert a.seq_len == b.seq_len
    b.gpu.check_error()
