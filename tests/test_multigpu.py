"""Fused GEMV + all-reduce kernels over NVLink peer memory: tensor-parallel decode on 2 GPUs must reproduce the
single-GPU engine (needs >= 2 B200s; spawns one process per GPU)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys, json, torch
sys.path.insert(0, os.environ["IHB_ROOT"])
import torch.distributed as dist
from inferencehackathon_b200.parallel.launch import init_distributed
from inferencehackathon_b200.runtime.engine import InferenceEngine
rank, world, local = init_distributed()
dev = torch.device("cuda", local)
weights = os.environ.get("IHB_TEST_WEIGHTS", "bf16")
prompt = torch.randint(0, 4096, (20,), generator=torch.Generator().manual_seed(3)).tolist()
plan = os.environ.get("IHB_TEST_PLAN", "tp")
tp, ep = {"tp": (world, 1), "ep": (1, world), "hybrid": (world, world)}[plan]
if os.environ.get("IHB_TEST_WINDOW", "0") != "1":
    os.environ["IHB_WINDOW_PREFILL"] = "0"      # the prompt goes through the persistent decode kernel, token by token
eng = InferenceEngine.build("small", tp=tp, ep=ep, rank=rank, world=world, weights=weights, device=dev, backend="cuda", max_seq=128)
pre = eng.prefill(prompt, return_logits=True)
tokens = [pre.next_token]
if os.environ.get("IHB_TEST_MANY", "0") == "1":
    tokens += eng.decode_many(11, per_launch=4)          # several tokens per cooperative launch, all-reduces included
else:
    for _ in range(11):
        tokens.append(eng.decode_step(want_routes=False).token_id)
eng.gpu.check_error()
ref_tokens, rel_err = None, None
if rank == 0:
    ref = InferenceEngine.build("small", weights=weights, device=dev, backend="cuda", max_seq=128)
    pr = ref.prefill(prompt, return_logits=True)
    ref_tokens = [pr.next_token]
    for t in tokens[:-1]:                        # teacher forcing: one near-tie cannot derail the rest
        ref_tokens.append(ref.decode_step(t, want_routes=False).token_id)
    rel_err = float((pr.logits[0].float() - pre.logits[0].float()).abs().max() / pr.logits.abs().max())
toks = [None] * world
dist.all_gather_object(toks, tokens)
if rank == 0:
    print("RESULT " + json.dumps({"tokens": toks, "ref": ref_tokens, "logits_rel_err": rel_err,
                                  "mc": bool(eng.gpu.symm.use_multicast)}))
dist.barrier()
dist.destroy_process_group()
"""


def _run(n, mode, weights, plan="tp", extra_env=None):
    env = dict(os.environ, IHB_ROOT=ROOT, IHB_COMM_MODE=mode, IHB_TEST_WEIGHTS=weights, IHB_TEST_PLAN=plan)
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29533", "-c", WORKER]
    # torchrun has no -c: write the worker to a temp file instead
    import tempfile
    with tempfile.NamedTemporaryFile("w", suffix=".py", delete=False) as f:
        f.write(WORKER)
        path = f.name
    cmd = cmd[:-2] + [path]
    r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    os.unlink(path)
    assert r.returncode == 0, r.stdout[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1]
    import json
    return json.loads(line[7:])


@pytest.mark.parametrize("mode", ["p2p", "auto"])
@pytest.mark.parametrize("weights", ["bf16", "fp8_block"])
def test_tp2_decode_matches_single_gpu(mode, weights):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = _run(2, mode, weights)
    assert out["tokens"][0] == out["tokens"][1], out          # ranks stay in lock step
    agree = sum(int(a == b) for a, b in zip(out["tokens"][0], out["ref"]))
    # bf16 shards hold the same numbers as the unsharded model: the logits after the prompt agree to rounding noise and
    # (teacher-forced) nearly every token. Block-fp8 shards are quantised per shard (other blocks, other scales): that
    # is a different set of weights, so only a loose bound applies there.
    if weights == "bf16":
        assert out["logits_rel_err"] < 0.02 and agree >= 11, out
    else:
        assert out["logits_rel_err"] < 0.25 and agree >= 8, out


def test_one_lagging_cta_changes_nothing():
    """One CTA of rank 1 idles 30 us before every all-reduce read (host-configured, bounded): every other CTA of
    both GPUs has to wait for it at the next round, nothing may time out, and the tokens are those of the undelayed
    run (the slot protocol depends on no CTA being 'only a reader')."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    base = _run(2, "auto", "bf16")
    for cta in (0, 17):
        out = _run(2, "auto", "bf16", extra_env={"IHB_MEGA_DELAY": f"1:{cta}:30000"})
        assert out["tokens"] == base["tokens"], (out, base)


@pytest.mark.parametrize("plan", ["ep", "hybrid"])
def test_expert_parallel_decode_in_the_persistent_kernel(plan):
    """Experts owned by ranks (full intermediate size), attention replicated (ep) or tensor-parallel (hybrid): the
    owners push their weighted expert outputs into every GPU's slot buffer, the same in-kernel combine as TP."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = _run(2, "auto", "bf16", plan)
    assert out["tokens"][0] == out["tokens"][1], out
    agree = sum(int(a == b) for a, b in zip(out["tokens"][0], out["ref"]))
    assert out["logits_rel_err"] < 0.02 and agree >= 11, out


@pytest.mark.parametrize("plan", ["tp", "ep", "hybrid"])
def test_batched_prompt_pass_on_two_gpus(plan):
    """The prompt through the batched window path (tensor-core GEMMs, device routing, fused all-reduce + norm) on two
    GPUs, tensor-, expert- and hybrid-parallel: logits and the tokens decoded after it against the one-GPU engine,
    whose prompt takes the same path."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = _run(2, "auto", "bf16", plan, extra_env={"IHB_TEST_WINDOW": "1"})
    assert out["tokens"][0] == out["tokens"][1], out
    agree = sum(int(a == b) for a, b in zip(out["tokens"][0], out["ref"]))
    assert out["logits_rel_err"] < 0.02 and agree >= 11, out


@pytest.mark.parametrize("plan", ["tp", "ep"])
def test_wide_build_of_the_persistent_kernel_on_two_gpus(plan):
    """The kernel build for large per-CTA shares (gate / up pairs with SwiGLU at the producer, 4-rows-per-warp shape),
    forced onto the small model: same checks as the default build."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = _run(2, "auto", "bf16", plan, extra_env={"IHB_MEGA_WIDE": "1"})
    assert out["tokens"][0] == out["tokens"][1], out
    agree = sum(int(a == b) for a, b in zip(out["tokens"][0], out["ref"]))
    assert out["logits_rel_err"] < 0.02 and agree >= 11, out


def test_several_tokens_per_launch_on_two_gpus():
    """``decode_many``: four tokens per cooperative launch on both GPUs (the in-kernel all-reduce rounds, slot clearing
    and the arg-max exchange run across token boundaries inside one launch); tokens as with one launch per token."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    base = _run(2, "auto", "bf16")
    out = _run(2, "auto", "bf16", extra_env={"IHB_TEST_MANY": "1"})
    assert out["tokens"][0] == out["tokens"][1], out
    assert out["tokens"] == base["tokens"], (out, base)
