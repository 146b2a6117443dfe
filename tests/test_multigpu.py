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
eng = InferenceEngine.build("small", tp=tp, ep=ep, rank=rank, world=world, weights=weights, device=dev, backend="cuda", max_seq=128)
res = eng.generate(prompt, 12)
eng.gpu.check_error()
ref_tokens = None
if rank == 0:
    ref = InferenceEngine.build("small", weights=weights, device=dev, backend="cuda", max_seq=128)
    ref_tokens = ref.generate(prompt, 12).tokens
toks = [None] * world
dist.all_gather_object(toks, res.tokens)
if rank == 0:
    print("RESULT " + json.dumps({"tokens": toks, "ref": ref_tokens, "mc": bool(eng.gpu.symm.use_multicast)}))
dist.barrier()
dist.destroy_process_group()
"""


def _run(n, mode, weights, plan="tp"):
    env = dict(os.environ, IHB_ROOT=ROOT, IHB_COMM_MODE=mode, IHB_TEST_WEIGHTS=weights, IHB_TEST_PLAN=plan)
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
    # TP changes the summation order (and, for fp8, the quantisation blocks of the shards)
    assert agree >= (9 if weights == "bf16" else 4), out


@pytest.mark.parametrize("plan", ["ep", "hybrid"])
def test_expert_parallel_decode_in_the_persistent_kernel(plan):
    """Experts owned by ranks (full intermediate size), attention replicated (ep) or tensor-parallel (hybrid): the
    owners push their weighted expert outputs into every GPU's slot buffer, the same in-kernel combine as TP."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = _run(2, "auto", "bf16", plan)
    assert out["tokens"][0] == out["tokens"][1], out
    agree = sum(int(a == b) for a, b in zip(out["tokens"][0], out["ref"]))
    assert agree >= 9, out
