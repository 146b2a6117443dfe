"""Stress and precision of the stand-alone fused all-reduce kernel over peer memory (needs >= 2 B200s; one process per
GPU): 100 rounds with a rank-skewed busy kernel before each pair of back-to-back all-reduces and no host
synchronisation between collectives, for the one-shot, the two-shot and the counted fixed-point variant, then a precision probe with fractional data against a float64 sum. The same
protocol the reference uses for its multicast all-reduce (kernels/nvls_engine_test.cu:46-68,
kernels/nvls_precision_test.cu:15-51)."""
import json
import os
import subprocess
import sys
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys, json, torch
sys.path.insert(0, os.environ["IHB_ROOT"])
import torch.distributed as dist
from inferencehackathon_b200.config import ParallelConfig
from inferencehackathon_b200.ops import lib as K
from inferencehackathon_b200.parallel.launch import init_distributed
from inferencehackathon_b200.parallel.symm import SymmetricComm
rank, world, local = init_distributed()
dev = torch.device("cuda", local)
K.load()
T, H = 4, 1024
par = ParallelConfig(tp=world, ep=1, rank=rank, world=world)
comm = SymmetricComm(par, dev, slot_floats=2 * world * T * H, extra_bytes=4 * 64 * H * 8)
epoch = torch.zeros(4, dtype=torch.int32, device=dev)
counter = torch.zeros(8, dtype=torch.int32, device=dev)
err = torch.zeros(1, dtype=torch.int32, device=dev)
cm = comm.comm_block(epoch)
cm_small = comm.comm_block(epoch, slot_offset_bytes=comm.extra_off)     # the counted variant keeps its own slot region
calls = torch.zeros(64, dtype=torch.int32, device=dev)
def counted(src, dst):
    K.allreduce_counted(cm_small, src, dst, counter, calls, err)
def plain(algo):
    return lambda src, dst: K.allreduce_norm(cm, src, dst, counter, err, algo=algo)
res = {"mode": "multicast" if comm.use_multicast else "p2p"}
for name, ar in (("oneshot", plain(1)), ("twoshot", plain(2)), ("counted", counted)):
    bad = 0
    x, a, b = torch.empty(T, H, device=dev), torch.empty(T, H, device=dev), torch.empty(T, H, device=dev)
    for rnd in range(100):
        x.fill_(float(rnd % 7 + rank + 1))
        torch.cuda._sleep(200000 * ((rank + rnd) % world))          # skew: ranks reach the collective at different times
        ar(x, a)
        ar(a, b)                                                     # second collective right behind the first
        want1 = float(sum(rnd % 7 + r + 1 for r in range(world)))
        bad += int((a != want1).any()) + int((b != want1 * world).any())
    torch.cuda.synchronize(dev)
    res[name + "_bad_rounds"] = bad
    res[name + "_err"] = int(err.item())
    err.zero_()
    # precision: fractional data, every rank different; reference in float64 on the host
    g = torch.Generator().manual_seed(17)
    parts = [torch.rand(T, H, generator=g, dtype=torch.float64) * 2 - 1 for _ in range(world)]
    mine = parts[rank].float().to(dev)
    out = torch.empty(T, H, device=dev)
    ar(mine, out)
    torch.cuda.synchronize(dev)
    exact = sum(p.float().double() for p in parts)
    res[name + "_max_abs_err"] = float((out.double().cpu() - exact).abs().max())
    # every rank must hold the same bits
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out)
    res[name + "_identical_on_all_ranks"] = all(torch.equal(gathered[0], t) for t in gathered)
out = [None] * world
dist.all_gather_object(out, res)
if rank == 0:
    print("RESULT " + json.dumps(out))
dist.barrier()
dist.destroy_process_group()
"""


@pytest.mark.parametrize("mode", ["p2p"])
def test_fused_allreduce_survives_skewed_back_to_back_rounds(mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    n = min(4, torch.cuda.device_count())
    env = dict(os.environ, IHB_ROOT=ROOT, IHB_COMM_MODE=mode, NCCL_NVLS_ENABLE="0")
    with tempfile.NamedTemporaryFile("w", suffix=".py", delete=False) as f:
        f.write(WORKER)
        path = f.name
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29547", path]
    r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    os.unlink(path)
    assert r.returncode == 0, r.stdout[-3000:]
    out = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    for res in out:
        for name in ("oneshot", "twoshot", "counted"):
            assert res[name + "_bad_rounds"] == 0 and res[name + "_err"] == 0, out
            assert res[name + "_max_abs_err"] < 1e-5 * n, out
            assert res[name + "_identical_on_all_ranks"], out
