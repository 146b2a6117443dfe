"""All-to-all exchange of rows over peer memory (expert-parallel dispatch / combine) against the NCCL path: needs
>= 2 B200s; spawns one process per GPU."""
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
from inferencehackathon_b200.parallel.launch import init_distributed
from inferencehackathon_b200.parallel.a2a import PeerRowExchange
from inferencehackathon_b200.parallel.collectives import Collectives
from inferencehackathon_b200.config import ParallelConfig
from inferencehackathon_b200.runtime.engine import InferenceEngine
rank, world, local = init_distributed()
dev = torch.device("cuda", local)
par = ParallelConfig(tp=1, ep=world, rank=rank, world=world)
ref = Collectives(par)
W, CAP = 72, 48
ex = PeerRowExchange(dev, W, CAP)
ok_rows, ok_gather = True, True
for rnd in range(5):
    g = torch.Generator().manual_seed(100 * rnd + rank)
    counts = torch.randint(0, CAP + 1, (world,), generator=g).tolist()
    if rnd == 3:
        counts = [0] * world                                   # an empty round
    P = sum(counts)
    rows = torch.randn(P, W, generator=g).to(dev)
    want, wc = ref.all_to_all_rows(rows, counts)
    got, gc = ex.exchange(rows, counts)
    ok_rows = ok_rows and gc == wc and torch.equal(got, want)
    # fused gather: an unsorted matrix and the list of source rows in destination order
    perm = torch.randperm(P, generator=g) if P else torch.zeros(0, dtype=torch.long)
    base = torch.empty_like(rows)
    base[perm.to(dev)] = rows
    got2, gc2 = ex.exchange(base, counts, gather=perm.to(dev).to(torch.int32))
    ok_gather = ok_gather and gc2 == wc and torch.equal(got2, want)
# the expert-parallel model forward (several tokens, so each rank routes only its own) with either exchange
prompt = torch.randint(0, 2048, (9,), generator=torch.Generator().manual_seed(5)).tolist()
eng = InferenceEngine.build("tiny", tp=1, ep=world, rank=rank, world=world, device=dev, backend="torch", max_seq=64)
la = eng.prefill(prompt, return_logits=True).logits.float().cpu()
eng.reset()
m = eng.cfg.model
eng.model.comm.fast_a2a = PeerRowExchange(dev, (m.hidden + 2 + 3) // 4 * 4, 9 * m.top_k)
n0 = eng.model.comm.n_collectives
lb = eng.prefill(prompt, return_logits=True).logits.float().cpu()
used = eng.model.comm.fast_a2a.round
res = {"rows": ok_rows, "gather": ok_gather, "model_max_diff": float((la - lb).abs().max()), "fast_rounds": used}
out = [None] * world
dist.all_gather_object(out, res)
if rank == 0:
    print("RESULT " + json.dumps(out))
dist.barrier()
dist.destroy_process_group()
"""


def test_peer_row_exchange_matches_nccl_all_to_all():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, IHB_ROOT=ROOT, NCCL_NVLS_ENABLE="0", IHB_A2A="0")      # the test installs the exchange itself
    with tempfile.NamedTemporaryFile("w", suffix=".py", delete=False) as f:
        f.write(WORKER)
        path = f.name
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29541", path]
    r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    os.unlink(path)
    assert r.returncode == 0, r.stdout[-3000:]
    out = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    for rank_res in out:
        assert rank_res["rows"] and rank_res["gather"], out
        assert rank_res["model_max_diff"] < 1e-4, out
        assert rank_res["fast_rounds"] == 2 * 4, out          # dispatch + combine in each of the tiny model's 4 layers
