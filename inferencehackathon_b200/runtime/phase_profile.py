"""Per-phase device times of the persistent decode kernel on ONE GPU, with the weight shapes of one rank of a
tensor-parallel group (``tp > 1``: the all-reduce sums only this rank's partial, so the numbers are timings, not
numerics; the cross-GPU barrier is not part of them).

    python -m inferencehackathon_b200.runtime.phase_profile LAYERS TP CTX [MODEL] [WEIGHTS] [LOOPBACK]

Prints ``MEGA_PHASES {json}``: microseconds per phase averaged over layers (CTA 0's %globaltimer stamps, and under
``last`` the latest stamp of any CTA per phase) and the CUDA-event time per token. ``LOOPBACK`` = k > 1 makes every
all-reduce slot receive k adds, the slot traffic of k ranks on one GPU.
"""
import os, sys, json, torch
os.environ["IHB_MEGA_PROF"] = "1"
if len(sys.argv) > 6:
    os.environ["IHB_MEGA_LOOPBACK"] = sys.argv[6]
from inferencehackathon_b200.config import get_model_config, ParallelConfig, QuantConfig, EngineConfig
from inferencehackathon_b200.models.weights import random_sharded_weights
from inferencehackathon_b200.runtime.gpu_decoder import GpuDecoder
from inferencehackathon_b200.parallel.collectives import Collectives
layers = int(sys.argv[1]); tp = int(sys.argv[2]); ctx = int(sys.argv[3])
model = sys.argv[4] if len(sys.argv) > 4 else "qwen3-235b-a22b"
wts = sys.argv[5] if len(sys.argv) > 5 else "fp8_block"
dev = torch.device("cuda:0")
mcfg = get_model_config(model, layers)
q = QuantConfig(weights=wts, kv="bf16")
w = random_sharded_weights(mcfg, ParallelConfig(tp=tp, ep=1, rank=0, world=tp), q, dev, 0, 0)
one = ParallelConfig(tp=1, ep=1, rank=0, world=1)
cfg = EngineConfig(model=mcfg, parallel=one, quant=q, max_seq=ctx + 64, seed=0, backend="cuda")
dec = GpuDecoder(cfg, w, Collectives(one), dev)
dec.pos.fill_(ctx); dec.cur_token.fill_(5)
for _ in range(5):
    dec._step()
torch.cuda.synchronize()
e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
e0.record()
for _ in range(20):
    dec._step()
e1.record(); torch.cuda.synchronize()
dec.check_error()
ph = dec.mega_phase_us()
ph["last"] = dec.mega_phase_us("last")
ph["detail"] = dec.mega_detail_us()
ph["ms_per_step_events"] = e0.elapsed_time(e1) / 20
ph["cfg"] = dict(layers=layers, tp=tp, ctx=ctx, model=model, weights=wts, grid=dec.mega_grid,
                 loopback=int(os.environ.get("IHB_MEGA_LOOPBACK", "0")))
print("MEGA_PHASES " + json.dumps(ph))
