"""Device and host time of the multi-token (prompt / verify) path on ONE GPU, with the weight shapes of one rank of a
tensor-parallel group (``tp > 1``: the all-reduces are skipped, so the numbers are timings, not numerics).

    python -m inferencehackathon_b200.runtime.window_profile LAYERS TP TOKENS [MODEL] [WEIGHTS] [REPS]

Prints ``WINDOW_PROFILE {json}``: CUDA-event milliseconds per pass, host wall milliseconds per pass (the difference
shows how far the path is bound by launches and host code), milliseconds per layer and the number of kernel launches
this package issued per pass. Run it under ``ncu --metrics gpu__time_duration.sum`` for the per-kernel list.
"""
import json
import sys
import time

import torch

from inferencehackathon_b200.config import EngineConfig, ParallelConfig, QuantConfig, get_model_config
from inferencehackathon_b200.models.weights import random_sharded_weights
from inferencehackathon_b200.parallel.collectives import Collectives
from inferencehackathon_b200.runtime.gpu_decoder import GpuDecoder


def main() -> None:
    layers, tp, tokens = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    model = sys.argv[4] if len(sys.argv) > 4 else "qwen3-235b-a22b"
    wts = sys.argv[5] if len(sys.argv) > 5 else "fp8_block"
    reps = int(sys.argv[6]) if len(sys.argv) > 6 else 3
    dev = torch.device("cuda:0")
    mcfg = get_model_config(model, layers)
    q = QuantConfig(weights=wts, kv="bf16")
    w = random_sharded_weights(mcfg, ParallelConfig(tp=tp, ep=1, rank=0, world=tp), q, dev, 0, 0)
    one = ParallelConfig(tp=1, ep=1, rank=0, world=1)
    cfg = EngineConfig(model=mcfg, parallel=one, quant=q, max_seq=tokens + 64, seed=0, backend="cuda")
    dec = GpuDecoder(cfg, w, Collectives(one), dev)
    win = dec.window()
    toks = torch.randint(0, mcfg.vocab, (tokens,), generator=torch.Generator().manual_seed(0)).to(dev)
    for _ in range(2):
        dec.reset()
        win.forward(toks, commit=True, last_only=True)
    torch.cuda.synchronize()
    ev, wall = [], []
    for _ in range(reps):
        dec.reset()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n0 = getattr(win, "n_launches", 0)
        t0 = time.perf_counter()
        e0.record()
        win.forward(toks, commit=True, last_only=True)
        e1.record()
        t1 = time.perf_counter()
        torch.cuda.synchronize()
        ev.append(e0.elapsed_time(e1))
        wall.append((t1 - t0) * 1e3)
        launches = getattr(win, "n_launches", 0) - n0
    out = {"ms_events": min(ev), "ms_host_enqueue": min(wall), "ms_per_layer": min(ev) / max(layers, 1),
           "package_launches_per_pass": launches,
           "cfg": dict(layers=layers, tp=tp, tokens=tokens, model=model, weights=wts)}
    print("WINDOW_PROFILE " + json.dumps(out))


if __name__ == "__main__":
    main()
