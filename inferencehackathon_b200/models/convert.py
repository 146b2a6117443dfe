"""Command line: Hugging Face Qwen3-MoE safetensors (bf16 or fp8 with ``weight_scale_inv``) -> this engine's sharded
on-disk layout, one directory per rank.

    python -m inferencehackathon_b200.models.convert --src /path/to/hf_checkpoint --dst /path/to/out \\
        --model qwen3-235b-a22b --tp 8 [--ep 1] [--weights fp8_block|bf16] [--layers N]

Each rank directory holds a manifest plus raw tensors (QKV fused, gate/up stacked per expert, block scales
re-cut for the shard, router in bf16) that ``models.weights.load_engine_layout`` maps straight into device memory.
Reference: tools/conifer_weight_convert.py:8-19,40-47,65-99.
"""
from __future__ import annotations

import argparse
import os
import sys

from ..config import ParallelConfig, QuantConfig, get_model_config
from .weights import save_engine_layout, shard_state_dict


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--src", required=True, help="directory with *.safetensors (HF names)")
    ap.add_argument("--dst", required=True)
    ap.add_argument("--model", default="qwen3-235b-a22b")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--weights", default="fp8_block", choices=["fp8_block", "bf16", "fp32"])
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--ranks", type=int, nargs="*", default=None, help="convert only these ranks")
    a = ap.parse_args(argv)
    mcfg = get_model_config(a.model, a.layers)
    world = max(a.tp, a.ep) if a.tp == 1 or a.ep == 1 else a.tp * a.ep
    q = QuantConfig(weights=a.weights, kv="fp32" if a.weights == "fp32" else "bf16")
    for rank in (a.ranks if a.ranks else range(world)):
        par = ParallelConfig(tp=a.tp, ep=a.ep, rank=rank, world=world)
        par.validate(mcfg)
        w = shard_state_dict(a.src, mcfg, par, q, device="cpu")
        out = os.path.join(a.dst, f"rank{rank:02d}")
        save_engine_layout(w, out)
        print(f"rank {rank}: {out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
