"""``python -m inferencehackathon_b200 <command>``: one-process front door to the engine.

  generate   build an engine (random weights of a named architecture, or a safetensors checkpoint directory), run one
             prompt through prefill + decode and print the text with TTFT and decode rate
  info       model presets, where the native libraries are and whether they are built

Multi-GPU runs start one process per GPU with ``python -m torch.distributed.run`` (see ``bench.py`` and ``parallel/launch.py``);
this command is the single-rank path a user tries first.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def _generate(a) -> int:
    import torch
    from .runtime.engine import InferenceEngine
    from .runtime.sampler import SamplingParams
    from .serve.tokenizer import ByteTokenizer, HFTokenizer
    weights = a.weights or ("fp32" if a.device == "cpu" else "fp8_block")
    eng = InferenceEngine.build(a.model, weights=weights, kv=a.kv, device=a.device, max_seq=a.max_seq, n_layers=a.layers,
                                checkpoint=a.checkpoint, seed=a.seed)
    tok = HFTokenizer(a.tokenizer) if a.tokenizer else ByteTokenizer(eng.cfg.model.vocab)
    prompt = tok.encode(a.prompt)
    room = eng.cfg.max_seq - len(prompt) - 1
    if room < 1:
        print(f"the prompt has {len(prompt)} tokens; --max-seq {a.max_seq} leaves no room to generate", file=sys.stderr)
        return 2
    eng.set_sampling(SamplingParams(temperature=a.temperature, top_p=a.top_p, seed=a.seed))
    res = eng.generate(prompt, min(a.max_new, room))
    if eng.gpu is not None:
        eng.gpu.check_error()
        torch.cuda.synchronize()
    out = {"model": eng.cfg.model.name, "device": str(eng.device), "backend": eng.backend, "weights": weights,
           "kv": eng.cfg.quant.kv, "prompt_tokens": len(prompt), "new_tokens": len(res.tokens),
           "ttft_ms": round(1e3 * res.ttft_s, 3), "decode_tok_per_s": round(res.decode_tok_per_s, 1),
           "text": tok.decode(res.tokens)}
    if a.json:
        print(json.dumps(out))
    else:
        print(out["text"])
        print(f"[{out['model']} on {out['device']} ({out['backend']}, {weights} weights, {out['kv']} KV): "
              f"{out['prompt_tokens']} prompt tokens, TTFT {out['ttft_ms']} ms, {out['new_tokens']} tokens at "
              f"{out['decode_tok_per_s']} tok/s]", file=sys.stderr)
    return 0


def _info(_a) -> int:
    from . import config
    from .ops import build
    here = os.path.dirname(os.path.abspath(build.__file__))
    libs = {name: os.path.exists(os.path.join(here, name)) for name in ("libihb_kernels.so", "libihb_ctrl.so")}
    presets = {}
    for name in ("tiny", "small", "qwen3-30b-a3b", "qwen3-235b-a22b"):
        m = config.get_model_config(name)
        presets[name] = {"layers": m.n_layers, "hidden": m.hidden, "q_heads": m.n_q_heads, "kv_heads": m.n_kv_heads,
                         "head_dim": m.head_dim, "experts": m.n_experts, "top_k": m.top_k, "expert_inter": m.moe_inter,
                         "vocab": m.vocab, "params_b": round(m.total_params() / 1e9, 3)}
    print(json.dumps({"native_libraries": libs, "library_dir": here, "presets": presets}, indent=1))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m inferencehackathon_b200", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="one prompt through prefill + decode")
    g.add_argument("--model", default="tiny")
    g.add_argument("--prompt", default="Mixture-of-experts decoding at batch one is a latency problem.")
    g.add_argument("--max-new", type=int, default=32)
    g.add_argument("--device", default="cpu")
    g.add_argument("--weights", default="", choices=["", "fp32", "bf16", "fp8_block"])
    g.add_argument("--kv", default=None, choices=[None, "fp32", "bf16", "fp8"])
    g.add_argument("--max-seq", type=int, default=1024)
    g.add_argument("--layers", type=int, default=None, help="truncate the layer count")
    g.add_argument("--checkpoint", default=None, help="directory of Hugging Face safetensors shards")
    g.add_argument("--tokenizer", default=None, help="Hugging Face tokenizer directory (default: reversible byte mapping)")
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--json", action="store_true")
    sub.add_parser("info", help="presets and native libraries")
    a = ap.parse_args(argv)
    return _generate(a) if a.cmd == "generate" else _info(a)


if __name__ == "__main__":
    raise SystemExit(main())
