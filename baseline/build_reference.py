"""Builds the reference's own decode drivers, unmodified, for sm_100a into ``baseline/_ref/bin``.

``baseline/_ref`` (git-ignored) holds (a) the reference's Python package installed with
``pip install --no-index --target baseline/_ref <copy of the reference>`` and (b) a verbatim copy of its
``kernels/`` directory, compiled here with the build lines from the sources' own headers
(kernels/decode_step.cu "Build" comment, kernels/decode_step_tp8.cu:65-72) with ``-arch=sm_100a`` in place of
``sm_90a``. The binaries are the reference's public entry points: ``main(ctx_len, iters, HBM_GBs[, run_check])``.

Also built: two of the reference's single-process 8-GPU microbenches, for same-box comparison rows:
``nvls_ar`` (kernels/nvls_ar.cu: one multimem ld_reduce + st kernel over an 8 KB fp16 vector, no flags, no waits) and
``ep_moe_sharded`` (kernels/ep_moe_sharded.cu: expert-parallel MoE layer with balanced / skewed / adversarial routing,
combined by ncclAllReduce). ``python baseline/build_reference.py --run-comms`` runs both on an 8-GPU box and prints
their result lines. kernels/oneshot_allreduce.cu is NOT built or run: its device code spins on peer flags without
a bound (kernels/oneshot_allreduce.cu:152), so one rank that fails to launch would hang the other seven GPUs.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def nccl_dirs():
    import importlib.util
    spec = importlib.util.find_spec("nvidia.nccl")
    base = list(spec.submodule_search_locations)[0]
    return os.path.join(base, "include"), os.path.join(base, "lib")


def build(reference_root: str = "") -> None:
    reference_root = reference_root or os.environ.get("REFERENCE_ROOT", "")
    if not os.path.isdir(os.path.join(reference_root, "kernels")) and not os.path.isdir(os.path.join(REF, "kernels")):
        raise SystemExit("usage: python baseline/build_reference.py <path of the reference checkout> (or REFERENCE_ROOT)")
    os.makedirs(os.path.join(REF, "bin"), exist_ok=True)
    kdir = os.path.join(REF, "kernels")
    if not os.path.isdir(kdir):
        shutil.copytree(os.path.join(reference_root, "kernels"), kdir)
    inc, lib = nccl_dirs()
    common = ["nvcc", "-arch=sm_100a", "-O3", "--use_fast_math", "-I", kdir]
    subprocess.check_call(common + [os.path.join(kdir, "decode_step.cu"), "-o", os.path.join(REF, "bin", "decode_step")])
    subprocess.check_call(common + ["-I", inc, os.path.join(kdir, "decode_step_tp8.cu"), "-L", lib, "-l:libnccl.so.2",
                                    "-lcublasLt", "-lcuda", "-o", os.path.join(REF, "bin", "decode_step_tp8")])
    subprocess.check_call(common + [os.path.join(kdir, "nvls_ar.cu"), "-lcuda", "-o", os.path.join(REF, "bin", "nvls_ar")])
    subprocess.check_call(common + ["-I", inc, os.path.join(kdir, "ep_moe_sharded.cu"), "-L", lib, "-l:libnccl.so.2",
                                    "-o", os.path.join(REF, "bin", "ep_moe_sharded")])


def run_comms(timeout_s: int = 600) -> dict:
    """Runs the two microbenches and returns their headline lines (``{"nvls_ar": [...], "ep_moe_sharded": [...]}``). A
    program that does not finish within ``timeout_s`` is reported as such and the other one's result is kept (on the
    8-GPU box of this pool ``ep_moe_sharded`` did not finish within 180 s)."""
    _, lib = nccl_dirs()
    env = dict(os.environ, LD_LIBRARY_PATH=lib + ":" + os.environ.get("LD_LIBRARY_PATH", ""))
    out = {}
    for name, keys in (("nvls_ar", ("validate", "C =")), ("ep_moe_sharded", ("balanced", "skewed", "adversarial", "per-token"))):
        exe = os.path.join(REF, "bin", name)
        if not os.path.exists(exe):
            out[name] = ["not built"]
            continue
        try:
            r = subprocess.run([exe], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout_s)
        except subprocess.TimeoutExpired as e:
            tail = (e.stdout or b"")
            tail = tail.decode(errors="replace") if isinstance(tail, bytes) else tail
            out[name] = [f"not finished after {timeout_s} s"] + tail.splitlines()[-5:]
            continue
        lines = [l.strip() for l in r.stdout.splitlines() if any(k in l for k in keys)]
        out[name] = lines if r.returncode == 0 else [f"exit {r.returncode}"] + r.stdout.splitlines()[-5:]
    return out


if __name__ == "__main__":
    if "--run-comms" in sys.argv[1:]:
        import json
        print(json.dumps(run_comms(), indent=1))
    else:
        build(*sys.argv[1:])
        print("built", os.listdir(os.path.join(REF, "bin")))
