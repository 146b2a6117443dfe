"""Builds the reference's own decode drivers, unmodified, for sm_100a into ``baseline/_ref/bin``.

``baseline/_ref`` (git-ignored) holds (a) the reference's Python package installed with
``pip install --no-index --target baseline/_ref <copy of the reference>`` and (b) a verbatim copy of its
``kernels/`` directory, compiled here with the build lines from the sources' own headers
(kernels/decode_step.cu "Build" comment, kernels/decode_step_tp8.cu:65-72) with ``-arch=sm_100a`` in place of
``sm_90a``. The binaries are the reference's public entry points: ``main(ctx_len, iters, HBM_GBs[, run_check])``.
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


if __name__ == "__main__":
    build(*sys.argv[1:])
    print("built", os.listdir(os.path.join(REF, "bin")))
