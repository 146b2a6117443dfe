"""Runs the tests of the C++ control plane against an AddressSanitizer + UndefinedBehaviorSanitizer build of it.

    python -m inferencehackathon_b200.ops.sanitize_ctrl [pytest arguments ...]

The library is compiled to a temporary file (the in-tree ``libihb_ctrl.so`` is not touched), the test process is
started with the sanitizer runtimes preloaded and ``IHB_CTRL_LIB`` pointing at the build; the first report ends the
run with a non-zero exit code. The GPU kernels have no such tool here (``compute-sanitizer`` is not available to
this project); their memory and ordering discipline is covered by reference comparisons, deterministic replay and
the protocol model tests.
"""
from __future__ import annotations

import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
DEFAULT_TESTS = ["tests/test_spec_native.py", "tests/test_routing_native.py", "tests/test_spec_driver.py"]


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    compilers = [c for c in dict.fromkeys([os.environ.get("CXX", ""), "g++", "c++"]) if c]
    srcs = sorted(os.path.join(HERE, "..", "csrc", "ctrl", f) for f in os.listdir(os.path.join(HERE, "..", "csrc", "ctrl"))
                  if f.endswith(".cpp"))
    with tempfile.TemporaryDirectory() as tmp:
        lib = os.path.join(tmp, "libihb_ctrl_san.so")
        cxx = None
        for cand in compilers:                       # not every compiler driver on a box ships the sanitizer runtimes
            r = subprocess.run([cand, "-O1", "-g", "-std=c++17", "-fPIC", "-shared", "-Wall", "-fsanitize=address,undefined",
                                "-fno-omit-frame-pointer"] + srcs + ["-o", lib], stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
            if r.returncode == 0:
                cxx = cand
                break
        if cxx is None:
            print("no compiler here can link the sanitizer runtimes")
            return 2
        runtimes = [subprocess.check_output([cxx, f"-print-file-name={n}"], text=True).strip()
                    for n in ("libasan.so", "libubsan.so")]
        env = dict(os.environ, IHB_CTRL_LIB=lib, LD_PRELOAD=":".join(runtimes),
                   ASAN_OPTIONS="detect_leaks=0:halt_on_error=1", UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1")
        cmd = [sys.executable, "-m", "pytest", "-x", "-q"] + (argv or DEFAULT_TESTS)
        return subprocess.call(cmd, cwd=ROOT, env=env)


if __name__ == "__main__":
    raise SystemExit(main())
