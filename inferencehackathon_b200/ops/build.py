"""In-tree build of the native libraries with nvcc / g++ for sm_100a.

``libihb_kernels.so`` (CUDA kernels, plain C ABI, loaded with ctypes) and ``libihb_ctrl.so`` (C++ control
plane: speculative acceptance, tree builder, routing optimiser/predictors/scheduler) are written next to this
file so that they travel with the source tree. nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "csrc")
KERNEL_LIB = os.path.join(HERE, "libihb_kernels.so")
CTRL_LIB = os.path.join(HERE, "libihb_ctrl.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
# IHB_BUILD_DEFINES="-DIHB_MEGA_DETAIL" adds the detail time stamps of the persistent kernel (profiling builds)
NVCC_FLAGS += [f for f in os.environ.get("IHB_BUILD_DEFINES", "").split() if f.startswith("-D")]


def _sources(sub: str, exts) -> List[str]:
    d = os.path.join(CSRC, sub)
    if not os.path.isdir(d):
        return []
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(tuple(exts)))


def _digest(paths: List[str], extra: str) -> str:
    """Content hash of the sources (names relative to the source tree, so that a copy of the tree elsewhere with
    its built libraries is not rebuilt)."""
    h = hashlib.sha256(extra.encode())
    for p in paths:
        with open(p, "rb") as f:
            h.update(os.path.relpath(p, CSRC).encode())
            h.update(f.read())
    return h.hexdigest()


class _BuildLock:
    """Inter-process lock: the ranks of a multi-GPU job import the package at the same time and only one of them
    may (re)build; the others wait and then find the library up to date."""

    def __init__(self, name: str):
        self.path = os.path.join(HERE, name)
        self.f = None

    def __enter__(self):
        import fcntl
        self.f = open(self.path, "w")
        fcntl.flock(self.f, fcntl.LOCK_EX)
        return self

    def __exit__(self, *exc):
        import fcntl
        fcntl.flock(self.f, fcntl.LOCK_UN)
        self.f.close()


def _stale(lib: str, digest: str) -> bool:
    stamp = lib + ".stamp"
    if not os.path.exists(lib) or not os.path.exists(stamp):
        return True
    with open(stamp) as f:
        return f.read().strip() != digest


def _run(cmd: List[str]) -> None:
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: " + " ".join(cmd) + "\n" + r.stdout)


def build_kernels(force: bool = False, verbose: bool = False) -> str:
    srcs = _sources("kernels", (".cu",))
    deps = srcs + _sources("kernels", (".cuh", ".h", ".inc"))
    digest = _digest(deps, " ".join(NVCC_FLAGS))
    if not force and not _stale(KERNEL_LIB, digest):
        return KERNEL_LIB
    with _BuildLock(".build_kernels.lock"):
        if not force and not _stale(KERNEL_LIB, digest):      # another process built it while this one waited
            return KERNEL_LIB
        return _build_kernels_locked(srcs, digest, verbose)


def _build_kernels_locked(srcs: List[str], digest: str, verbose: bool) -> str:
    nvcc = os.environ.get("NVCC", "nvcc")
    objs = []
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    for s in srcs:
        o = os.path.join(objdir, os.path.basename(s) + ".o")
        objs.append(o)
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose:
            print(out)
        if p.returncode != 0:
            raise RuntimeError("build failed: " + " ".join(cmd) + "\n" + out)
    tmp = KERNEL_LIB + ".tmp"
    _run([nvcc, "-shared", "-o", tmp] + objs)          # no driver library: see tc_gemm.cu::encode_tiled_fn
    os.replace(tmp, KERNEL_LIB)                               # readers never see a half-written library
    with open(KERNEL_LIB + ".stamp", "w") as f:
        f.write(digest)
    return KERNEL_LIB


def build_ctrl(force: bool = False) -> str:
    srcs = _sources("ctrl", (".cpp",))
    if not srcs:
        return ""
    deps = srcs + _sources("ctrl", (".hpp", ".h"))
    flags = ["-O2", "-std=c++17", "-fPIC", "-shared", "-Wall"]
    digest = _digest(deps, " ".join(flags))
    if not force and not _stale(CTRL_LIB, digest):
        return CTRL_LIB
    with _BuildLock(".build_ctrl.lock"):
        if not force and not _stale(CTRL_LIB, digest):
            return CTRL_LIB
        tmp = CTRL_LIB + ".tmp"
        _run([os.environ.get("CXX", "g++")] + flags + srcs + ["-o", tmp])
        os.replace(tmp, CTRL_LIB)
        with open(CTRL_LIB + ".stamp", "w") as f:
            f.write(digest)
    return CTRL_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force, verbose)
    build_ctrl(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", KERNEL_LIB, CTRL_LIB if os.path.exists(CTRL_LIB) else "")
