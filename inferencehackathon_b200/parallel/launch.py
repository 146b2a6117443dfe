"""Process launch and ``torch.distributed`` initialisation: one process per rank (gloo on CPU, NCCL on GPU).

The reference runs all eight GPUs from one process with a host thread per rank
(kernels/decode_step_tp8.cu:1327-1338, 2862); with a process per GPU the ordering hazards of that model
(kernels/decode_step_tp8.cu:1142-1154) do not arise.
"""
from __future__ import annotations

import datetime
import os
import socket
import traceback
from typing import Any, Callable, List, Optional

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def init_distributed(backend: Optional[str] = None, timeout_s: float = 600.0) -> tuple:
    """Initialise from the ``torchrun`` environment. Returns ``(rank, world, local_rank)``; a no-op when
    ``WORLD_SIZE`` is unset or 1."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world == 1:
        return 0, 1, local
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(local)
    if not dist.is_initialized():
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return rank, world, local


def _worker(rank: int, world: int, port: int, fn: Callable, args: tuple, q, timeout_s: float) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    try:
        torch.set_num_threads(max(1, (os.cpu_count() or 2) // world))
        dist.init_process_group("gloo", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s))
        out = fn(rank, world, *args)
        q.put((rank, "ok", out))
    except BaseException as e:  # reported to the parent, which raises
        q.put((rank, "error", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
    finally:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


def run_cpu_ranks(fn: Callable, world: int, args: tuple = (), timeout_s: float = 120.0,
                  expect_failures: bool = False) -> List[Any]:
    """Run ``fn(rank, world, *args)`` in ``world`` gloo processes; returns the per-rank results in rank order.

    With ``expect_failures`` a rank's error (or a rank that never reports) is returned as
    ``("error", message)`` instead of raising: the host-side failure-detection tests use this."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, args, q, timeout_s)) for r in range(world)]
    for p in procs:
        p.start()
    results: dict = {}
    try:
        for _ in range(world):
            try:
                rank, status, payload = q.get(timeout=timeout_s + 30)
            except Exception:
                break
            results[rank] = (status, payload)
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.terminate()                      # exact child we started
                p.join(timeout=5)
    out = []
    for r in range(world):
        status, payload = results.get(r, ("error", "rank did not report"))
        if status != "ok" and not expect_failures:
            raise RuntimeError(f"rank {r} failed: {payload}")
        out.append(payload if status == "ok" else ("error", payload))
    return out
