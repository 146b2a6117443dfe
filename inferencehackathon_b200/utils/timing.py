"""Device-side timing helpers: CUDA events on the launching stream, max over ranks, L2 flush.

The reference times only rank 0's events with a stream synchronise per iteration
(kernels/decode_step_tp8.cu:2937-2958); multi-GPU numbers here are always the maximum over ranks."""
from __future__ import annotations

import time
from typing import Callable, List, Optional

import torch


class StepTimer:
    """Times a region in seconds: CUDA events when ``device`` is a GPU, ``perf_counter`` otherwise."""

    def __init__(self, device):
        self.cuda = torch.device(device).type == "cuda"
        if self.cuda:
            self._e0 = torch.cuda.Event(enable_timing=True)
            self._e1 = torch.cuda.Event(enable_timing=True)
        self._t0 = 0.0

    def start(self) -> None:
        if self.cuda:
            self._e0.record()
        else:
            self._t0 = time.perf_counter()

    def stop(self) -> float:
        if self.cuda:
            self._e1.record()
            self._e1.synchronize()
            return self._e0.elapsed_time(self._e1) * 1e-3
        return time.perf_counter() - self._t0


class L2Flusher:
    """Writes a buffer larger than the 126 MB L2 so that the next timed launch starts cold."""

    def __init__(self, device, nbytes: int = 256 << 20):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)

    def flush(self) -> None:
        self.buf.fill_(1)


def time_cuda(fn: Callable[[], None], iters: int = 20, warmup: int = 3, flusher: Optional[L2Flusher] = None) -> List[float]:
    """Per-iteration seconds of ``fn`` measured with CUDA events, after ``warmup`` untimed calls."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        if flusher is not None:
            flusher.flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        out.append(e0.elapsed_time(e1) * 1e-3)
    return out


def max_over_ranks(value: float, device=None) -> float:
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
