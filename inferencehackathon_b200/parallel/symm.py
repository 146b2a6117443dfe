"""Symmetric (peer-mapped + NVLS multicast) memory for the fused compute+collective kernels.

Every rank allocates the same buffer; after the rendezvous each rank holds (a) its own pointer, (b) every peer's
buffer mapped into its address space and (c) one multicast address whose stores NVSwitch replicates into all
ranks' copies. The kernels use them directly: partial GEMV outputs are pushed with ``multimem.st`` (or per-peer
stores), a monotonic arrival counter is bumped with ``multimem.red.release`` and polled locally with a bounded
spin. Allocation and handle exchange across processes go through ``torch.distributed._symmetric_memory``
(CUDA VMM + fd passing); the reference does the same by hand inside one process
(kernels/nvls_engine.cuh:207-303) and, for vLLM workers, by re-opening ``/proc/<pid>/fd``
(tools/patch_vllm_nvls.py:253-350).
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from ..config import ParallelConfig
from ..ops import lib as K

_FLAG_BYTES = 256
_ARG_BYTES = 256


class SymmetricComm:
    def __init__(self, par: ParallelConfig, device: torch.device, slot_floats: int, group=None,
                 extra_bytes: int = 0):
        import torch.distributed._symmetric_memory as symm_mem
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised (backend nccl) before SymmetricComm")
        self.par, self.device = par, device
        self.group = group if group is not None else dist.group.WORLD
        self.nranks = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.nranks > K.MAX_RANKS:
            raise ValueError(f"at most {K.MAX_RANKS} ranks")
        self.slot_bytes = (slot_floats * 4 + 255) // 256 * 256
        self.extra_off = self.slot_bytes + _FLAG_BYTES + _ARG_BYTES
        total = self.extra_off + (extra_bytes + 255) // 256 * 256
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.buf.zero_()
        torch.cuda.synchronize(device)
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        mc = 0
        try:
            mc = int(self.handle.multicast_ptr or 0)
        except Exception:
            mc = 0
        mode = os.environ.get("IHB_COMM_MODE", "auto")
        self.use_multicast = bool(mc) and mode in ("auto", "mc")
        if mode == "mc" and not mc:
            raise RuntimeError("IHB_COMM_MODE=mc but the symmetric buffer has no multicast mapping")
        self.mc_ptr = mc if self.use_multicast else 0
        self.local_ptr = self.buf.data_ptr()
        self.slots_local = self.buf[: slot_floats * 4].view(torch.float32)
        self.barrier_host()

    def barrier_host(self) -> None:
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def comm_block(self, epoch: torch.Tensor, slot_offset_bytes: int = 0) -> K.IhbComm:
        """The kernels' view of this buffer. ``slot_offset_bytes`` (a multiple of 16) moves the slot pointers into the
        buffer, e.g. to the caller-defined tail region (``self.extra_off``): kernels that keep different slot layouts
        must not share storage."""
        cm = self._comm_block(epoch)
        if slot_offset_bytes:
            cm.slots_local = self.local_ptr + slot_offset_bytes
            if self.use_multicast:
                cm.slots_mc = self.mc_ptr + slot_offset_bytes
            for r in range(self.nranks):
                cm.slots_peer[r] = self.peer_ptrs[r] + slot_offset_bytes
        return cm

    def _comm_block(self, epoch: torch.Tensor) -> K.IhbComm:
        cm = K.IhbComm()
        cm.nranks, cm.rank = self.nranks, self.rank
        f_off, a_off = self.slot_bytes, self.slot_bytes + _FLAG_BYTES
        cm.slots_local = self.local_ptr
        cm.flag_local = self.local_ptr + f_off
        cm.arg_slots_local = self.local_ptr + a_off
        if self.use_multicast:
            cm.slots_mc, cm.flag_mc, cm.arg_slots_mc = self.mc_ptr, self.mc_ptr + f_off, self.mc_ptr + a_off
        for r in range(self.nranks):
            cm.slots_peer[r] = self.peer_ptrs[r]
            cm.flag_peer[r] = self.peer_ptrs[r] + f_off
            cm.arg_slots_peer[r] = self.peer_ptrs[r] + a_off
        cm.epoch = epoch.data_ptr()
        return cm

    def extra(self, nbytes: int, offset: int = 0) -> torch.Tensor:
        """View of the caller-defined tail region of the local buffer."""
        return self.buf[self.extra_off + offset: self.extra_off + offset + nbytes]

    def reset(self, epoch: torch.Tensor) -> None:
        """Bring all ranks back to the initial state (arrival counter and epoch zero); collective."""
        self.barrier_host()
        self.buf[: self.extra_off].zero_()          # slots too: tagged slots must not survive an epoch restart
        epoch.zero_()
        self.barrier_host()
