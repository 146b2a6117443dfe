"""All-to-all exchange of rows over peer memory (expert-parallel dispatch / combine of multi-token windows).

``PeerRowExchange`` owns a symmetric receive region ``[2][world][cap][row_floats]`` and runs ONE kernel per exchange
(``csrc/kernels/a2a.cu``): rows go straight into the destination GPU's memory with peer stores, counts travel beside
them, one arrive / bounded wait ends the round. It has the interface of ``Collectives.all_to_all_rows`` and can be
installed there (``Collectives.fast_a2a``); the NCCL ``all_to_all_single`` path stays as the reference and for CPU.
Reference counterpart: the NVSHMEM put-based all-to-all (kernels/nvshmem_comms.cu:170-191).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import lib as K


class PeerRowExchange:
    def __init__(self, device: torch.device, row_floats: int, cap: int, group=None, grid: int = 32):
        import torch.distributed._symmetric_memory as symm_mem
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised (backend nccl) before PeerRowExchange")
        if row_floats % 4:
            raise ValueError("row_floats must be a multiple of 4 (16-byte pieces)")
        self.device, self.row_floats, self.cap, self.grid = device, row_floats, cap, grid
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > K.MAX_RANKS:
            raise ValueError(f"at most {K.MAX_RANKS} ranks")
        self.recv_bytes = 2 * self.world * cap * row_floats * 4
        self.count_off = (self.recv_bytes + 255) // 256 * 256
        self.flag_off = self.count_off + 256
        total = self.flag_off + 256
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.buf.zero_()
        torch.cuda.synchronize(device)
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.recv = self.buf[: self.recv_bytes].view(torch.float32).view(2, self.world, cap, row_floats)
        self.counts = self.buf[self.count_off: self.count_off + 2 * self.world * 4].view(torch.int32).view(2, self.world)
        self.err = torch.zeros(1, dtype=torch.int32, device=device)
        self.round = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)

    def exchange(self, rows: torch.Tensor, send_counts, gather: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, List[int]]:
        """``rows [P, row_floats]`` fp32 ordered by destination (or any matrix plus ``gather [P]`` int32 giving the
        source row of each pair in destination order); ``send_counts[d]`` rows go to rank ``d``. Returns the received
        rows ordered by source rank and the per-source counts."""
        if rows.dtype != torch.float32 or rows.shape[-1] != self.row_floats:
            raise ValueError("rows must be fp32 [P, row_floats]")
        sc = torch.as_tensor(send_counts, dtype=torch.int32)
        if int(sc.max()) > self.cap:
            raise ValueError(f"{int(sc.max())} rows for one rank exceed the slot capacity {self.cap}")
        offsets = torch.zeros(self.world + 1, dtype=torch.int32)
        offsets[1:] = torch.cumsum(sc, 0)
        offsets = offsets.to(self.device, non_blocking=True)
        rows = rows.contiguous()
        a = K.IhbA2AArgs()
        a.nranks, a.rank, a.row_floats, a.cap, a.round = self.world, self.rank, self.row_floats, self.cap, self.round
        a.send, a.offsets = rows.data_ptr(), offsets.data_ptr()
        a.gather = gather.data_ptr() if gather is not None else None
        for r in range(self.world):
            a.recv_peer[r] = self.peer_ptrs[r]
            a.count_peer[r] = self.peer_ptrs[r] + self.count_off
            a.flag_peer[r] = self.peer_ptrs[r] + self.flag_off
        a.flag_local = self.buf.data_ptr() + self.flag_off
        a.err = self.err.data_ptr()
        K.a2a_rows(a, self.grid)
        parity = self.round & 1
        self.round += 1
        got = self.counts[parity].tolist()                      # device -> host: also the synchronisation point
        code = int(self.err.item())
        if code:
            self.err.zero_()
            raise RuntimeError(f"row exchange gave up: {K.ERR_NAMES.get(code, code)}")
        out = torch.cat([self.recv[parity, s, : got[s]] for s in range(self.world)], 0) if sum(got) else \
            rows.new_zeros((0, self.row_floats))
        return out, [int(g) for g in got]
