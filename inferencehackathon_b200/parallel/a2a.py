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

    def exchange_device(self, rows: torch.Tensor, offsets: torch.Tensor, gather: Optional[torch.Tensor] = None):
        """The exchange with nothing on the host: ``offsets [world + 1]`` int32 ON THE DEVICE (rows
        ``offsets[d] .. offsets[d + 1]`` go to rank ``d``; at most ``cap`` per rank, which the caller guarantees).
        Returns ``(recv [world, cap, row_floats], counts [world] int32)``: views of the receive region of this round,
        valid until the round after the next one; rows ``[0, counts[s])`` of ``recv[s]`` came from rank ``s``. No
        synchronisation, no upload: a wait that gave up shows in :meth:`check`."""
        if rows.dtype != torch.float32 or rows.shape[-1] != self.row_floats or not rows.is_contiguous():
            raise ValueError("rows must be contiguous fp32 [P, row_floats]")
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
        return self.recv[parity], self.counts[parity]

    def check(self) -> None:
        """Raises if a wait of an earlier exchange gave up (one device -> host read)."""
        code = int(self.err.item())
        if code:
            self.err.zero_()
            raise RuntimeError(f"row exchange gave up: {K.ERR_NAMES.get(code, code)}")

    def exchange(self, rows: torch.Tensor, send_counts, gather: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, List[int]]:
        """``rows [P, row_floats]`` fp32 ordered by destination (or any matrix plus ``gather [P]`` int32 giving the
        source row of each pair in destination order); ``send_counts[d]`` rows go to rank ``d``. Returns the received
        rows ordered by source rank and the per-source counts as Python ints (the interface of
        ``Collectives.all_to_all_rows``, whose callers split on the host): ONE device -> host read, which carries the
        counts and the error word together."""
        sc = torch.as_tensor(send_counts, dtype=torch.int32)
        if int(sc.max()) > self.cap:
            raise ValueError(f"{int(sc.max())} rows for one rank exceed the slot capacity {self.cap}")
        offsets = torch.zeros(self.world + 1, dtype=torch.int32)
        offsets[1:] = torch.cumsum(sc, 0)
        offsets = offsets.to(self.device, non_blocking=True)
        recv, counts = self.exchange_device(rows.contiguous(), offsets, gather)
        both = torch.cat([counts, self.err]).tolist()            # device -> host: also the synchronisation point
        got, code = both[:-1], both[-1]
        if code:
            self.err.zero_()
            raise RuntimeError(f"row exchange gave up: {K.ERR_NAMES.get(code, code)}")
        out = torch.cat([recv[s, : got[s]] for s in range(self.world)], 0) if sum(got) else \
            rows.new_zeros((0, self.row_floats))
        return out, [int(g) for g in got]


def main(argv=None) -> int:
    """Latency of one exchange, device-timed, max over ranks, against NCCL ``all_to_all_single`` of the same rows
    (run under ``torch.distributed.run``): ``python -m inferencehackathon_b200.parallel.a2a [ROWS_PER_PEER] [ROW_FLOATS]``.
    The reference's figures for this role: 17 us put + barrier over NVSHMEM, ~125 us NCCL all-to-all at 8-16 KB
    (docs/kernel-design/benched-results.md:32-33, docs/onbox-collective-latency-e0.md:10)."""
    import json
    import sys
    from .launch import init_distributed
    argv = sys.argv[1:] if argv is None else argv
    per = int(argv[0]) if len(argv) > 0 else 8
    rf = int(argv[1]) if len(argv) > 1 else 4096
    rank, world, local = init_distributed()
    dev = torch.device("cuda", local)
    K.load()
    ex = PeerRowExchange(dev, rf, max(per, 1))
    rows = torch.randn(world * per, rf, device=dev)
    offsets = (torch.arange(world + 1, dtype=torch.int32) * per).to(dev)
    recv_nccl = torch.empty_like(rows)

    def timed(fn, iters=50):
        for _ in range(5):
            fn()
        torch.cuda.synchronize(dev)
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    recv, counts = ex.exchange_device(rows, offsets)
    dist.all_to_all_single(recv_nccl, rows)
    torch.cuda.synchronize(dev)
    same = bool(torch.equal(recv[:, :per].reshape(world * per, rf), recv_nccl)) and counts.tolist() == [per] * world
    t_own = timed(lambda: ex.exchange_device(rows, offsets))
    ex.check()
    t_nccl = timed(lambda: dist.all_to_all_single(recv_nccl, rows))
    if rank == 0:
        print("A2A " + json.dumps({"n_gpus": world, "rows_per_peer": per, "row_bytes": rf * 4, "peer_kernel_us": round(t_own, 2),
                                   "nccl_all_to_all_us": round(t_nccl, 2), "matches_nccl": same}))
    dist.barrier()
    dist.destroy_process_group()
    return 0 if same else 1


if __name__ == "__main__":
    import sys
    sys.exit(main())
