"""Reference collectives over ``torch.distributed`` (gloo on CPU, NCCL on GPU).

This is the baseline/fallback communication path and the oracle for the fused kernels: a sum all-reduce inside
the tensor-parallel group after o_proj and after the MoE block (the reference's AR1/AR2,
kernels/decode_step_tp8.cu:1093-1135), a (max, arg) exchange for the vocabulary-sharded head
(kernels/decode_step_tp8.cu:1181-1183), and an expert-parallel dispatch/combine built on
``all_to_all_single`` (the reference only has the put-based all-to-all microbenchmark,
kernels/nvshmem_comms.cu:170-191, and combines EP outputs with an all-reduce,
kernels/ep_moe_sharded.cu:309-337).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..config import ParallelConfig


class Collectives:
    """Process-group bundle for one rank. With ``world == 1`` every call is the identity."""

    def __init__(self, par: ParallelConfig):
        self.par = par
        self.world_group = None
        self.tp_group = None
        self.kv_group = None
        self.n_collectives = 0
        if par.world > 1:
            if not dist.is_initialized():
                raise RuntimeError("torch.distributed must be initialised before building Collectives")
            self.world_group = dist.group.WORLD
            if par.tp == par.world:
                self.tp_group = self.world_group
            elif par.tp > 1:
                # every rank must create every subgroup, in the same order
                for g0 in range(0, par.world, par.tp):
                    ranks = list(range(g0, g0 + par.tp))
                    grp = dist.new_group(ranks)
                    if par.rank in ranks:
                        self.tp_group = grp
            if par.kv_share > 1:
                # consecutive ranks of a tensor-parallel group hold the same KV head: one subgroup per head
                for g0 in range(0, par.world, par.kv_share):
                    ranks = list(range(g0, g0 + par.kv_share))
                    grp = dist.new_group(ranks)
                    if par.rank in ranks:
                        self.kv_group = grp

    # tensor parallel -------------------------------------------------------------------------------------
    def all_reduce_tp(self, x: torch.Tensor) -> torch.Tensor:
        if self.par.tp > 1:
            self.n_collectives += 1
            dist.all_reduce(x, op=dist.ReduceOp.SUM, group=self.tp_group)
        return x

    def all_gather_kv(self, x: torch.Tensor) -> List[torch.Tensor]:
        """``x`` of every rank that shares this rank's KV head, in rank order (``kv_share`` tensors)."""
        if self.par.kv_share <= 1 or self.par.world == 1:
            return [x]
        self.n_collectives += 1
        out = [torch.empty_like(x) for _ in range(self.par.kv_share)]
        dist.all_gather(out, x.contiguous(), group=self.kv_group)
        return out

    def all_reduce_world(self, x: torch.Tensor) -> torch.Tensor:
        if self.par.world > 1:
            self.n_collectives += 1
            dist.all_reduce(x, op=dist.ReduceOp.SUM, group=self.world_group)
        return x

    def all_gather_world(self, x: torch.Tensor) -> List[torch.Tensor]:
        if self.par.world == 1:
            return [x]
        self.n_collectives += 1
        out = [torch.empty_like(x) for _ in range(self.par.world)]
        dist.all_gather(out, x.contiguous(), group=self.world_group)
        return out

    def gather_logits(self, local_logits: torch.Tensor, vocab: int, chunk: int) -> torch.Tensor:
        """Vocabulary-sharded head: assemble ``[T, vocab]`` from per-rank ``[T, chunk]`` (zero padded) shards."""
        if self.par.world == 1:
            return local_logits[..., :vocab]
        T = local_logits.shape[0]
        pad = torch.zeros(T, chunk, dtype=local_logits.dtype, device=local_logits.device)
        pad[:, : local_logits.shape[1]] = local_logits
        parts = self.all_gather_world(pad)
        return torch.cat(parts, dim=1)[:, :vocab]

    def argmax_sharded(self, local_logits: torch.Tensor, vocab0: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Global (max value, arg) per row from vocabulary shards; ties resolve to the lowest token id."""
        if local_logits.shape[1] > 0:
            v, i = local_logits.max(dim=1)
            i = i + vocab0
        else:
            v = torch.full((local_logits.shape[0],), float("-inf"), dtype=local_logits.dtype, device=local_logits.device)
            i = torch.zeros(local_logits.shape[0], dtype=torch.long, device=local_logits.device)
        if self.par.world == 1:
            return v, i
        packed = torch.stack([v.float(), i.float()], dim=1)
        parts = torch.stack(self.all_gather_world(packed))          # [world, T, 2]
        vals, ids = parts[..., 0], parts[..., 1]
        best = vals.max(dim=0).values
        cand = torch.where(vals == best[None], ids, torch.full_like(ids, float("inf")))
        return best, cand.min(dim=0).values.long()

    # expert parallel ---------------------------------------------------------------------------------------
    def all_to_all_rows(self, rows: torch.Tensor, send_counts: List[int], allow_fast: bool = True) -> Tuple[torch.Tensor, List[int]]:
        """Variable-size row exchange: ``rows`` is ordered by destination rank with ``send_counts[d]`` rows for
        rank ``d``. Returns the received rows ordered by source rank and the per-source counts. ``allow_fast`` must be
        the same on every rank (it selects the peer-memory kernel when one is installed)."""
        world = self.par.world
        if world == 1:
            return rows, list(send_counts)
        fast = getattr(self, "fast_a2a", None)
        if fast is not None and allow_fast and rows.is_cuda and rows.dtype == torch.float32 and rows.dim() == 2 \
                and rows.shape[1] <= fast.row_floats:
            # one kernel over peer memory (parallel/a2a.py); narrower rows are padded to the region's row width. The
            # choice depends only on properties that are the same on every rank (a count above the capacity raises).
            self.n_collectives += 1
            width = rows.shape[1]
            if width < fast.row_floats:
                rows = torch.nn.functional.pad(rows, (0, fast.row_floats - width))
            out, counts = fast.exchange(rows, send_counts)
            return (out[:, :width].contiguous() if width < fast.row_floats else out), counts
        self.n_collectives += 2
        sc = torch.tensor(send_counts, dtype=torch.int64, device=rows.device)
        rc = torch.empty(world, dtype=torch.int64, device=rows.device)
        dist.all_to_all_single(rc, sc, group=self.world_group)
        recv_counts = [int(v) for v in rc.tolist()]
        out = torch.empty((sum(recv_counts),) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
        dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_counts,
                               input_split_sizes=list(send_counts), group=self.world_group)
        return out, recv_counts

    def barrier(self) -> None:
        if self.par.world > 1:
            dist.barrier(group=self.world_group)
