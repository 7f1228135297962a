"""Host-side sharding of the operator set across the GPUs of one node.

Row operators shard by contiguous row ranges, GEMMs by M-blocks with B replicated; no operator has an
exchange step, so the only collectives are the set-up broadcast of B and the max-over-ranks of a
timing.  These helpers are backend-agnostic (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class RowShard:
    """Rows [begin, end) of a [rows, cols] tensor owned by one rank."""

    begin: int
    end: int
    cols: int

    @property
    def rows(self) -> int:
        return self.end - self.begin

    @property
    def elem_offset(self) -> int:
        """Index of the shard's first element in the global tensor (seeds the counter-based fills)."""
        return self.begin * self.cols


def row_shard(total_rows: int, cols: int, rank: int, world: int, multiple_of: int = 1) -> RowShard:
    """Contiguous, balanced split of `total_rows`; shard boundaries fall on multiples of `multiple_of`
    (e.g. 512 so that a causal 512-row block never straddles two GPUs, or the GEMM tile height)."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    if total_rows % multiple_of:
        raise ValueError(f"{total_rows} rows are not a multiple of {multiple_of}")
    units = total_rows // multiple_of
    begin = units * rank // world * multiple_of
    end = units * (rank + 1) // world * multiple_of
    return RowShard(begin, end, cols)


def weak_scaled_rows(rows_per_gpu: int, cols: int, rank: int, world: int) -> RowShard:
    """Weak scaling: every rank owns `rows_per_gpu` rows of a [world * rows_per_gpu, cols] tensor."""
    return row_shard(rows_per_gpu * world, cols, rank, world, multiple_of=rows_per_gpu)


def max_over_ranks(value: float, device=None) -> float:
    """A timing is the maximum over ranks (the slowest GPU decides); identity without a process group."""
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def replicate_from_rank0(tensor):
    """Replicate the GEMM's B operand: one broadcast from rank 0 at set-up, outside any timed region."""
    import torch.distributed as dist

    import torch

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        # 16-bit operands travel as raw integers, which NCCL does not move: broadcast the bytes
        payload = tensor.view(torch.uint8) if tensor.dtype in (torch.int16, torch.uint16) else tensor
        dist.broadcast(payload, src=0)
    return tensor
