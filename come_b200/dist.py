"""Multi-GPU pieces of the Co-Me hot path (one process per GPU, ``torch.distributed``).

The path shards naturally by frame: selection, merge, frame attention and unmerge of a frame never look at another
frame.  Only global attention has an exchange step: every rank attends ITS packed rows to the keys / values of ALL
ranks, so the merged K/V rows (and nothing else) are all-gathered once per global layer.  The gathered rows land in
this GPU's own memory and are read from there by the attention kernel.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

__all__ = ["shard_range", "rows_per_rank", "gather_rows", "GlobalExchange"]


def shard_range(n_items: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced share ``[lo, hi)`` of ``n_items`` for ``rank`` (the first ``n_items % world`` ranks get
    one extra item).  Contiguity keeps every rank's packed rows one slice of the global packed sequence."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world size {world}")
    base, extra = divmod(n_items, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def rows_per_rank(frame_offsets: Sequence[int], world: int) -> List[int]:
    """Packed rows owned by every rank when frames are sharded with :func:`shard_range`; ``frame_offsets`` are the
    ``frames + 1`` packed offsets of the whole scene."""
    frames = len(frame_offsets) - 1
    out = []
    for r in range(world):
        lo, hi = shard_range(frames, world, r)
        out.append(int(frame_offsets[hi]) - int(frame_offsets[lo]))
    return out


def gather_rows(local: torch.Tensor, rows: Sequence[int], group: Optional[dist.ProcessGroup] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather row blocks of different heights: rank ``r`` contributes ``local`` with ``rows[r]`` rows; the result
    holds all blocks back to back, ``[sum(rows), ...]``, on every rank.

    Tries the backend's own uneven all-gather into views of the result; backends without one (gloo) go through a
    padded equal-size all-gather and a compaction copy.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if len(rows) != world or local.shape[0] != rows[rank]:
        raise ValueError(f"rank {rank} holds {local.shape[0]} rows but rows = {list(rows)}")
    total = int(sum(rows))
    if out is None:
        out = torch.empty((total,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    if world == 1:
        out.copy_(local)
        return out
    starts = [0]
    for n in rows:
        starts.append(starts[-1] + int(n))
    views = [out[starts[r]:starts[r + 1]] for r in range(world)]
    local = local.contiguous()
    if all(n == rows[0] for n in rows):
        dist.all_gather_into_tensor(out, local, group=group)
        return out
    try:
        dist.all_gather(views, local, group=group)
        return out
    except (RuntimeError, ValueError, NotImplementedError):
        pass
    most = int(max(rows))
    padded = torch.zeros((most,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[: rows[rank]] = local
    stage = torch.empty((world * most,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(stage, padded, group=group)
    for r in range(world):
        views[r].copy_(stage[r * most: r * most + rows[r]])
    return out


class GlobalExchange:
    """What a rank needs to run global attention on ITS packed rows of a scene whose frames are spread over the ranks:
    the row counts of all ranks, where its own rows start, the per-key bias of all rows (the plan of the whole scene is
    replicated, so this needs no communication) and the gather of the key / value rows.

    ``gather`` defaults to :func:`gather_rows` over ``group``; tests pass their own to stand in for the other ranks.
    """

    def __init__(self, rows: Sequence[int], rank: int, weight_all: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                 gather=None):
        self.rows = [int(n) for n in rows]
        self.rank = int(rank)
        self.total = int(sum(self.rows))
        self.row_begin = int(sum(self.rows[: self.rank]))
        if weight_all.shape != (self.total,):
            raise ValueError(f"weight_all must hold {self.total} counts, got {tuple(weight_all.shape)}")
        self.weight_all = weight_all
        self.cu_seqlens = torch.tensor([0, self.total], dtype=torch.int32, device=weight_all.device)
        self.group = group
        self._gather = gather
        self._bias = {}

    def bias(self, dtype: torch.dtype) -> torch.Tensor:
        """``log(count)`` of every packed row of the scene in the attention dtype."""
        if dtype not in self._bias:
            self._bias[dtype] = self.weight_all.log().to(dtype)
        return self._bias[dtype]

    def gather(self, local: torch.Tensor) -> torch.Tensor:
        """``[rows[rank], ...]`` of this rank -> ``[total, ...]`` of all ranks, in this GPU's memory."""
        if local.shape[0] != self.rows[self.rank]:
            raise ValueError(f"rank {self.rank} holds {local.shape[0]} rows, expected {self.rows[self.rank]}")
        if self._gather is not None:
            return self._gather(local, self.rows, self.rank)
        if len(self.rows) == 1:
            return local
        return gather_rows(local, self.rows, self.group)
