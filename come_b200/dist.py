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

__all__ = ["shard_range", "rows_per_rank", "gather_rows", "block_order", "GlobalExchange"]


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
                out: Optional[torch.Tensor] = None, remote_first: bool = False) -> torch.Tensor:
    """All-gather row blocks of different heights: rank ``r`` contributes ``local`` with ``rows[r]`` rows; the result
    holds all blocks back to back, ``[sum(rows), ...]``, on every rank.

    ``remote_first``: the blocks are laid out in the order ``rank + 1, ..., world - 1, 0, ..., rank - 1, rank`` instead of
    ``0 .. world - 1``: the rows of the OTHER ranks form one contiguous range at the front (attention does not care about
    the order of its keys, so they can be attended as one segment while the local block is handled separately).

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
    elif out.shape[0] != total:
        raise ValueError(f"out holds {out.shape[0]} rows, the blocks add up to {total}")
    order = block_order(world, rank, remote_first)
    starts = {}
    at = 0
    for r in order:
        starts[r] = at
        at += int(rows[r])
    views = [out[starts[r]:starts[r] + int(rows[r])] for r in range(world)]
    if world == 1:
        out.copy_(local)
        return out
    local = local.contiguous()
    if not remote_first and all(n == rows[0] for n in rows):
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


def block_order(world: int, rank: int, remote_first: bool) -> List[int]:
    """Order of the ranks' blocks in a gathered buffer (see :func:`gather_rows`)."""
    if not remote_first:
        return list(range(world))
    return [(rank + 1 + i) % world for i in range(world)]


class GlobalExchange:
    """What a rank needs to run global attention on ITS packed rows of a scene whose frames are spread over the ranks:
    the row counts of all ranks, where its own rows start, the per-key bias of all rows (the plan of the whole scene is
    replicated, so this needs no communication) and the gather of the key / value rows.

    ``gather`` defaults to :func:`gather_rows` over ``group``; tests pass their own to stand in for the other ranks.

    ``overlap``: hide the exchange behind compute.  The all-gather of the key / value rows is issued on a side stream;
    meanwhile the local query rows attend to the LOCAL keys / values; when the gather has landed they attend to the other
    ranks' rows (one contiguous range of the gathered buffer, see :func:`gather_rows`), and the two partial results are
    merged from their log-sum-exps.  The merged result equals the one-launch result up to the rounding of the two partial
    outputs to the attention dtype; without ``overlap`` the sharded result is bit-identical to the single-GPU one.
    """

    def __init__(self, rows: Sequence[int], rank: int, weight_all: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                 gather=None, overlap: bool = False, comm_sms: int = 16):
        """``comm_sms``: SMs left to the all-gather kernel while the attention to the local keys runs beside it.  The
        collective completes only when all its CTAs have run, so the communicator must not use more CTAs than that
        (``NCCL_MAX_CTAS`` in the environment before the process group is created, or the ``max_ctas`` option of the NCCL
        process group); otherwise its last CTAs wait for the attention kernel to end and nothing overlaps."""
        self.comm_sms = int(comm_sms)
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
        self.overlap = bool(overlap) and len(self.rows) > 1
        self._bias = {}
        self._bias_split = {}
        self._side = None
        self._buf = None
        self.events = None  # set to a list to collect (gather start, gather end, local end, remote end) CUDA events

    def bias(self, dtype: torch.dtype) -> torch.Tensor:
        """``log(count)`` of every packed row of the scene in the attention dtype."""
        if dtype not in self._bias:
            self._bias[dtype] = self.weight_all.log().to(dtype)
        return self._bias[dtype]

    def bias_local_remote(self, dtype: torch.dtype):
        """``(bias of this rank's rows, bias of the other ranks' rows in the remote-first order of the gathered buffer)``."""
        if dtype not in self._bias_split:
            b = self.bias(dtype)
            lo, n = self.row_begin, self.rows[self.rank]
            starts = [sum(self.rows[:r]) for r in range(len(self.rows))]
            order = block_order(len(self.rows), self.rank, True)[:-1]
            remote = torch.cat([b[starts[r]:starts[r] + self.rows[r]] for r in order]) if order else b[:0]
            self._bias_split[dtype] = (b[lo:lo + n].contiguous(), remote.contiguous())
        return self._bias_split[dtype]

    def gather(self, local: torch.Tensor, remote_first: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``[rows[rank], ...]`` of this rank -> ``[total, ...]`` of all ranks, in this GPU's memory."""
        if local.shape[0] != self.rows[self.rank]:
            raise ValueError(f"rank {self.rank} holds {local.shape[0]} rows, expected {self.rows[self.rank]}")
        if self._gather is not None:
            full = self._gather(local, self.rows, self.rank)  # rank order
            if not remote_first:
                return full
            starts = [sum(self.rows[:r]) for r in range(len(self.rows))]
            return torch.cat([full[starts[r]:starts[r] + self.rows[r]] for r in block_order(len(self.rows), self.rank, True)])
        if len(self.rows) == 1:
            return local
        return gather_rows(local, self.rows, self.group, out=out, remote_first=remote_first)

    def attend(self, q: torch.Tensor, kv: torch.Tensor, scale: float, use_bias: bool = True) -> torch.Tensor:
        """Global attention of this rank's query rows ``q [rows, H, D]`` to the keys / values of ALL ranks, of which this
        rank holds ``kv [rows, 2, H, D]`` (key rows ``kv[:, 0]``, value rows ``kv[:, 1]``).  Returns ``[rows, H, D]``."""
        from .flash_attn_fwd_cuda import combine, cross_fwd, cta_limit, varlen_fwd_rows
        dtype = q.dtype
        kv = kv.contiguous()
        if not self.overlap:
            kv_all = self.gather(kv)
            out, _ = varlen_fwd_rows(q, kv_all[:, 0], kv_all[:, 1], self.cu_seqlens, self.total,
                                     self.bias(dtype) if use_bias else None, scale, self.row_begin)
            return out
        n_local = self.rows[self.rank]
        n_remote = self.total - n_local
        main = torch.cuda.current_stream(q.device)
        if self._side is None:
            self._side = torch.cuda.Stream(device=q.device)
            self._cu_local = torch.tensor([0, n_local], dtype=torch.int32, device=q.device)
        shape = (self.total,) + tuple(kv.shape[1:])
        if self._buf is None or tuple(self._buf.shape) != shape or self._buf.dtype != kv.dtype:
            self._buf = torch.empty(shape, dtype=kv.dtype, device=kv.device)  # reused by every global layer
        side = self._side
        side.wait_stream(main)  # kv is ready, and the previous layer has finished reading the buffer
        ev = [torch.cuda.Event(enable_timing=self.events is not None) for _ in range(4)]
        with torch.cuda.stream(side):
            ev[0].record(side)
            gathered = self.gather(kv, remote_first=True, out=self._buf)
            ev[1].record(side)
        kv.record_stream(side)
        bias_local, bias_remote = self.bias_local_remote(dtype) if use_bias else (None, None)
        sms = torch.cuda.get_device_properties(q.device).multi_processor_count
        with cta_limit(sms - self.comm_sms if 0 < self.comm_sms < sms else 0):  # the gather's CTAs keep their SMs
            out, lse = varlen_fwd_rows(q, kv[:, 0], kv[:, 1], self._cu_local, n_local, bias_local, scale, 0)
        ev[2].record(main)
        main.wait_event(ev[1])
        if gathered.data_ptr() != self._buf.data_ptr():  # a stand-in gather allocated its own result on the side stream
            gathered.record_stream(main)
        remote = gathered[:n_remote]
        out_r, lse_r = cross_fwd(q, remote[:, 0], remote[:, 1], bias_remote, scale)
        combine(out, lse, out_r, lse_r, out_=out, lse_out=lse)
        ev[3].record(main)
        if self.events is not None:
            self.events.append(ev)
        return out
