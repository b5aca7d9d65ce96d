"""Multi-GPU pieces of the Co-Me hot path (one process per GPU, ``torch.distributed``).

The path shards naturally by frame: selection, merge, frame attention and unmerge of a frame never look at another
frame.  Only global attention has an exchange step: every rank attends ITS packed rows to the keys / values of ALL
ranks, so the merged K/V rows (and nothing else) are all-gathered once per global layer.  The gathered rows land in
this GPU's own memory and are read from there by the attention kernel.

Two transports: NCCL (:func:`gather_rows`) and, for the exchange that is hidden behind attention to the local keys,
driver copies out of peer-mapped windows (:class:`PeerGather`), which leave the attention kernel all but two SMs.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

__all__ = ["shard_range", "rows_per_rank", "gather_rows", "block_order", "hiding_exchange_pays", "pulls_first_pays", "PeerGather", "GlobalExchange"]


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


def hiding_exchange_pays(total_rows: int, world: int, row_bytes: int, num_heads: int, head_dim: int,
                         attn_tflops: float = 780.0, exchange_gbs: float = 380.0, exchange_hidden_gbs: float = 110.0) -> bool:
    """Whether a global layer is shorter with its key / value exchange hidden behind attention to the local keys than with
    the exchange in line, from a two-line model of the layer on one rank:

    * in line:  ``bytes_in / exchange_gbs  +  attention(rows/world queries x all keys)``
    * hidden:   ``max(attention(local queries x local keys), bytes_in / exchange_hidden_gbs)  +  attention(local queries x
      remote keys)``

    The defaults are what B200 nodes measured: the attention kernel sustains ~780 TFLOP/s; an exchange that has the GPU to
    itself moves 360-470 GB/s into every GPU (NCCL or peer copies alike), one that runs beside the attention kernel
    60-120 GB/s.  With 80,672 rows of 4 KB the model gives 8.9 against 8.6 ms per layer on 4 GPUs (measured 8.97 and 8.66):
    hidden pays on 2 to 4 GPUs, where the attention to the local keys outlasts the slowed exchange; in line pays from 5 GPUs
    on (on 8, 0.5 ms of local attention cannot cover a 2.6 ms exchange: 4.9 against 6.2 ms).  The model is pessimistic for
    the peer windows at 8 GPUs, where the hidden form measured 119 ms per scene against 148 in line: callers of that
    transport hide the exchange at every rank count."""
    if world <= 1:
        return False
    local_rows = total_rows / world
    bytes_in = (total_rows - local_rows) * row_bytes
    t_attn = lambda q, k: 4.0 * q * k * head_dim * num_heads / (attn_tflops * 1e12)  # noqa: E731
    in_line = bytes_in / (exchange_gbs * 1e9) + t_attn(local_rows, total_rows)
    hidden = max(t_attn(local_rows, local_rows), bytes_in / (exchange_hidden_gbs * 1e9)) + t_attn(local_rows, total_rows - local_rows)
    return hidden < in_line


def pulls_first_pays(total_rows: int, world: int, row_bytes: int, num_heads: int, head_dim: int,
                     attn_tflops: float = 780.0, exchange_gbs: float = 380.0, stolen: float = 0.3) -> bool:
    """For the peer transport, where :func:`hiding_exchange_pays` says no: whether the layer is still shorter with the pulls
    started BEFORE the attention to the local keys gets the machine (``GlobalExchange(pulls_first=True)``) than with the
    exchange in line.  The driver's copies then take the SMs they want and run at their full speed, and the attention to the
    local keys fills in behind them, delayed by about ``stolen`` of the exchange time (measured on 4 GPUs: a 0.77 ms exchange
    instead of 2.1 ms, the local attention 2.43 instead of 2.20 ms).  Model: ``max(exchange, local attention + stolen x
    exchange) + remote attention`` against ``exchange + attention``; 4.4 against 4.9 ms per layer for the 100-frame scene on
    8 GPUs.  (Measured there: 118.7 ms per scene with the pulls first, 118.9 with the attention first, 148.3 in line.)"""
    if world <= 1:
        return False
    block = total_rows / world
    bytes_in = (total_rows - block) * row_bytes
    t_attn = lambda k: 4.0 * block * k * head_dim * num_heads / (attn_tflops * 1e12)  # noqa: E731
    t_x = bytes_in / (exchange_gbs * 1e9)
    in_line = t_x + t_attn(total_rows)
    first = max(t_x, t_attn(block) + stolen * t_x) + t_attn(total_rows - block) + 0.00005
    return first < in_line


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


class PeerGather:
    """All-gather of row blocks of different heights through peer-mapped windows of one node (one process per GPU).

    Every rank owns a window (two slots of ``max(rows)`` rows + one flag word per rank) that the other ranks map through a
    CUDA IPC handle (``come_peer_alloc`` / ``come_peer_open``).  One exchange: :meth:`stage` copies the local block into
    the own window; :meth:`exchange` tells the peers (``come_peer_signal``), waits until all of them have told us
    (``come_peer_wait``: bounded, raises bit 18 of the device status word instead of hanging), then pulls the peers'
    blocks with ``come_peer_copy`` (plain ``cudaMemcpyAsync`` calls on a few side streams).  Nothing of this library but the
    two one-CTA kernels occupies an SM, so a persistent attention kernel on the same GPU can keep all but two SMs (an NCCL
    all-gather beside it needs its CTAs resident: 16 SMs in this package's set-up).  Measured on B200s: alone an exchange
    moves 360-470 GB/s into every GPU; started while the attention kernel already holds the machine 60-120 GB/s (the
    driver's peer copies behave like kernels that want SMs: NCCL, these copies and a copy kernel of this library on 4 to
    16 SMs were all slowed alike), started together with it again 320-450 GB/s.  So the exchange hides behind a long
    attention to the local keys (:func:`hiding_exchange_pays`) or is started together with a short one
    (:func:`pulls_first_pays`).  Construction is collective over ``group`` (the handles travel through
    ``all_gather_object``).  Two slots suffice: a rank that signals exchange k + 1 has finished its pulls
    of exchange k.
    """

    def __init__(self, rows: Sequence[int], rank: int, row_bytes: int, device: torch.device,
                 group: Optional[dist.ProcessGroup] = None, pull_streams: int = 7, wait_limit_s: float = 20.0,
                 capacity_rows: Optional[int] = None):
        """``capacity_rows``: rows a slot of every window can hold (default: the largest block of ``rows``).  A caller whose
        block heights change from scene to scene sizes the windows once for the largest block it can ever have and calls
        :meth:`set_rows` per scene; all ranks must pass the same value."""
        import ctypes as C

        from . import _lib
        self._lib, self._C = _lib, C
        lib = _lib.lib()
        self.rows = [int(n) for n in rows]
        self.world, self.rank = len(self.rows), int(rank)
        self.row_bytes = int(row_bytes)
        self.device = torch.device(device)
        self.capacity_rows = int(capacity_rows) if capacity_rows is not None else max(self.rows)
        if self.capacity_rows < max(self.rows):
            raise ValueError(f"capacity_rows {self.capacity_rows} is smaller than the largest block {max(self.rows)}")
        self.slot_bytes = -(-self.capacity_rows * self.row_bytes // 256) * 256
        self.flag_offset = 2 * self.slot_bytes
        self.limit_ns = int(wait_limit_s * 1e9)
        self.seq = 0
        self._staged = None
        self._own = None
        self._peer = [None] * self.world
        self.error = None  # why the transport could not be built (on this or another rank)
        # Every rank runs every collective of the set-up whatever happened to it before, so that a failure on one rank
        # cannot leave the others waiting; the ranks agree on the outcome at the end.
        handle_bytes = None
        with torch.cuda.device(self.device):
            try:
                own = C.c_void_p()
                handle = (C.c_char * _lib.COME_PEER_HANDLE_BYTES)()
                _lib.check(lib.come_peer_alloc(self.flag_offset + 256, C.byref(own), handle))
                self._own = own.value
                handle_bytes = bytes(handle.raw)
            except Exception as e:  # noqa: BLE001
                self.error = repr(e)
            handles = [None] * self.world
            dist.all_gather_object(handles, handle_bytes, group=group)
            if self.error is None and any(h is None for h in handles):
                self.error = "another rank could not allocate its window"
            if self.error is None:
                try:
                    for p in range(self.world):
                        if p == self.rank:
                            self._peer[p] = self._own
                            continue
                        ptr = C.c_void_p()
                        _lib.check(lib.come_peer_open(C.create_string_buffer(handles[p], _lib.COME_PEER_HANDLE_BYTES), C.byref(ptr)))
                        self._peer[p] = ptr.value
                except Exception as e:  # noqa: BLE001
                    self.error = repr(e)
            ok = torch.tensor([1 if self.error is None else 0], dtype=torch.int32, device=self.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)  # also: every window is mapped everywhere before the first signal
            if int(ok.item()) != 1 and self.error is None:
                self.error = "another rank could not map the windows"
        self.ok = self.error is None
        if not self.ok:
            self.close()
            return
        self._flag_ptrs = torch.tensor([int(b) + self.flag_offset for b in self._peer], dtype=torch.int64, device=self.device)
        self._streams = [torch.cuda.Stream(device=self.device) for _ in range(max(1, min(int(pull_streams), self.world - 1)))]

    def close(self) -> None:
        """Unmaps the peers' windows and frees the own one.  Collective in effect: call it on every rank, after the last
        exchange has completed everywhere (e.g. behind a barrier)."""
        lib = self._lib.lib()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for p, ptr in enumerate(self._peer):
                if p != self.rank and ptr is not None:
                    lib.come_peer_close(ptr)
            if self._own is not None:
                lib.come_peer_free(self._own)
        self._own, self._peer = None, [None] * self.world

    def set_rows(self, rows: Sequence[int]) -> None:
        """New block heights for the following exchanges (every rank calls it with the same list, between exchanges)."""
        rows = [int(n) for n in rows]
        if len(rows) != self.world or max(rows) > self.capacity_rows:
            raise ValueError(f"need {self.world} block heights of at most {self.capacity_rows} rows, got {rows}")
        self.rows = rows

    def stage(self, local: torch.Tensor) -> None:
        """First half of an exchange, on the current stream: this rank's block goes into the next slot of its window.
        (A same-device copy; issue it where the whole GPU is available, e.g. on the compute stream before the attention
        launch the exchange is meant to hide behind.)"""
        from ._torch_util import stream_ptr
        n_local = self.rows[self.rank]
        if local.shape[0] != n_local or not local.is_contiguous() or local[0].numel() * local.element_size() != self.row_bytes:
            raise ValueError(f"rank {self.rank}: expected a contiguous block of {n_local} rows of {self.row_bytes} bytes")
        self.seq += 1
        slot = (self.seq & 1) * self.slot_bytes
        self._lib.check(self._lib.lib().come_peer_copy(self._own + slot, local.data_ptr(), n_local * self.row_bytes, stream_ptr(self.device)))
        self._staged = local

    def sync(self) -> None:
        """Second step, on the current stream (which must be ordered behind :meth:`stage`): tell the peers that this rank's
        block is in its window and wait (bounded) until all of them have said the same."""
        from ._torch_util import stream_ptr
        lib, check = self._lib.lib(), self._lib.check
        if self._staged is None:
            raise RuntimeError("sync() without a staged block")
        seq = self.seq & 0x3fffffff
        st = stream_ptr(self.device)
        check(lib.come_peer_signal(self._flag_ptrs.data_ptr(), self.world, self.rank, seq, st))
        check(lib.come_peer_wait(self._own + self.flag_offset, self.world, self.rank, seq, self.limit_ns, st))

    def pull(self, out: torch.Tensor, remote_first: bool = False, include_local: bool = True,
             peers: Optional[Sequence[int]] = None) -> torch.Tensor:
        """Third step, on the current stream behind :meth:`sync`, as often as needed: copies the blocks of ``peers`` (default:
        all the other ranks) out of their windows into their places in ``out [sum(rows), ...]`` (block order of
        :func:`block_order`); ``include_local`` also copies this rank's own block into its place."""
        from ._torch_util import stream_ptr
        lib, check = self._lib.lib(), self._lib.check
        local = self._staged
        if local is None:
            raise RuntimeError("pull() without a staged block")
        if not out.is_contiguous() or out.shape[0] != sum(self.rows) or out.dtype != local.dtype or out.shape[1:] != local.shape[1:]:
            raise ValueError("out must be a contiguous [sum(rows), ...] tensor of the blocks' dtype and row shape")
        n_local = self.rows[self.rank]
        slot = (self.seq & 1) * self.slot_bytes
        cur = torch.cuda.current_stream(self.device)
        st = stream_ptr(self.device)
        ready = torch.cuda.Event()
        ready.record(cur)
        order = block_order(self.world, self.rank, remote_first)
        at, starts = 0, {}
        for r in order:
            starts[r] = at
            at += self.rows[r]
        base = out.data_ptr()
        if include_local:
            check(lib.come_peer_copy(base + starts[self.rank] * self.row_bytes, local.data_ptr(), n_local * self.row_bytes, st))
        wanted = [r for r in order if r != self.rank] if peers is None else [int(p) for p in peers]
        if any(p == self.rank or not (0 <= p < self.world) for p in wanted):
            raise ValueError(f"peers must be other ranks of the group, got {wanted}")
        used = []
        for i, p in enumerate(wanted):
            s = self._streams[i % len(self._streams)]
            if i < len(self._streams):
                s.wait_event(ready)
                used.append(s)
            check(lib.come_peer_copy(base + starts[p] * self.row_bytes, self._peer[p] + slot, self.rows[p] * self.row_bytes, s.cuda_stream))
        for s in used:
            done = torch.cuda.Event()
            done.record(s)
            cur.wait_event(done)
        return out

    def exchange(self, out: torch.Tensor, remote_first: bool = False, include_local: bool = True) -> torch.Tensor:
        """:meth:`sync` + :meth:`pull` of every peer's block on the current stream."""
        self.sync()
        return self.pull(out, remote_first=remote_first, include_local=include_local)

    def gather(self, local: torch.Tensor, out: torch.Tensor, remote_first: bool = False) -> torch.Tensor:
        """``local [rows[rank], ...]`` of every rank -> ``out [sum(rows), ...]``: :meth:`stage` + :meth:`exchange` on the
        current stream."""
        self.stage(local)
        return self.exchange(out, remote_first=remote_first)


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
                 gather=None, overlap: bool = False, comm_sms: int = 16, transport: str = "nccl", pulls_first: bool = False,
                 peer_capacity_rows: Optional[int] = None):
        """``transport`` of the hidden exchange: ``"nccl"`` (an all-gather kernel beside the attention kernel) or ``"peer"``
        (:class:`PeerGather`: copy engines, built at the first :meth:`attend`; when a rank cannot set it up, all ranks
        fall back to NCCL together).  The in-line exchange (``overlap=False``) always uses NCCL.

        ``comm_sms``: SMs left free while the attention to the local keys runs beside the exchange.  An NCCL collective
        completes only when all its CTAs have run, so the communicator must not use more CTAs than that
        (``NCCL_MAX_CTAS`` in the environment before the process group is created, or the ``max_ctas`` option of the NCCL
        process group); otherwise its last CTAs wait for the attention kernel to end and nothing overlaps.  The peer
        transport needs two SMs for its two small kernels.

        ``pulls_first`` (peer transport): the attention to the local keys is launched only once the peers have signalled, so
        that the pulls and the attention become runnable together: the driver's copies then take the SMs they want and run
        at the speed of an exchange that has the GPU to itself, and the attention fills in behind them.  For many ranks,
        where the attention to the local keys is too short to cover a slowed exchange (:func:`pulls_first_pays`)."""
        if transport not in ("nccl", "peer"):
            raise ValueError(f"transport must be 'nccl' or 'peer', got {transport!r}")
        self.pulls_first = bool(pulls_first)
        self.peer_capacity_rows = peer_capacity_rows  # rows a window slot is sized for (default: the largest block now)
        self.transport = transport
        self._peer_gather = None
        self.peer_error = None
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

    def adopt(self, previous: "GlobalExchange") -> None:
        """Takes over the side stream, the gather buffer and the peer windows of the exchange object of the previous scene
        (same ranks).  Windows that are too small for the new block heights are released and rebuilt at the next
        :meth:`attend`; every rank adopts at the same point of its program."""
        if previous is None or len(previous.rows) != len(self.rows):
            return
        self._side, self.events = previous._side, previous.events
        if previous._side is not None:
            self._cu_local = torch.tensor([0, self.rows[self.rank]], dtype=torch.int32, device=self.weight_all.device)
        if previous._buf is not None and previous._buf.shape[0] == self.total:
            self._buf = previous._buf
        pg = previous._peer_gather
        previous._peer_gather = None
        if pg is None:
            if previous.peer_error is not None:  # the transport could not be built before: do not try again every scene
                self.transport, self.peer_error = previous.transport, previous.peer_error
            return
        if pg.capacity_rows >= max(self.rows):
            pg.set_rows(self.rows)
            self._peer_gather = pg
        else:
            torch.cuda.synchronize(pg.device)
            dist.barrier(group=self.group)  # nobody still pulls out of a window that is about to go
            pg.close()

    def close(self) -> None:
        """Releases the peer windows, if any (call on every rank once the last exchange has completed everywhere)."""
        if self._peer_gather is not None:
            self._peer_gather.close()
            self._peer_gather = None

    def _setup_peer(self, kv: torch.Tensor) -> None:
        """Builds the copy-engine transport (collective; the ranks agree on the outcome inside).  If any rank failed, the
        exchange stays on NCCL on all of them and ``peer_error`` says why."""
        pg = PeerGather(self.rows, self.rank, kv[0].numel() * kv.element_size(), kv.device, self.group,
                        capacity_rows=self.peer_capacity_rows)
        if pg.ok:
            self._peer_gather = pg
        else:
            self.transport = "nccl"
            self.peer_error = pg.error

    def attend(self, q: torch.Tensor, kv: torch.Tensor, scale: float, use_bias: bool = True) -> torch.Tensor:
        """Global attention of this rank's query rows ``q [rows, H, D]`` to the keys / values of ALL ranks, of which this
        rank holds ``kv [rows, 2, H, D]`` (key rows ``kv[:, 0]``, value rows ``kv[:, 1]``).  Returns ``[rows, H, D]``."""
        from .flash_attn_fwd_cuda import combine, cross_fwd_balanced, cta_limit, varlen_fwd_rows
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
        if self.transport == "peer" and self._gather is None and self._peer_gather is None:
            self._setup_peer(kv)
        if self._peer_gather is not None:
            self._peer_gather.stage(kv)  # into this rank's window while the whole GPU is available (tens of microseconds)
        side.wait_stream(main)  # kv is ready, and the previous layer has finished reading the buffer
        ev = [torch.cuda.Event(enable_timing=self.events is not None) for _ in range(4)]
        with torch.cuda.stream(side):
            ev[0].record(side)
            synced = None
            if self._peer_gather is not None:
                self._peer_gather.sync()
                synced = torch.cuda.Event()
                synced.record(side)
                gathered = self._peer_gather.pull(self._buf, remote_first=True, include_local=False)
            else:
                gathered = self.gather(kv, remote_first=True, out=self._buf)
            ev[1].record(side)
        kv.record_stream(side)
        if synced is not None and self.pulls_first:
            main.wait_event(synced)  # the pulls and the attention launch become runnable together
        bias_local, bias_remote = self.bias_local_remote(dtype) if use_bias else (None, None)
        sms = torch.cuda.get_device_properties(q.device).multi_processor_count
        free = 2 if self._peer_gather is not None else self.comm_sms
        with cta_limit(sms - free if 0 < free < sms else 0):  # the exchange's kernels keep their SMs
            out, lse = cross_fwd_balanced(q, kv[:, 0], kv[:, 1], bias_local, scale)  # the local rows are the only keys here
        ev[2].record(main)
        main.wait_event(ev[1])
        if self._peer_gather is None and gathered.data_ptr() != self._buf.data_ptr():  # a stand-in gather allocated its own result on the side stream
            gathered.record_stream(main)
        remote = gathered[:n_remote]
        out_r, lse_r = cross_fwd_balanced(q, remote[:, 0], remote[:, 1], bias_remote, scale)
        combine(out, lse, out_r, lse_r, out_=out, lse_out=lse)
        ev[3].record(main)
        if self.events is not None:
            self.events.append(ev)
        return out
