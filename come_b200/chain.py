"""The standalone Co-Me operator chain: confidence -> window selection -> merge -> biased variable-length
attention -> unmerge, as one callable over device tensors.

This is the call sequence the reference's accelerated VGGT runs around every attention layer
(``src/accelerate/vggt/direct.py:71-124``: merge, attention with ``log(count)`` key bias on frame segments or on
one global segment per scene, split), with the index plan built once per scene instead of once per layer.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from . import _lib
from .flash_attn import flash_attn_varlen_qkvpacked_func_w_perkey_bias
from .token_merger import MergePlan, select_windows

__all__ = ["CoMeOpChain", "ShardedOpChain"]


class CoMeOpChain:
    """Merge / attention / unmerge layers of one scene of ``frames`` frames on a ``grid_h x grid_w`` patch grid.

    ``layer_kinds`` lists the attention layers of a forward pass, ``"frame"`` (one segment per frame) or
    ``"global"`` (all frames of the scene in one segment).
    """

    def __init__(self, frames: int, start_index: int = 5, grid_h: int = 37, grid_w: int = 37, group_h: int = 3,
                 group_w: int = 3, threshold: float = 0.5, num_heads: int = 16, head_dim: int = 64,
                 layer_kinds: Optional[Sequence[str]] = None, scope: str = "frame"):
        self.frames = frames
        self.layout = _lib.Layout.two_d(start_index, grid_h, grid_w, group_h, group_w)
        self.grid = (grid_h, grid_w, group_h, group_w)
        self.threshold = threshold
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.scale = head_dim ** -0.5
        self.layer_kinds: List[str] = list(layer_kinds) if layer_kinds is not None else ["frame", "global"] * 24
        self.scope = scope
        self.launches_per_scene = 3 + 3 * len(self.layer_kinds)  # select + 2 plan kernels + 3 per layer

    def build_plan(self, confidence: torch.Tensor) -> MergePlan:
        """Per-patch confidence ``[1, frames * H * W]`` -> merge plan (one host read for the packed length)."""
        H, W, gh, gw = self.grid
        mask = select_windows(confidence, 1, self.frames, H, W, gh, gw, self.threshold, "pairwise-rank", self.scope)
        return MergePlan(mask, self.layout)

    def layer(self, plan: MergePlan, x: torch.Tensor, qkv: torch.Tensor, kind: str) -> torch.Tensor:
        """One attention layer: merge ``x [frames, N, C]``, attend with ``qkv [P, 3, heads, head_dim]`` standing
        in for the projection of the merged tokens, unmerge the attention output to ``[frames, N, C]``."""
        merged = plan.merge(x)
        if kind == "global":
            cu, max_len = plan.cu_seqlens(self.frames), plan.total
        else:
            cu, max_len = plan.cu_seqlens(1), plan.max_seqlen
        attn = flash_attn_varlen_qkvpacked_func_w_perkey_bias(qkv, cu, max_len, perkey_bias=plan.perkey_bias(qkv.dtype),
                                                               softmax_scale=self.scale)
        y = attn.reshape(plan.total, self.num_heads * self.head_dim)
        # the merged tokens feed the projection in a model; here they only have to stay alive until attention ran
        del merged
        return plan.split(y).reshape(self.frames, plan.tokens_per_frame, -1)

    def forward_scene(self, x: torch.Tensor, confidence: torch.Tensor, qkv_for_total) -> torch.Tensor:
        """Run every layer of a scene.  ``qkv_for_total(P)`` returns the packed qkv tensor for ``P`` merged
        tokens (the benchmark slices a pre-drawn random buffer)."""
        plan = self.build_plan(confidence)
        qkv = qkv_for_total(plan.total)
        out = x
        for kind in self.layer_kinds:
            out = self.layer(plan, x, qkv, kind)
        return out


class ShardedOpChain:
    """The operator chain of ONE scene sharded over the ranks of a process group by frame.

    Every rank owns a contiguous range of frames: its selection, merge, frame attention and unmerge are local.  A
    global layer all-gathers the merged key / value rows (``[P_local, 2, heads, head_dim]`` per rank, nothing else)
    and attends the local query rows to all of them with the row-range attention kernel.  The confidence of all
    frames is replicated (a few hundred KB), so every rank derives the same global packed offsets without a collective.
    """

    def __init__(self, frames_total: int, group=None, start_index: int = 5, grid_h: int = 37, grid_w: int = 37,
                 group_h: int = 3, group_w: int = 3, threshold: float = 0.5, num_heads: int = 16, head_dim: int = 64,
                 layer_kinds: Optional[Sequence[str]] = None, overlap: bool = False, world: Optional[int] = None,
                 rank: Optional[int] = None, transport: str = "nccl", pulls_first: bool = False):
        """``overlap``: hide the key / value exchange of a global layer behind attention to the local keys
        (:class:`come_b200.dist.GlobalExchange`); the result then differs from the single-GPU one by the rounding of two
        partial outputs.  Off: bit-identical to the single-GPU chain.  ``transport`` of the hidden exchange: ``"nccl"`` or
        ``"peer"`` (pulls out of peer-mapped windows, :class:`come_b200.dist.PeerGather`; ``pulls_first``: the pulls start
        before the attention to the local keys gets the machine, see :class:`come_b200.dist.GlobalExchange`).  ``world`` / ``rank`` default
        to the process group's; ``world=1`` runs the whole scene on this GPU whatever the group is."""
        import torch.distributed as dist

        from .dist import shard_range
        self.group = group
        self.world = int(world) if world is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.rank = int(rank) if rank is not None else (dist.get_rank(group) if dist.is_initialized() and self.world > 1 else 0)
        self.frames_total = frames_total
        self.f_lo, self.f_hi = shard_range(frames_total, self.world, self.rank)
        self.layout = _lib.Layout.two_d(start_index, grid_h, grid_w, group_h, group_w)
        self.grid = (grid_h, grid_w, group_h, group_w)
        self.threshold = threshold
        self.num_heads, self.head_dim = num_heads, head_dim
        self.scale = head_dim ** -0.5
        self.layer_kinds = list(layer_kinds) if layer_kinds is not None else ["frame", "global"] * 24
        self.overlap = bool(overlap)
        self.transport = transport
        self.pulls_first = bool(pulls_first)
        self.exchange = None

    def build_plans(self, confidence_all: torch.Tensor):
        """``confidence_all [1, frames_total * H * W]`` (replicated) -> ``(global_plan, local_plan)``."""
        from .dist import rows_per_rank, shard_range
        H, W, gh, gw = self.grid
        mask_all = select_windows(confidence_all, 1, self.frames_total, H, W, gh, gw, self.threshold, "pairwise-rank", "frame")
        global_plan = MergePlan(mask_all, self.layout)
        local_plan = MergePlan(mask_all[self.f_lo:self.f_hi].contiguous(), self.layout)
        offsets = global_plan.offset.tolist()
        self.rows = rows_per_rank(offsets, self.world)
        self.row_begin = int(offsets[self.f_lo])
        assert self.rows[self.rank] == local_plan.total
        self.cu_global = torch.tensor([0, global_plan.total], dtype=torch.int32, device=mask_all.device)
        from .dist import GlobalExchange
        keep = self.exchange
        # peer windows sized once for the largest block a rank can ever hold: all its frames unmerged
        most_frames = max(shard_range(self.frames_total, self.world, r)[1] - shard_range(self.frames_total, self.world, r)[0]
                          for r in range(self.world))
        self.exchange = GlobalExchange(self.rows, self.rank, global_plan.weight, self.group, overlap=self.overlap,
                                       transport=self.transport, pulls_first=self.pulls_first,
                                       peer_capacity_rows=most_frames * local_plan.tokens_per_frame)
        self.exchange.adopt(keep)  # keep the side stream, the gather buffer and the windows across scenes
        return global_plan, local_plan

    def layer(self, global_plan: MergePlan, local_plan: MergePlan, x_local: torch.Tensor, q_local: torch.Tensor,
              kv_local: torch.Tensor, kind: str, timers: Optional[list] = None) -> torch.Tensor:
        """``x_local [frames_local, N, C]``; ``q_local [P_local, heads, head_dim]`` and ``kv_local [P_local, 2, heads,
        head_dim]`` stand in for the projections of the merged local tokens.  ``timers``: a list that receives
        ``(kind, [4 CUDA events])`` bracketing merge, attention and unmerge on the current stream."""
        from .flash_attn_fwd_cuda import varlen_fwd_rows
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if timers is not None else None
        if ev:
            ev[0].record()
        merged = local_plan.merge(x_local)
        if ev:
            ev[1].record()
        dtype = q_local.dtype
        if kind == "frame":
            out, _ = varlen_fwd_rows(q_local, kv_local[:, 0], kv_local[:, 1], local_plan.cu_seqlens(1), local_plan.max_seqlen,
                                     local_plan.perkey_bias(dtype), self.scale, 0)
        else:
            out = self.exchange.attend(q_local, kv_local, self.scale, use_bias=True)
        if ev:
            ev[2].record()
        del merged
        y = out.reshape(local_plan.total, self.num_heads * self.head_dim)
        restored = local_plan.split(y).reshape(self.f_hi - self.f_lo, local_plan.tokens_per_frame, -1)
        if ev:
            ev[3].record()
            timers.append((kind, ev))
        return restored
