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

__all__ = ["CoMeOpChain"]


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
