"""Per-layer ("direct") acceleration of an attention block, mirroring the forward the reference patches into every
VGGT attention module (``src/accelerate/vggt/direct.py:71-124``): merge the dense tokens, run the jagged attention
with the ``log(count)`` key bias on the merged tokens, split back to the dense layout.

Differences from the reference's closure, none of them visible in the result:

* the index plan (offsets, ``rev_id``, counts, longest segment, packed positions) comes from a
  :class:`~come_b200.token_merger.MergePlan` built once per scene, not from a fresh merge of the features and a second
  merge of the positions in every layer;
* frame and global segmentation are two views of the plan's offsets (``cu_seqlens(1)`` / ``cu_seqlens(S)``), and the
  longest segment is known without a device-to-host read.
"""
from __future__ import annotations

from typing import Optional

import torch

from .bias_attention import JaggedAttention_w_Bias
from .token_merger import JaggedTokens, MergePlan

__all__ = ["DirectAttention", "DirectMlp"]


class DirectAttention(torch.nn.Module):
    """Drop-in for ``block.attn.forward(x, pos)`` of a frame (``is_global=False``) or global attention block.

    ``x`` is ``[B*S, N, C]`` (frame blocks) or ``[B, S*N, C]`` (global blocks) exactly as the aggregator passes it;
    the result has the same shape and dtype.  ``plan`` is the merge plan of the current scene(s) with
    ``frames = B*S``; ``frames_per_scene = S``.
    """

    def __init__(self, original_attn: torch.nn.Module, *, is_global: bool, run_dtype: str = "bf16"):
        super().__init__()
        self.is_global = is_global
        self.attn_op = JaggedAttention_w_Bias(original_attn, run_dtype=run_dtype)

    def forward(self, x: torch.Tensor, plan: MergePlan, frames_per_scene: int, use_pos: bool = True) -> torch.Tensor:
        input_shape, input_dtype = x.shape, x.dtype
        C = x.shape[-1]
        dense = x.reshape(plan.frames, plan.tokens_per_frame, C).to(self.attn_op.run_dtype)
        merged = plan.merge(dense)
        if self.is_global:
            offset = plan.offset[::frames_per_scene]
            max_seqlen = plan.total if plan.frames == frames_per_scene else None  # several scenes: read it back
        else:
            offset, max_seqlen = plan.offset, plan.max_seqlen
        jag = JaggedTokens(tokens=merged.unsqueeze(0), weight=plan.weight, offset=offset)
        pos: Optional[torch.Tensor] = plan.positions() if use_pos else None
        out = self.attn_op(jag, pos=pos, max_seqlen=max_seqlen)
        return plan.split(out.tokens.squeeze(0)).view(*input_shape).to(input_dtype)

    def forward_residual(self, x: torch.Tensor, plan: MergePlan, frames_per_scene: int, norm1: torch.nn.LayerNorm,
                         ls1_gamma: Optional[torch.Tensor] = None, use_pos: bool = True) -> torch.Tensor:
        """The whole attention branch of a block, ``x + ls1(attn(norm1(x)))`` (``src/thirdparty/vggt/layers/block.py:73,90``),
        with the dense tokens read once and written once: ``norm1`` runs inside the merge (``come_merge_layernorm``), the
        unmerge applies LayerScale and adds the residual (``come_unmerge_residual``).  ``x`` must already be in the run
        dtype (the block's tensors in the reference's per-layer mode are)."""
        if x.dtype != self.attn_op.run_dtype:
            raise RuntimeError(f"forward_residual expects tokens in {self.attn_op.run_dtype}, got {x.dtype}")
        input_shape = x.shape
        C = x.shape[-1]
        dense = x.reshape(plan.frames, plan.tokens_per_frame, C)
        merged = plan.merge_layernorm(dense, norm1)
        if self.is_global:
            offset = plan.offset[::frames_per_scene]
            max_seqlen = plan.total if plan.frames == frames_per_scene else None
        else:
            offset, max_seqlen = plan.offset, plan.max_seqlen
        jag = JaggedTokens(tokens=merged.unsqueeze(0), weight=plan.weight, offset=offset)
        out = self.attn_op(jag, pos=plan.positions() if use_pos else None, max_seqlen=max_seqlen)
        gamma = None if ls1_gamma is None else ls1_gamma.detach().to(device=x.device, dtype=x.dtype)
        return plan.split_add(out.tokens.squeeze(0), dense, gamma).view(*input_shape)


class DirectMlp(torch.nn.Module):
    """Drop-in for ``block.mlp.forward(x)`` in the per-layer mode (``src/accelerate/vggt/direct.py:148-168``): the MLP runs
    on the merged tokens -- a merged window passes through ``fc1 -> act -> fc2`` once instead of ``G`` times -- and the
    result is split back to the dense layout.  ``x`` is ``[B*S, N, C]`` or ``[B, S*N, C]`` as the aggregator passes it;
    the result has the same shape and dtype.  The two GEMMs stay the module's own (PyTorch); merge and split are this
    library's kernels driven by the scene's :class:`~come_b200.token_merger.MergePlan`."""

    def __init__(self, original_mlp: torch.nn.Module):
        super().__init__()
        self.mlp = original_mlp

    def forward(self, x: torch.Tensor, plan: MergePlan) -> torch.Tensor:
        input_shape = x.shape
        C = x.shape[-1]
        merged = plan.merge(x.reshape(plan.frames, plan.tokens_per_frame, C))
        out = self.mlp(merged.unsqueeze(0)).squeeze(0)
        return plan.split(out.contiguous()).view(*input_shape)

    def forward_residual(self, x: torch.Tensor, plan: MergePlan, norm2: torch.nn.LayerNorm,
                         ls2_gamma: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The whole MLP branch of a block, ``x + ls2(mlp(norm2(x)))`` (``src/thirdparty/vggt/layers/block.py:74,91``), with
        the dense tokens read once and written once: ``norm2`` inside the merge, LayerScale and the residual add inside
        the unmerge."""
        input_shape = x.shape
        C = x.shape[-1]
        dense = x.reshape(plan.frames, plan.tokens_per_frame, C)
        merged = plan.merge_layernorm(dense, norm2)
        out = self.mlp(merged.unsqueeze(0)).squeeze(0)
        gamma = None if ls2_gamma is None else ls2_gamma.detach().to(device=x.device, dtype=x.dtype)
        return plan.split_add(out.contiguous(), dense, gamma).view(*input_shape)
