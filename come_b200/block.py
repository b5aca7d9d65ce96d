"""Transformer blocks over packed (jagged) tokens, mirroring ``JaggedBlock`` and ``JaggedBlock_w_Bias`` of the
reference (``src/accelerate/vggt/module/block.py:18-81``).

A wrapper takes an existing block (``norm1, attn, ls1, norm2, mlp, ls2``) and evaluates it on
:class:`~come_b200.token_merger.JaggedTokens`: the attention branch through the jagged attention module of this
package in ``attn_dtype``, everything else (the norms, the MLP, LayerScale, the residual adds) as the PyTorch
modules the block already holds, in the dtype of the incoming tokens -- the order and the casts of the reference's
``forward`` (``block.py:58-81``).
"""
from __future__ import annotations

from typing import Optional

import torch

from .bias_attention import JaggedAttention_w_Bias
from .plain_attention import JaggedAttention
from .token_merger import JaggedTokens

__all__ = ["JaggedBlock", "JaggedBlock_w_Bias"]


class _JaggedBlockBase(torch.nn.Module):
    attention_class = None

    def __init__(self, original_block: torch.nn.Module, attn_dtype: str):
        super().__init__()
        if original_block.training:
            raise AssertionError(f"{type(self).__name__} is invalid in training mode!")
        self.block = original_block
        self.attn = type(self).attention_class(original_block.attn, run_dtype=attn_dtype)

    def forward(self, x: JaggedTokens, pos: Optional[torch.Tensor] = None) -> JaggedTokens:
        block = self.block
        original_dtype, attn_dtype = x.tokens.dtype, self.attn.run_dtype
        # attention sub-block: x + ls1(attn(norm1(x)))
        attn_x = self.attn(x.apply(block.norm1).apply(lambda y: y.to(dtype=attn_dtype)), pos=pos)
        attn_x = attn_x.apply(lambda y: y.to(dtype=original_dtype)).apply(block.ls1)
        x = x.apply(lambda residual_x: residual_x + attn_x.tokens)
        # MLP sub-block: x + ls2(mlp(norm2(x)))
        mlp_x = x.apply(block.norm2).apply(block.mlp).apply(block.ls2)
        return x.apply(lambda residual_x: residual_x + mlp_x.tokens)


class JaggedBlock(_JaggedBlockBase):
    """Block without the count bias (``block.py:18-43``)."""
    attention_class = JaggedAttention


class JaggedBlock_w_Bias(_JaggedBlockBase):
    """Block whose attention adds ``log(weight)`` per key (``block.py:46-81``)."""
    attention_class = JaggedAttention_w_Bias
