"""Attention module over packed (jagged) tokens without the count bias, mirroring ``JaggedAttention`` of the
reference (``src/accelerate/vggt/module/plain_attention.py:13-55``): what the accelerated model uses when
``use_attn_bias_correction`` is off, and what runs a block on unmerged tokens.

Same constructor and ``forward(x, pos)`` contract; between the two PyTorch GEMMs run ``come_qkv_prepare`` (q/k
LayerNorm and the 2-D rotary embedding in one pass) and the variable-length attention kernel.
"""
from __future__ import annotations

from typing import Literal, Optional

import torch

from .bias_attention import _JaggedAttentionBase
from .token_merger import JaggedTokens

__all__ = ["JaggedAttention"]


class JaggedAttention(_JaggedAttentionBase):
    SupportType = Literal["fp16", "bf16"]

    def __init__(self, original_attn: torch.nn.Module, run_dtype: "JaggedAttention.SupportType"):
        super().__init__(original_attn, run_dtype)

    def forward(self, x: JaggedTokens, pos: Optional[torch.Tensor] = None, *, max_seqlen: Optional[int] = None) -> JaggedTokens:
        return self._forward(x, pos, max_seqlen, use_bias=False)
