"""Random-initialised transformer blocks with the attribute layout of the VGGT aggregator, for tests and benchmarks
of the merged forward pass (there are no pretrained weights to load).

The accelerated modules of this package (:mod:`come_b200.block`, :mod:`come_b200.fused`) only read attributes:
``block.norm1 / attn / ls1 / norm2 / mlp / ls2`` (``src/thirdparty/vggt/layers/block.py:43-66``) and
``attn.qkv / proj / q_norm / k_norm / rope / num_heads / head_dim / scale``
(``src/thirdparty/vggt/layers/attention.py:31-44``); ``aggregator.frame_blocks / global_blocks / aa_order /
aa_block_size / aa_block_num / retain_layers / patch_start_idx`` (``src/thirdparty/vggt/models/aggregator.py:76-131``).
The classes here provide exactly those, with the VGGT-1B sizes as defaults: width 1024, 16 heads, MLP ratio 4, q/k
LayerNorm over the head dimension, 2-D rotary embedding with base 100, LayerScale 0.01, 24 frame + 24 global blocks.
The dense ``forward`` methods of the original model are not provided: the blocks are run by the jagged block
wrappers, on merged or unmerged tokens alike.
"""
from __future__ import annotations

from typing import FrozenSet, Optional, Sequence

import torch
from torch import nn

from .qkv import RotaryPositionEmbedding2D

__all__ = ["LayerScale", "Mlp", "Attention", "Block", "AggregatorCore"]


class LayerScale(nn.Module):
    def __init__(self, dim: int, init_values: float = 0.01):
        super().__init__()
        self.gamma = nn.Parameter(torch.full((dim,), float(init_values)))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x * self.gamma


class Mlp(nn.Module):
    def __init__(self, dim: int, hidden: int, bias: bool = True):
        super().__init__()
        self.fc1 = nn.Linear(dim, hidden, bias=bias)
        self.act = nn.GELU()
        self.fc2 = nn.Linear(hidden, dim, bias=bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.fc2(self.act(self.fc1(x)))


class Attention(nn.Module):
    """Parameter holder of a self-attention layer; evaluated by ``JaggedAttention`` / ``JaggedAttention_w_Bias``."""

    def __init__(self, dim: int, num_heads: int, qkv_bias: bool = True, proj_bias: bool = True, qk_norm: bool = True,
                 rope: Optional[RotaryPositionEmbedding2D] = None):
        super().__init__()
        if dim % num_heads != 0:
            raise ValueError("dim should be divisible by num_heads")
        self.num_heads = num_heads
        self.head_dim = dim // num_heads
        self.scale = self.head_dim ** -0.5
        self.qkv = nn.Linear(dim, 3 * dim, bias=qkv_bias)
        self.q_norm = nn.LayerNorm(self.head_dim) if qk_norm else nn.Identity()
        self.k_norm = nn.LayerNorm(self.head_dim) if qk_norm else nn.Identity()
        self.attn_drop = nn.Dropout(0.0)
        self.proj = nn.Linear(dim, dim, bias=proj_bias)
        self.proj_drop = nn.Dropout(0.0)
        self.rope = rope


class Block(nn.Module):
    def __init__(self, dim: int, num_heads: int, mlp_ratio: float = 4.0, init_values: Optional[float] = 0.01,
                 qk_norm: bool = True, rope: Optional[RotaryPositionEmbedding2D] = None):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim)
        self.attn = Attention(dim, num_heads, qk_norm=qk_norm, rope=rope)
        self.ls1 = LayerScale(dim, init_values) if init_values else nn.Identity()
        self.norm2 = nn.LayerNorm(dim)
        self.mlp = Mlp(dim, int(dim * mlp_ratio))
        self.ls2 = LayerScale(dim, init_values) if init_values else nn.Identity()


class AggregatorCore(nn.Module):
    """The alternating-attention stack of the aggregator (everything after the patch encoder)."""

    def __init__(self, embed_dim: int = 1024, depth: int = 24, num_heads: int = 16, mlp_ratio: float = 4.0,
                 aa_order: Sequence[str] = ("frame", "global"), aa_block_size: int = 1, qk_norm: bool = True,
                 rope_freq: float = 100.0, init_values: Optional[float] = 0.01,
                 retain_layers: Optional[FrozenSet[int]] = frozenset({4, 11, 17, 23}), patch_start_idx: int = 5,
                 seed: int = 0, weight_std: float = 0.02):
        super().__init__()
        if depth % aa_block_size != 0:
            raise ValueError(f"depth ({depth}) must be divisible by aa_block_size ({aa_block_size})")
        self.rope = RotaryPositionEmbedding2D(frequency=rope_freq) if rope_freq > 0 else None
        mk = lambda: Block(embed_dim, num_heads, mlp_ratio, init_values, qk_norm, self.rope)  # noqa: E731
        self.frame_blocks = nn.ModuleList([mk() for _ in range(depth)])
        self.global_blocks = nn.ModuleList([mk() for _ in range(depth)])
        self.depth, self.aa_order, self.aa_block_size = depth, list(aa_order), aa_block_size
        self.aa_block_num = depth // aa_block_size
        self.retain_layers = retain_layers
        self.patch_start_idx = patch_start_idx
        gen = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                if name.endswith("gamma"):
                    continue  # LayerScale keeps its init value
                if p.dim() == 2:
                    p.copy_(torch.randn(p.shape, generator=gen) * weight_std)
                elif "norm" in name and name.endswith("weight"):
                    p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=gen))
                else:
                    p.copy_(0.02 * torch.randn(p.shape, generator=gen))
        self.eval()
