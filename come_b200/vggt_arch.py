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

__all__ = ["LayerScale", "Mlp", "Attention", "Block", "AggregatorCore", "PatchEncoderCore", "ConfidenceHead"]


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
        # camera and register tokens: entry 0 for the first frame of a scene, entry 1 for the others
        # (src/thirdparty/vggt/models/aggregator.py:117-126, slice_expand_and_flatten :335-360)
        self.camera_token = nn.Parameter(torch.zeros(1, 2, 1, embed_dim))
        self.register_token = nn.Parameter(torch.zeros(1, 2, patch_start_idx - 1, embed_dim))
        gen = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                if name.endswith("gamma"):
                    continue  # LayerScale keeps its init value
                if name.endswith("_token"):
                    p.copy_(torch.randn(p.shape, generator=gen) * 1e-1)
                elif p.dim() == 2:
                    p.copy_(torch.randn(p.shape, generator=gen) * weight_std)
                elif "norm" in name and name.endswith("weight"):
                    p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=gen))
                else:
                    p.copy_(0.02 * torch.randn(p.shape, generator=gen))
        self.eval()

    def assemble_tokens(self, patch_tokens: torch.Tensor, B: int, S: int) -> torch.Tensor:
        """``patch_tokens [B*S, h*w, C]`` -> ``[B, S, patch_start_idx + h*w, C]`` with the camera and register tokens in
        front of every frame (``aggregator.py:205-215``)."""
        Cc = patch_tokens.shape[-1]

        def expand(tok):  # [1, 2, X, C] -> [B*S, X, C]: entry 0 for frame 0 of every scene, entry 1 for the rest
            first = tok[:, 0:1].expand(B, 1, -1, -1)
            rest = tok[:, 1:2].expand(B, S - 1, -1, -1)
            return torch.cat([first, rest], dim=1).reshape(B * S, -1, Cc)

        cam, reg = expand(self.camera_token.to(patch_tokens.dtype)), expand(self.register_token.to(patch_tokens.dtype))
        return torch.cat([cam, reg, patch_tokens], dim=1).reshape(B, S, -1, Cc)


class PatchEncoderCore(nn.Module):
    """Patch encoder in the shape of the ViT-L/14 with four register tokens that VGGT uses (``aggregator.py:76-101``:
    DINOv2 ``vit_large``, patch 14, ``num_register_tokens=4``, LayerScale, no q/k norm, no rotary embedding): patch
    embedding, class + register tokens, learned position embedding, ``depth`` blocks, final norm.  Random-initialised;
    the blocks are evaluated by the jagged block wrappers like the aggregator's."""

    def __init__(self, embed_dim: int = 1024, depth: int = 24, num_heads: int = 16, patch_size: int = 14, registers: int = 4,
                 grid: Sequence[int] = (37, 37), mlp_ratio: float = 4.0, init_values: Optional[float] = 1.0, seed: int = 1,
                 weight_std: float = 0.02):
        super().__init__()
        self.patch_size, self.registers, self.embed_dim = patch_size, registers, embed_dim
        self.num_features = embed_dim
        self.proj = nn.Conv2d(3, embed_dim, kernel_size=patch_size, stride=patch_size)
        self.cls_token = nn.Parameter(torch.zeros(1, 1, embed_dim))
        self.register_tokens = nn.Parameter(torch.zeros(1, registers, embed_dim))
        self.pos_embed = nn.Parameter(torch.zeros(1, 1 + grid[0] * grid[1], embed_dim))  # class token + patches
        self.grid = tuple(grid)
        self.blocks = nn.ModuleList([Block(embed_dim, num_heads, mlp_ratio, init_values, qk_norm=False, rope=None)
                                     for _ in range(depth)])
        self.norm = nn.LayerNorm(embed_dim, eps=1e-6)
        gen = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                if name.endswith("gamma"):
                    continue
                if name in ("cls_token", "register_tokens", "pos_embed"):
                    p.copy_(torch.randn(p.shape, generator=gen) * weight_std)
                elif p.dim() >= 2:
                    p.copy_(torch.randn(p.shape, generator=gen) * weight_std)
                elif "norm" in name and name.endswith("weight"):
                    p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=gen))
                else:
                    p.copy_(0.02 * torch.randn(p.shape, generator=gen))
        self.eval()

    @property
    def prefix_tokens(self) -> int:
        return 1 + self.registers

    def embed(self, images: torch.Tensor) -> torch.Tensor:
        """``images [F, 3, H, W]`` -> tokens ``[F, 1 + registers + h*w, C]``: class token, register tokens, patches."""
        Fr, _, Hh, Ww = images.shape
        h, w = Hh // self.patch_size, Ww // self.patch_size
        if (h, w) != self.grid:
            raise ValueError(f"images give a {h}x{w} patch grid, the position embedding was built for {self.grid}")
        x = self.proj(images.to(self.proj.weight.dtype)).flatten(2).transpose(1, 2)  # [F, h*w, C]
        x = torch.cat([self.cls_token.expand(Fr, -1, -1), x], dim=1) + self.pos_embed
        return torch.cat([x[:, :1], self.register_tokens.expand(Fr, -1, -1), x[:, 1:]], dim=1)


class ConfidenceHead(nn.Module):
    """Seeded two-layer MLP ``C -> hidden -> 1`` on the patch tokens: the stand-in for the distilled confidence predictor
    in the synthetic benchmark configurations.  Call signature of the reference's predictor
    (``feature [B, S, H, W, C]``, ``BPHWC=...`` -> ``[B, S*H*W, 1]``)."""

    def __init__(self, embed_dim: int = 1024, hidden: int = 128, seed: int = 2):
        super().__init__()
        self.fc1, self.act, self.fc2 = nn.Linear(embed_dim, hidden), nn.GELU(), nn.Linear(hidden, 1)
        gen = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for p in self.parameters():
                p.copy_(torch.randn(p.shape, generator=gen) * (0.05 if p.dim() == 2 else 0.01))
        self.eval()

    def forward(self, feature: torch.Tensor, BPHWC=None) -> torch.Tensor:
        B = feature.shape[0]
        return self.fc2(self.act(self.fc1(feature.to(self.fc1.weight.dtype)))).reshape(B, -1, 1)
