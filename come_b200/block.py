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

__all__ = ["JaggedBlock", "JaggedBlock_w_Bias", "residual_layernorm", "fusable", "forward_fused"]


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


# ---------------------------------------------------------------------------------------------------------------
# the block with its elementwise steps fused
# ---------------------------------------------------------------------------------------------------------------
def residual_layernorm(x: torch.Tensor, branch: Optional[torch.Tensor], scale: Optional[torch.Tensor],
                       norm: Optional[torch.nn.LayerNorm], store_stream: bool = True):
    """``x_out = x + scale * branch`` and ``normed = norm(x_out)`` in one pass over packed rows ``[P, C]``
    (``come_residual_layernorm``): the LayerScale, the residual add and the next LayerNorm of the jagged block
    (``src/accelerate/vggt/module/block.py:66-79``), which the module path runs as three elementwise kernels.
    ``branch`` None: the norm of ``x`` alone; ``scale`` None: no LayerScale; ``norm`` None: the update alone.
    Returns ``(x_out, normed)``; ``x_out`` is ``x`` itself when there is no branch and None when ``store_stream`` is off."""
    from . import _lib
    from ._torch_util import dtype_code, ptr, require_cuda, stream_ptr
    require_cuda(x, "x")
    if x.dim() != 2 or not x.is_contiguous():
        raise ValueError(f"x must be a contiguous [rows, C] tensor, got {tuple(x.shape)}")
    rows, Cc = x.shape
    dt, dev = x.dtype, x.device
    if branch is not None and (branch.shape != x.shape or branch.dtype != dt or not branch.is_contiguous()):
        raise ValueError(f"branch must be contiguous and match x {tuple(x.shape)} {dt}, got {tuple(branch.shape)} {branch.dtype}")
    if scale is not None:
        if branch is None:
            raise ValueError("scale without a branch")
        scale = scale.detach().to(device=dev, dtype=dt).contiguous()
        if scale.shape != (Cc,):
            raise ValueError(f"scale must be [{Cc}], got {tuple(scale.shape)}")
    gamma = beta = None
    eps = 0.0
    if norm is not None:
        if not isinstance(norm, torch.nn.LayerNorm) or tuple(norm.normalized_shape) != (Cc,):
            raise NotImplementedError("residual_layernorm needs an nn.LayerNorm over the channel dimension")
        gamma = (norm.weight if norm.weight is not None else torch.ones(Cc, device=dev)).detach().to(device=dev, dtype=dt).contiguous()
        beta = (norm.bias if norm.bias is not None else torch.zeros(Cc, device=dev)).detach().to(device=dev, dtype=dt).contiguous()
        eps = float(norm.eps)
    elif branch is None:
        raise ValueError("nothing to compute: neither a branch nor a norm")
    x_out = torch.empty_like(x) if (branch is not None and store_stream) else None
    normed = torch.empty_like(x) if norm is not None else None
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().come_residual_layernorm(ptr(x), ptr(branch), ptr(scale), rows, Cc, dtype_code(dt, "x"), ptr(gamma),
                                                      ptr(beta), eps, ptr(x_out), ptr(normed), stream_ptr(dev)))
    return (x if branch is None else x_out), normed


def _layer_scale_gamma(ls: torch.nn.Module):
    """(supported, gamma or None) of a LayerScale-like module: ``x * gamma`` or the identity."""
    if isinstance(ls, torch.nn.Identity):
        return True, None
    gamma = getattr(ls, "gamma", None)
    return (isinstance(gamma, torch.Tensor) and gamma.dim() == 1), gamma


def fusable(wrapper: _JaggedBlockBase, dtype: torch.dtype) -> bool:
    """Whether :func:`forward_fused` can evaluate this block: residual stream already in the attention dtype, plain
    ``nn.LayerNorm`` norms and LayerScale (or identity) scales."""
    b = wrapper.block
    return (dtype == wrapper.attn.run_dtype and isinstance(b.norm1, torch.nn.LayerNorm) and isinstance(b.norm2, torch.nn.LayerNorm)
            and _layer_scale_gamma(b.ls1)[0] and _layer_scale_gamma(b.ls2)[0])


def forward_fused(wrapper: _JaggedBlockBase, x: JaggedTokens, normed: torch.Tensor, pos: Optional[torch.Tensor],
                  next_norm: Optional[torch.nn.LayerNorm]):
    """The block of :class:`JaggedBlock` / :class:`JaggedBlock_w_Bias` with each ``LayerScale -> residual add ->
    LayerNorm`` run as one kernel.  ``normed`` is ``norm1(x.tokens)`` (computed by the previous block's call, or by
    :func:`residual_layernorm` for the first block); ``next_norm`` is the ``norm1`` of the block that follows (None after
    the last).  Returns ``(x_out, next_normed)``.  Same arithmetic as the module path up to the summation order inside
    the LayerNorm statistics."""
    block = wrapper.block
    P, Cc = x.tokens.shape[1], x.tokens.shape[2]
    attn_x = wrapper.attn(JaggedTokens(normed.unsqueeze(0), x.weight, x.offset, x.max_seqlen, x.max_seqlen_dev, x.exchange, x.cu_seqlens), pos=pos)
    stream, h = residual_layernorm(x.tokens.reshape(P, Cc), attn_x.tokens.reshape(P, Cc), _layer_scale_gamma(block.ls1)[1], block.norm2)
    mlp_x = block.mlp(h)
    stream, next_normed = residual_layernorm(stream, mlp_x, _layer_scale_gamma(block.ls2)[1], next_norm)
    return JaggedTokens(stream.unsqueeze(0), x.weight, x.offset, x.max_seqlen, x.max_seqlen_dev, x.exchange, x.cu_seqlens), next_normed
