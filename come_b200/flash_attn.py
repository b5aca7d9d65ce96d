"""Forward-only variable-length attention API with the reference's names and argument meaning
(``src/cuda_extension/flash_attn/__init__.py:21-33,235-295,439-477``), backed by the sm_100a kernels.

``flash_attn_varlen_qkvpacked_func_w_perkey_bias`` computes, per packed segment and head,
``softmax(Q @ K.T * scale + perkey_bias[kv_idx]) @ V``.  Backward raises ``RuntimeError`` like the reference.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import flash_attn_fwd_cuda as _C

ONNX_DOMAIN = "comesdk"
FLASH_ATTN_VARLEN_QKVPACKED_OP = "FlashAttnVarlenQKVPacked"
FLASH_ATTN_VARLEN_QKVPACKED_W_BIAS_OP = "FlashAttnVarlenQKVPackedWBias"

__all__ = [
    "FLASH_ATTN_VARLEN_QKVPACKED_OP",
    "FLASH_ATTN_VARLEN_QKVPACKED_W_BIAS_OP",
    "ONNX_DOMAIN",
    "flash_attn_varlen_qkvpacked_func",
    "flash_attn_varlen_qkvpacked_func_w_perkey_bias",
    "infer_flash_attn_varlen_max_seqlen",
]


def infer_flash_attn_varlen_max_seqlen(cu_seqlens: torch.Tensor) -> int:
    """Longest segment as a Python int (0 while an ONNX export is tracing); forces a device->host read.
    A :class:`come_b200.token_merger.MergePlan` already carries this number without a read."""
    if torch.onnx.is_in_onnx_export():
        return 0
    return int((cu_seqlens[1:] - cu_seqlens[:-1]).max().item())


def _pad_head(t: torch.Tensor, head_size_og: int) -> torch.Tensor:
    if head_size_og % 8 != 0:
        return torch.nn.functional.pad(t, [0, 8 - head_size_og % 8])
    return t


class _VarlenQKVPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cu_seqlens, max_seqlen, perkey_bias, has_bias, dropout_p, softmax_scale, causal,
                window_size, softcap, alibi_slopes, return_softmax, max_seqlen_dev=None):
        if softmax_scale is None:
            softmax_scale = qkv.shape[-1] ** (-0.5)
        q, k, v = qkv[:, 0].detach(), qkv[:, 1].detach(), qkv[:, 2].detach()
        head_size_og = q.size(2)
        q, k, v = (_pad_head(x, head_size_og) for x in (q, k, v))
        common = (dropout_p, softmax_scale, False, causal, window_size[0], window_size[1], softcap,
                  return_softmax and dropout_p > 0, None)
        if has_bias:
            out_padded, softmax_lse, S_dmask, rng_state = _C.varlen_fwd_w_perkey_bias(
                q, k, v, None, cu_seqlens, cu_seqlens, None, None, None, alibi_slopes, perkey_bias,
                max_seqlen, max_seqlen, *common, max_seqlen_dev=max_seqlen_dev)
        else:
            out_padded, softmax_lse, S_dmask, rng_state = _C.varlen_fwd(
                q, k, v, None, cu_seqlens, cu_seqlens, None, None, None, alibi_slopes, max_seqlen, max_seqlen, *common,
                max_seqlen_dev=max_seqlen_dev)
        ctx.mark_non_differentiable(softmax_lse, S_dmask, rng_state)
        out = out_padded[..., :head_size_og]
        return out if not return_softmax else (out, softmax_lse, S_dmask)

    @staticmethod
    def backward(ctx, *args):
        raise RuntimeError(
            "flash_attn_varlen_qkvpacked_func backward is not supported in this forward-only build.")


def flash_attn_varlen_qkvpacked_func(
    qkv: torch.Tensor,
    cu_seqlens: torch.Tensor,
    max_seqlen: int,
    dropout_p: float = 0.0,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
    window_size: Tuple[int, int] = (-1, -1),
    softcap: float = 0.0,
    alibi_slopes: Optional[torch.Tensor] = None,
    deterministic: bool = False,
    return_attn_probs: bool = False,
    *,
    max_seqlen_dev: Optional[torch.Tensor] = None,
):
    """Attention over packed variable-length segments.

    Arguments:
        qkv: ``(total, 3, nheads, headdim)`` fp16 / bf16.
        cu_seqlens: ``(batch_size + 1,)`` int32 cumulative segment lengths.
        max_seqlen: longest segment.
        softmax_scale: defaults to ``1 / sqrt(headdim)``.
        dropout_p, causal, window_size, softcap, alibi_slopes: accepted for signature compatibility; any value
            other than the inference defaults raises ``NotImplementedError``.
        max_seqlen_dev (keyword only, not in the reference): one-element int32 device tensor with the exact longest
            segment when ``max_seqlen`` is only an upper bound (launches of fixed shape, e.g. inside a CUDA graph).
    Return:
        out ``(total, nheads, headdim)``; with ``return_attn_probs`` also ``softmax_lse (nheads, total)`` and an
        empty probabilities tensor.
    """
    return _VarlenQKVPacked.apply(qkv, cu_seqlens, max_seqlen, None, False, dropout_p, softmax_scale, causal,
                                  tuple(window_size), softcap, alibi_slopes, return_attn_probs, max_seqlen_dev)


def flash_attn_varlen_qkvpacked_func_w_perkey_bias(
    qkv: torch.Tensor,
    cu_seqlens: torch.Tensor,
    max_seqlen: int,
    perkey_bias: torch.Tensor,
    dropout_p: float = 0.0,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
    window_size: Tuple[int, int] = (-1, -1),
    softcap: float = 0.0,
    alibi_slopes: Optional[torch.Tensor] = None,
    deterministic: bool = False,
    return_attn_probs: bool = False,
    *,
    max_seqlen_dev: Optional[torch.Tensor] = None,
):
    """Same as :func:`flash_attn_varlen_qkvpacked_func` with an additive per-key bias on the scaled scores:
    ``softmax(Q @ K.T * scale + perkey_bias[kv_idx]) @ V``.

    Arguments:
        perkey_bias: ``(total,)`` tensor, same dtype as ``qkv``, indexed like the packed K/V rows.
    """
    return _VarlenQKVPacked.apply(qkv, cu_seqlens, max_seqlen, perkey_bias, True, dropout_p, softmax_scale, causal,
                                  tuple(window_size), softcap, alibi_slopes, return_attn_probs, max_seqlen_dev)
