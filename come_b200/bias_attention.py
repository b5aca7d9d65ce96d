"""Attention module over packed (jagged) merged tokens with the per-key ``log(count)`` bias, mirroring
``JaggedAttention_w_Bias`` of the reference (``src/accelerate/vggt/module/bias_attention.py:84-137``).

Same constructor and ``forward(x, pos)`` contract.  The two linear layers stay PyTorch GEMMs as in the reference;
everything between them runs in two kernels of this library: ``come_qkv_prepare`` (q/k LayerNorm, 2-D rotary
embedding and the bias ``log(weight)`` in one pass, replacing ``prepare_packed_self_attention_qkv`` and the
``x.weight.float().log()`` expression) and the biased variable-length attention.
"""
from __future__ import annotations

from typing import Literal, Optional

import torch

from .flash_attn import (flash_attn_varlen_qkvpacked_func, flash_attn_varlen_qkvpacked_func_w_perkey_bias,
                         infer_flash_attn_varlen_max_seqlen)
from .qkv import RotaryPositionEmbedding2D, prepare_packed_self_attention_qkv
from .token_merger import JaggedTokens

__all__ = ["JaggedAttention_w_Bias"]


class _JaggedAttentionBase(torch.nn.Module):
    """What the two attention wrappers share: dtype handling, the rotary tables and the forward pass."""

    def __init__(self, original_attn: torch.nn.Module, run_dtype: str):
        super().__init__()
        if run_dtype == "bf16":
            self.run_dtype = torch.bfloat16
        elif run_dtype == "fp16":
            self.run_dtype = torch.float16
        else:
            raise ValueError(f"FlashAttention can only run on fp16/bf16, get {run_dtype}")
        self.attn = original_attn.to(dtype=self.run_dtype)
        rope = getattr(original_attn, "rope", None)
        if rope is None or isinstance(rope, RotaryPositionEmbedding2D):
            self._rope = rope
        else:  # the model's own rotary module: only its base frequency matters
            self._rope = RotaryPositionEmbedding2D(frequency=float(rope.base_frequency))

    def _attend_local(self, x: JaggedTokens, prepared, max_seqlen: Optional[int], use_bias: bool) -> torch.Tensor:
        cu_seqlens = x.cu_seqlens if x.cu_seqlens is not None else x.offset.to(torch.int32)
        max_seqlen_dev = None
        if max_seqlen is None:
            max_seqlen, max_seqlen_dev = x.max_seqlen, x.max_seqlen_dev
        if max_seqlen is None:
            max_seqlen = infer_flash_attn_varlen_max_seqlen(cu_seqlens)
        if use_bias:
            qkv, perkey_bias = prepared
            return flash_attn_varlen_qkvpacked_func_w_perkey_bias(qkv, cu_seqlens, max_seqlen, perkey_bias=perkey_bias,
                                                                  dropout_p=0.0, softmax_scale=self.attn.scale,
                                                                  max_seqlen_dev=max_seqlen_dev)
        return flash_attn_varlen_qkvpacked_func(prepared, cu_seqlens, max_seqlen, dropout_p=0.0,
                                                softmax_scale=self.attn.scale, max_seqlen_dev=max_seqlen_dev)

    def _attend_all_ranks(self, x: JaggedTokens, prepared, use_bias: bool) -> torch.Tensor:
        """These tokens are this rank's rows of one segment spread over the ranks: gather the prepared key / value rows
        of all ranks (the only exchange of the path) and attend the local query rows to them."""
        ex = x.exchange
        qkv = prepared[0] if use_bias else prepared
        return ex.attend(qkv[:, 0], qkv[:, 1:], self.attn.scale, use_bias)

    def _forward(self, x: JaggedTokens, pos: Optional[torch.Tensor], max_seqlen: Optional[int], use_bias: bool) -> JaggedTokens:
        attn = self.attn
        if self.training and getattr(getattr(attn, "attn_drop", None), "p", 0.0) > 0.0:
            raise NotImplementedError("attention dropout is not supported (inference path)")
        tokens = x.tokens.squeeze(0)  # (P, C)
        P, C = tokens.shape
        qkv = attn.qkv(tokens).reshape(P, 3, attn.num_heads, attn.head_dim)
        prepared = prepare_packed_self_attention_qkv(qkv, attn.q_norm, attn.k_norm, self._rope, pos, self.run_dtype,
                                                     weight=x.weight if use_bias else None)
        if x.exchange is not None:
            out = self._attend_all_ranks(x, prepared, use_bias)
        else:
            out = self._attend_local(x, prepared, max_seqlen, use_bias)
        out = attn.proj(out.reshape(P, C))
        proj_drop = getattr(attn, "proj_drop", None)
        if proj_drop is not None:
            out = proj_drop(out)
        return JaggedTokens(tokens=out.unsqueeze(0), weight=x.weight, offset=x.offset, max_seqlen=x.max_seqlen,
                            max_seqlen_dev=x.max_seqlen_dev, exchange=x.exchange, cu_seqlens=x.cu_seqlens)


class JaggedAttention_w_Bias(_JaggedAttentionBase):
    """``original_attn`` is an attention block with the attributes the reference's wrapper reads: ``qkv`` and
    ``proj`` (``nn.Linear``), ``q_norm`` / ``k_norm`` (``nn.LayerNorm(head_dim)`` or ``nn.Identity``), ``rope``
    (an object with ``base_frequency``, or None), ``num_heads``, ``head_dim``, ``scale``."""

    def __init__(self, original_attn: torch.nn.Module, run_dtype: Literal["bf16", "fp16"],
                 backend: Literal["flash_attn", "flex_attn"] = "flash_attn"):
        super().__init__(original_attn, run_dtype)
        if backend != "flash_attn":
            raise NotImplementedError(f"backend {backend!r}: only the CUDA attention kernel is provided")
        self.backend = backend

    def forward(self, x: JaggedTokens, pos: Optional[torch.Tensor] = None, *, max_seqlen: Optional[int] = None) -> JaggedTokens:
        """``max_seqlen`` (keyword, optional) is the longest segment if the caller already knows it, e.g. from a
        merge plan; ``x.max_seqlen`` / ``x.max_seqlen_dev`` serve the same purpose; without any of them the
        reference's device-to-host read is performed."""
        return self._forward(x, pos, max_seqlen, use_bias=True)
