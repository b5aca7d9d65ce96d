"""Pre-attention preparation of the packed qkv tensor, mirroring ``src/accelerate/common/qkv.py``.

``prepare_packed_self_attention_qkv(qkv, q_norm, k_norm, rope, pos, run_dtype)`` keeps the reference's name,
argument order and in-place inference semantics (``src/accelerate/common/qkv.py:7-39``) but runs as ONE kernel
(``come_qkv_prepare``): q/k LayerNorm over the head dimension, the 2-D rotary embedding and, when a ``weight``
vector is passed, the per-key bias ``log(weight)`` of the attention module
(``src/accelerate/vggt/module/bias_attention.py:120``).  There is no PyTorch fallback.
"""
from __future__ import annotations

import numpy as np
import torch

from . import _lib
from ._torch_util import dtype_code, ptr, require_cuda, stream_ptr

__all__ = ["RotaryPositionEmbedding2D", "prepare_packed_self_attention_qkv"]


def _round_to(x: np.ndarray, dtype: torch.dtype) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(dtype).float().numpy()


class RotaryPositionEmbedding2D:
    """Holder of the rotary tables with the constructor of the reference module
    (``src/thirdparty/vggt/layers/rope.py:79-85``).  The tables are built once per (feature_dim, dtype, device)
    on the host with the reference's arithmetic -- ``inv_freq = 1 / base ** (arange(0, dim, 2) / dim)``, angles
    rounded to the run dtype, cos / sin rounded again (``rope.py:87-114``) -- for ``max_position`` rows instead
    of ``positions.max() + 1``: row ``p`` does not depend on the table's length, and a fixed length needs no
    device-to-host read per call.  A position beyond the table raises the device status word.
    """

    def __init__(self, frequency: float = 100.0, scaling_factor: float = 1.0, max_position: int = 256):
        self.base_frequency = float(frequency)
        self.scaling_factor = float(scaling_factor)  # accepted and unused, as in the reference
        self.max_position = int(max_position)
        self.frequency_cache: dict = {}

    def tables(self, feature_dim: int, device, dtype: torch.dtype):
        key = (feature_dim, self.max_position, torch.device(device), dtype)
        if key not in self.frequency_cache:
            exponents = np.arange(0, feature_dim, 2, dtype=np.float32) / np.float32(feature_dim)
            inv_freq = (np.float32(1.0) / np.power(np.float32(self.base_frequency), exponents, dtype=np.float32))
            positions = np.arange(self.max_position, dtype=np.float32)
            angles = _round_to(positions[:, None] * inv_freq[None, :].astype(np.float32), dtype)
            angles = np.concatenate([angles, angles], axis=-1)
            cos = torch.from_numpy(np.cos(angles, dtype=np.float32)).to(dtype).to(device).contiguous()
            sin = torch.from_numpy(np.sin(angles, dtype=np.float32)).to(dtype).to(device).contiguous()
            self.frequency_cache[key] = (cos, sin)
        return self.frequency_cache[key]


def _norm_params(norm, name: str, D: int, dtype: torch.dtype, device):
    """(gamma, beta, eps) of an ``nn.LayerNorm(head_dim)``; (None, None, 0) for ``nn.Identity`` / None."""
    if norm is None or isinstance(norm, torch.nn.Identity):
        return None, None, 0.0
    if not isinstance(norm, torch.nn.LayerNorm):
        raise NotImplementedError(f"{name}: only nn.LayerNorm and nn.Identity are supported, got {type(norm).__name__}")
    if tuple(norm.normalized_shape) != (D,):
        raise RuntimeError(f"{name}: normalized_shape {tuple(norm.normalized_shape)} does not match head_dim {D}")
    w = norm.weight if norm.weight is not None else torch.ones(D, device=device)
    b = norm.bias if norm.bias is not None else torch.zeros(D, device=device)
    return (w.detach().to(device=device, dtype=dtype).contiguous(),
            b.detach().to(device=device, dtype=dtype).contiguous(), float(norm.eps))


def prepare_packed_self_attention_qkv(qkv: torch.Tensor, q_norm, k_norm, rope, pos, run_dtype: torch.dtype,
                                      weight: torch.Tensor | None = None):
    """Normalise packed q / k and apply the 2-D rotary embedding, IN PLACE, like the reference's inference branch.

    qkv       ``[P, 3, H, D]`` CUDA, contiguous, float16 or bfloat16 (== ``run_dtype``)
    q_norm    ``nn.LayerNorm(D)`` or ``nn.Identity`` (both or neither, as the attention module builds them)
    rope      a :class:`RotaryPositionEmbedding2D` or None
    pos       ``[1, P, 2]`` / ``[P, 2]`` int64 (y, x) or None
    weight    optional ``[P]`` float32 merge counts: when given the function returns ``(qkv, bias)`` with
              ``bias = log(weight)`` in ``run_dtype``, produced by the same kernel; otherwise it returns ``qkv``.

    Gradients are not supported (the reference's out-of-place training branch, ``qkv.py:21-27``, is outside the
    inference path): a tensor that requires grad is refused.
    """
    require_cuda(qkv, "qkv")
    if qkv.dim() != 4 or qkv.shape[1] != 3:
        raise RuntimeError(f"qkv must be [P, 3, H, D], got {tuple(qkv.shape)}")
    if qkv.requires_grad and torch.is_grad_enabled():
        raise RuntimeError("prepare_packed_self_attention_qkv: inference only (no autograd)")
    if qkv.dtype != run_dtype:
        raise RuntimeError(f"qkv dtype {qkv.dtype} != run_dtype {run_dtype}")
    if not qkv.is_contiguous():
        raise RuntimeError("qkv must be contiguous (it is updated in place)")
    P, _, H, D = qkv.shape
    dev = qkv.device
    code = dtype_code(run_dtype, "qkv")
    qg, qb, q_eps = _norm_params(q_norm, "q_norm", D, run_dtype, dev)
    kg, kb, k_eps = _norm_params(k_norm, "k_norm", D, run_dtype, dev)
    if (qg is None) != (kg is None):
        raise NotImplementedError("q_norm and k_norm must both be LayerNorm or both Identity")
    if qg is not None and q_eps != k_eps:
        raise NotImplementedError("q_norm and k_norm must share eps")
    cos = sin = None
    rows = 0
    if rope is not None and pos is not None:
        pos = pos.reshape(-1, 2)
        if pos.shape[0] != P or pos.dtype != torch.int64:
            raise RuntimeError(f"pos must hold {P} int64 (y, x) pairs, got {tuple(pos.shape)} {pos.dtype}")
        require_cuda(pos, "pos")
        pos = pos.contiguous()
        cos, sin = rope.tables(D // 2, dev, run_dtype)
        rows = cos.shape[0]
    else:
        pos = None
    bias = None
    if weight is not None:
        require_cuda(weight, "weight")
        if weight.shape != (P,):
            raise RuntimeError(f"weight must be [{P}], got {tuple(weight.shape)}")
        weight = weight.to(torch.float32).contiguous()
        bias = torch.empty(P, dtype=run_dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().come_qkv_prepare(
            ptr(qkv), code, P, H, D, ptr(qg), ptr(qb), ptr(kg), ptr(kb), q_eps, ptr(pos), ptr(cos), ptr(sin), rows,
            ptr(weight), ptr(bias), stream_ptr(dev)))
    return qkv if weight is None else (qkv, bias)
