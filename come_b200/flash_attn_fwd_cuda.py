"""Stand-in for the reference's compiled ``flash_attn_fwd_cuda`` module
(``src/cuda_extension/flash_attn/flash_api.cpp:538-607``): ``varlen_fwd`` and ``varlen_fwd_w_perkey_bias``
with the reference's positional signature and return value ``[out, softmax_lse, p, rng_state]``.

Only what the Co-Me inference path uses is implemented (self-attention over packed segments, no dropout,
non-causal, no window, no softcap, no ALiBi, no paged KV); every other request raises instead of being
ignored.
"""
from __future__ import annotations

import threading

import torch

from . import _lib
from ._torch_util import dtype_code, ptr, stream_ptr

__all__ = ["varlen_fwd", "varlen_fwd_w_perkey_bias", "varlen_fwd_rows", "cross_fwd", "cross_fwd_balanced", "plan_tail_split",
           "combine"]

BACKEND_AUTO, BACKEND_CUDA_CORE, BACKEND_TCGEN05 = 0, 1, 2
_backend = BACKEND_AUTO


def set_backend(backend: int) -> int:
    """Select the attention kernel (0 automatic, 1 CUDA-core kernel, 2 require tcgen05); returns the old value."""
    global _backend
    old, _backend = _backend, int(backend)
    return old


class cta_limit:
    """``with cta_limit(n):`` the tensor-core attention launches of this thread inside the block use at most ``n`` CTAs
    (``come_attn_set_cta_limit``), leaving the other SMs to a kernel that runs beside them; ``n <= 0``: no limit."""

    current = threading.local()  # the limit in force in this thread (0: none), for callers that size their launches by it

    def __init__(self, max_ctas: int):
        self.max_ctas = max(int(max_ctas), 0)

    def __enter__(self):
        _lib.check(_lib.lib().come_attn_set_cta_limit(self.max_ctas))
        cta_limit.current.value = self.max_ctas
        return self

    def __exit__(self, *exc):
        _lib.check(_lib.lib().come_attn_set_cta_limit(0))
        cta_limit.current.value = 0
        return False


def _unsupported(what: str):
    raise NotImplementedError(f"come_b200 attention: {what} is not supported (forward-only Co-Me inference build)")


def _impl(q, k, v, out_, cu_seqlens_q, cu_seqlens_k, seqused_k, leftpad_k, block_table, alibi_slopes, perkey_bias,
          max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale, zero_tensors, is_causal, window_size_left,
          window_size_right, softcap, return_softmax, gen_, max_seqlen_dev=None):
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("FlashAttention only support fp16 and bf16 data type")
    if k.dtype != q.dtype:
        raise RuntimeError("query and key must have the same dtype")
    if v.dtype != q.dtype:
        raise RuntimeError("query and value must have the same dtype")
    if cu_seqlens_q.dtype != torch.int32:
        raise RuntimeError("cu_seqlens_q must have dtype int32")
    if cu_seqlens_k.dtype != torch.int32:
        raise RuntimeError("cu_seqlens_k must have dtype int32")
    for name, t in (("q", q), ("k", k), ("v", v), ("cu_seqlens_q", cu_seqlens_q), ("cu_seqlens_k", cu_seqlens_k)):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be on CUDA")
    for t in (q, k, v):
        if t.stride(-1) != 1:
            raise RuntimeError("Input tensor must have contiguous last dimension")
    if not cu_seqlens_q.is_contiguous() or not cu_seqlens_k.is_contiguous():
        raise RuntimeError("cu_seqlens must be contiguous")
    if block_table is not None:
        _unsupported("paged KV (block_table)")
    if seqused_k is not None:
        _unsupported("seqused_k")
    if leftpad_k is not None:
        _unsupported("leftpad_k")
    if alibi_slopes is not None:
        _unsupported("alibi_slopes")
    if p_dropout != 0.0:
        _unsupported("dropout")
    if return_softmax:
        raise RuntimeError("return_softmax is only supported when p_dropout > 0.0")
    if is_causal and max_seqlen_q != 1:
        _unsupported("causal masking")
    if (window_size_left >= 0 and window_size_left < max_seqlen_k) or (window_size_right >= 0 and window_size_right < max_seqlen_k):
        _unsupported("sliding-window attention")
    if softcap > 0.0:
        _unsupported("softcap")

    total_q, num_heads, head_size = q.shape
    batch_size = cu_seqlens_q.numel() - 1
    if batch_size <= 0:
        raise RuntimeError("batch size must be positive")
    if head_size > 256:
        raise RuntimeError("FlashAttention forward only supports head dimension at most 256")
    if head_size % 8 != 0:
        raise RuntimeError("query, key, value, and out_ must have a head_size that is a multiple of 8")
    if tuple(k.shape) != (k.shape[0], num_heads, head_size) or tuple(v.shape) != tuple(k.shape):
        if k.shape[1] != num_heads:
            _unsupported("grouped-query attention (num_heads_k != num_heads)")
        raise RuntimeError("k / v must have shape (total_k, num_heads, head_size)")
    total_k = k.shape[0]
    if cu_seqlens_k.numel() != batch_size + 1:
        raise RuntimeError("cu_seqlens_k must have shape (batch_size + 1)")
    same_cu = cu_seqlens_q.data_ptr() == cu_seqlens_k.data_ptr() or (
        total_q == total_k and max_seqlen_q == max_seqlen_k and torch.equal(cu_seqlens_q, cu_seqlens_k))
    if not same_cu:
        _unsupported("cross attention (cu_seqlens_q != cu_seqlens_k)")

    if out_ is not None:
        out = out_
        if out.dtype != q.dtype:
            raise RuntimeError("Output must have the same dtype as inputs")
        if not out.is_cuda:
            raise RuntimeError("out must be on CUDA")
        if out.stride(-1) != 1 or out.stride(1) != head_size:
            raise RuntimeError("Output tensor must have contiguous last dimension")
        if tuple(out.shape) != (total_q, num_heads, head_size):
            raise RuntimeError("out must have shape (total_q, num_heads, head_size)")
    else:
        out = torch.empty((total_q, num_heads, head_size), dtype=q.dtype, device=q.device)
    softmax_lse = torch.empty((num_heads, total_q), dtype=torch.float32, device=q.device)
    p = torch.empty((0,), dtype=q.dtype, device=q.device)
    rng_state = torch.empty((2,), dtype=torch.int64, device=q.device)

    bias = None
    if perkey_bias is not None:
        if perkey_bias.dtype != q.dtype:
            raise RuntimeError(f"perkey_bias dtype must match QKV dtype ({q.dtype}), got {perkey_bias.dtype}")
        if not perkey_bias.is_cuda:
            raise RuntimeError("perkey_bias must be on CUDA")
        if not perkey_bias.is_contiguous():
            raise RuntimeError("perkey_bias must be contiguous")
        if tuple(perkey_bias.shape) != (total_k,):
            raise RuntimeError(f"perkey_bias must have shape (total_k,), got {tuple(perkey_bias.shape)}")
        bias = perkey_bias

    if zero_tensors:
        out.zero_()
        softmax_lse.fill_(float("-inf"))
    if max_seqlen_k <= 0 or total_q == 0:
        out.zero_()
        softmax_lse.fill_(float("inf"))
        return [out, softmax_lse, p, rng_state]

    def head_packed(t):
        # heads must be adjacent (stride head_size); a strided view over a packed qkv buffer qualifies
        return t if t.stride(1) == head_size else t.contiguous()

    q, k, v = head_packed(q), head_packed(k), head_packed(v)
    with torch.cuda.device(q.device):
        if max_seqlen_dev is None:
            _lib.check(_lib.lib().come_attn_varlen_fwd(
                ptr(q), ptr(k), ptr(v), dtype_code(q.dtype), total_q, num_heads, head_size, q.stride(0), k.stride(0),
                v.stride(0), ptr(bias), ptr(cu_seqlens_q), batch_size, int(max_seqlen_q), float(softmax_scale),
                ptr(out), out.stride(0), ptr(softmax_lse), _backend, stream_ptr(q.device)))
        else:  # max_seqlen_q is an upper bound; the exact longest segment is read on the device
            if max_seqlen_dev.dtype != torch.int32 or not max_seqlen_dev.is_cuda or max_seqlen_dev.numel() != 1:
                raise RuntimeError("max_seqlen_dev must be a one-element int32 CUDA tensor")
            _lib.check(_lib.lib().come_attn_varlen_fwd_rows(
                ptr(q), ptr(k), ptr(v), dtype_code(q.dtype), total_q, 0, total_q, num_heads, head_size, q.stride(0),
                k.stride(0), v.stride(0), ptr(bias), ptr(cu_seqlens_q), batch_size, int(max_seqlen_q),
                ptr(max_seqlen_dev), float(softmax_scale), ptr(out), out.stride(0), ptr(softmax_lse), _backend,
                stream_ptr(q.device)))
    return [out, softmax_lse, p, rng_state]


def varlen_fwd(q, k, v, out_, cu_seqlens_q, cu_seqlens_k, seqused_k, leftpad_k, block_table, alibi_slopes,
               max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale, zero_tensors, is_causal, window_size_left,
               window_size_right, softcap, return_softmax, gen_, *, max_seqlen_dev=None):
    """Forward pass (variable length); see ``flash_api.cpp:538-567``.  ``max_seqlen_dev`` (keyword, not in the
    reference): exact longest segment as a one-element int32 device tensor when ``max_seqlen_q`` is only a bound."""
    return _impl(q, k, v, out_, cu_seqlens_q, cu_seqlens_k, seqused_k, leftpad_k, block_table, alibi_slopes, None,
                 max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale, zero_tensors, is_causal, window_size_left,
                 window_size_right, softcap, return_softmax, gen_, max_seqlen_dev)


def varlen_fwd_w_perkey_bias(q, k, v, out_, cu_seqlens_q, cu_seqlens_k, seqused_k, leftpad_k, block_table,
                             alibi_slopes, perkey_bias, max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale,
                             zero_tensors, is_causal, window_size_left, window_size_right, softcap, return_softmax,
                             gen_, *, max_seqlen_dev=None):
    """Forward pass (variable length) with a per-key additive bias; see ``flash_api.cpp:570-599``.
    ``max_seqlen_dev`` as in :func:`varlen_fwd`."""
    return _impl(q, k, v, out_, cu_seqlens_q, cu_seqlens_k, seqused_k, leftpad_k, block_table, alibi_slopes,
                 perkey_bias, max_seqlen_q, max_seqlen_k, p_dropout, softmax_scale, zero_tensors, is_causal,
                 window_size_left, window_size_right, softcap, return_softmax, gen_, max_seqlen_dev)


def varlen_fwd_rows(q_rows, k, v, cu_seqlens, max_seqlen, perkey_bias, softmax_scale, row_begin, out_=None,
                    max_seqlen_dev=None):
    """Attention of a slice of the query rows against all keys / values (no counterpart in the reference: the
    per-GPU piece of global attention sharded by query rows).

    ``q_rows`` ``[rows, H, D]`` holds the global packed rows ``[row_begin, row_begin + rows)``; ``k`` / ``v``
    ``[total, H, D]``, ``perkey_bias`` ``[total]`` or ``None`` and ``cu_seqlens`` describe all packed tokens.
    Returns ``[out [rows, H, D], softmax_lse [H, rows]]``.
    """
    if q_rows.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("FlashAttention only support fp16 and bf16 data type")
    if k.dtype != q_rows.dtype or v.dtype != q_rows.dtype:
        raise RuntimeError("query, key and value must have the same dtype")
    if cu_seqlens.dtype != torch.int32 or not cu_seqlens.is_contiguous():
        raise RuntimeError("cu_seqlens must be a contiguous int32 tensor")
    rows, num_heads, head_size = q_rows.shape
    total = k.shape[0]
    if tuple(k.shape) != (total, num_heads, head_size) or tuple(v.shape) != (total, num_heads, head_size):
        raise RuntimeError("k / v must have shape (total, num_heads, head_size)")
    if row_begin < 0 or row_begin + rows > total:
        raise RuntimeError(f"query rows [{row_begin}, {row_begin + rows}) must lie inside [0, {total})")
    for t in (q_rows, k, v):
        if not t.is_cuda:
            raise RuntimeError("q / k / v must be on CUDA")
        if t.stride(-1) != 1 or t.stride(1) != head_size:
            raise RuntimeError("q / k / v must have adjacent heads and a contiguous last dimension")
    if perkey_bias is not None and (perkey_bias.dtype != q_rows.dtype or tuple(perkey_bias.shape) != (total,)
                                    or not perkey_bias.is_contiguous()):
        raise RuntimeError("perkey_bias must be a contiguous (total,) tensor of the q/k/v dtype")
    out = out_ if out_ is not None else torch.empty((rows, num_heads, head_size), dtype=q_rows.dtype, device=q_rows.device)
    lse = torch.empty((num_heads, rows), dtype=torch.float32, device=q_rows.device)
    with torch.cuda.device(q_rows.device):
        _lib.check(_lib.lib().come_attn_varlen_fwd_rows(
            ptr(q_rows), ptr(k), ptr(v), dtype_code(q_rows.dtype), total, int(row_begin), rows, num_heads, head_size,
            q_rows.stride(0), k.stride(0), v.stride(0), ptr(perkey_bias), ptr(cu_seqlens), cu_seqlens.numel() - 1,
            int(max_seqlen), ptr(max_seqlen_dev), float(softmax_scale), ptr(out), out.stride(0), ptr(lse), _backend,
            stream_ptr(q_rows.device)))
    return [out, lse]


def cross_fwd(q_rows, k, v, perkey_bias, softmax_scale, out_=None):
    """Attention of ``q_rows [rows, H, D]`` to ONE set of keys / values ``k`` / ``v`` ``[kv_rows, H, D]`` that need not
    contain those rows (no counterpart in the reference): the piece of row-sharded global attention that runs on the
    key / value rows gathered from the other GPUs.  ``perkey_bias`` ``[kv_rows]`` or ``None``.
    Returns ``[out [rows, H, D], softmax_lse [H, rows]]``."""
    if q_rows.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("FlashAttention only support fp16 and bf16 data type")
    if k.dtype != q_rows.dtype or v.dtype != q_rows.dtype:
        raise RuntimeError("query, key and value must have the same dtype")
    rows, num_heads, head_size = q_rows.shape
    kv_rows = k.shape[0]
    if tuple(k.shape) != (kv_rows, num_heads, head_size) or tuple(v.shape) != (kv_rows, num_heads, head_size):
        raise RuntimeError("k / v must have shape (kv_rows, num_heads, head_size)")
    if kv_rows == 0 and rows > 0:
        raise RuntimeError("cross attention needs at least one key")
    for t in (q_rows, k, v):
        if not t.is_cuda:
            raise RuntimeError("q / k / v must be on CUDA")
        if t.stride(-1) != 1 or t.stride(1) != head_size:
            raise RuntimeError("q / k / v must have adjacent heads and a contiguous last dimension")
    if perkey_bias is not None and (perkey_bias.dtype != q_rows.dtype or tuple(perkey_bias.shape) != (kv_rows,)
                                    or not perkey_bias.is_contiguous()):
        raise RuntimeError("perkey_bias must be a contiguous (kv_rows,) tensor of the q/k/v dtype")
    out = out_ if out_ is not None else torch.empty((rows, num_heads, head_size), dtype=q_rows.dtype, device=q_rows.device)
    lse = torch.empty((num_heads, rows), dtype=torch.float32, device=q_rows.device)
    with torch.cuda.device(q_rows.device):
        _lib.check(_lib.lib().come_attn_cross_fwd(
            ptr(q_rows), ptr(k), ptr(v), dtype_code(q_rows.dtype), rows, kv_rows, num_heads, head_size, q_rows.stride(0),
            k.stride(0), v.stride(0), ptr(perkey_bias), float(softmax_scale), ptr(out), out.stride(0), ptr(lse), _backend,
            stream_ptr(q_rows.device)))
    return [out, lse]


_ROWS_PER_ITEM = 384  # query rows of a work item of the tensor-core kernel (three 128-row tiles)


def plan_tail_split(rows: int, num_heads: int, kv_rows: int, ctas: int):
    """``(main_rows, key_parts)`` for a one-segment attention launch of ``rows`` query rows on ``ctas`` persistent CTAs.
    The kernel's work items (384 query rows of one head, all keys) are dealt round-robin; when the last round holds only a
    few items, the query blocks behind the full rounds are better run with their keys split ``key_parts`` ways (one short
    round that fills the machine).  ``key_parts == 1``: leave the launch alone (``main_rows == rows``)."""
    blocks = -(-rows // _ROWS_PER_ITEM)
    items = blocks * num_heads
    full = items // max(ctas, 1)
    if ctas <= 0 or full == 0 or items == full * ctas:
        return rows, 1
    main_blocks = (full * ctas) // num_heads
    tail_items = (blocks - main_blocks) * num_heads
    tiles = -(-kv_rows // 64)
    parts = min(64, ctas // max(tail_items, 1), tiles)
    if main_blocks == 0 or parts < 2:
        return rows, 1
    per = -(-tiles // parts)
    parts = -(-tiles // per)  # no empty share
    return (main_blocks * _ROWS_PER_ITEM, parts) if parts >= 2 else (rows, 1)


def cross_fwd_balanced(q_rows, k, v, perkey_bias, softmax_scale, out_=None):
    """:func:`cross_fwd` with the launch shaped by :func:`plan_tail_split`: the query blocks that would make up a nearly
    empty last round are attended with their keys split into shares (``come_attn_cross_fwd_parts``) and merged from the
    shares' log-sum-exps (``come_attn_combine_parts``).  Those rows differ from the one-launch result by the rounding of
    the shares' outputs.  Returns ``[out [rows, H, D], softmax_lse [H, rows]]``."""
    rows, num_heads, head_size = q_rows.shape
    ctas = getattr(cta_limit.current, "value", 0) or torch.cuda.get_device_properties(q_rows.device).multi_processor_count
    # key shares exist in the tensor-core kernel only (head_dim 64, not with the CUDA-core kernel forced)
    main_rows, parts = plan_tail_split(rows, num_heads, k.shape[0], ctas) if (head_size == 64 and _backend != BACKEND_CUDA_CORE) else (rows, 1)
    if parts == 1:
        return cross_fwd(q_rows, k, v, perkey_bias, softmax_scale, out_=out_)
    out = out_ if out_ is not None else torch.empty((rows, num_heads, head_size), dtype=q_rows.dtype, device=q_rows.device)
    if not out.is_contiguous():
        raise RuntimeError("out_ must be contiguous")
    _, lse_main = cross_fwd(q_rows[:main_rows], k, v, perkey_bias, softmax_scale, out_=out[:main_rows])
    tail = q_rows[main_rows:]
    n_tail = rows - main_rows
    out_parts = torch.empty((parts, n_tail, num_heads, head_size), dtype=q_rows.dtype, device=q_rows.device)
    lse_parts = torch.empty((parts, num_heads, n_tail), dtype=torch.float32, device=q_rows.device)
    lse_tail = torch.empty((num_heads, n_tail), dtype=torch.float32, device=q_rows.device)
    with torch.cuda.device(q_rows.device):
        lib, st = _lib.lib(), stream_ptr(q_rows.device)
        rc = lib.come_attn_cross_fwd_parts(
            ptr(tail), ptr(k), ptr(v), dtype_code(q_rows.dtype), n_tail, k.shape[0], num_heads, head_size, tail.stride(0),
            k.stride(0), v.stride(0), ptr(perkey_bias), float(softmax_scale), parts, ptr(out_parts), ptr(lse_parts), _backend, st)
        if rc == _lib.COME_ERR_UNSUPPORTED:  # tensors the tensor-core kernel cannot take (alignment, strides): one more plain launch
            _, lse_tail = cross_fwd(tail, k, v, perkey_bias, softmax_scale, out_=out[main_rows:])
            return [out, torch.cat([lse_main, lse_tail], dim=1)]
        _lib.check(rc)
        _lib.check(lib.come_attn_combine_parts(ptr(out_parts), ptr(lse_parts), parts, dtype_code(q_rows.dtype), n_tail, num_heads,
                                               head_size, ptr(out[main_rows:]), ptr(lse_tail), st))
    return [out, torch.cat([lse_main, lse_tail], dim=1)]


def combine(out_a, lse_a, out_b, lse_b, out_=None, lse_out=None):
    """Merge two attention results of the same query rows over disjoint key sets from their log-sum-exps
    (``come_attn_combine``).  ``out_* [rows, H, D]`` contiguous, ``lse_* [H, rows]`` float32; ``out_`` / ``lse_out`` may be
    one of the inputs.  Returns ``[out, lse]``."""
    rows, num_heads, head_size = out_a.shape
    if out_b.shape != out_a.shape or out_b.dtype != out_a.dtype or out_a.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("combine needs two fp16 / bf16 results of the same shape")
    for t in (lse_a, lse_b):
        if tuple(t.shape) != (num_heads, rows) or t.dtype != torch.float32 or not t.is_contiguous():
            raise RuntimeError("lse must be a contiguous float32 (num_heads, rows) tensor")
    if not out_a.is_contiguous() or not out_b.is_contiguous():
        raise RuntimeError("combine needs contiguous results")
    out = out_ if out_ is not None else torch.empty_like(out_a)
    lse = lse_out if lse_out is not None else torch.empty_like(lse_a)
    with torch.cuda.device(out_a.device):
        _lib.check(_lib.lib().come_attn_combine(ptr(out_a), ptr(lse_a), ptr(out_b), ptr(lse_b), dtype_code(out_a.dtype), rows,
                                                num_heads, head_size, ptr(out), ptr(lse), stream_ptr(out_a.device)))
    return [out, lse]
