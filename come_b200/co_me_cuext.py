"""Stand-in for the reference's compiled ``co_me_cuext`` module (pybind surface
``src/cuda_extension/co_me/src/binding.cpp:33-51``), backed by ``libcome_b200.so``.

``co_me_token_merge_cuda`` and ``co_me_token_split_cuda`` keep the reference's signatures, return types
and error behaviour (``RuntimeError`` where the reference's ``TORCH_CHECK`` fires,
``src/cuda_extension/co_me/src/kernel_token_merge.cu:246-261,360-363``).  Unlike the reference they launch on
the caller's current stream of the tensors' device.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._torch_util import dtype_code, ptr, require_cuda, stream_ptr

__all__ = ["co_me_token_merge_cuda", "co_me_token_split_cuda", "merge_plan_raw"]


def merge_plan_raw(mask_u8: torch.Tensor, layout: _lib.Layout, tokens_per_frame: int):
    """Run the index plan of a merge.  Returns device tensors
    ``(group_prefix i32 [F,M], offsets i32 [F+1], rev_id i64 [F*N], weight f32 [F*N] (first P valid), seg_max i32 [1])``.
    """
    frames, M = mask_u8.shape
    dev = mask_u8.device
    group_prefix = torch.empty((frames, M), dtype=torch.int32, device=dev)
    offsets = torch.empty((frames + 1,), dtype=torch.int32, device=dev)
    rev = torch.empty((frames * tokens_per_frame,), dtype=torch.int64, device=dev)
    weight = torch.empty((max(frames * tokens_per_frame, 1),), dtype=torch.float32, device=dev)
    seg_max = torch.empty((1,), dtype=torch.int32, device=dev)
    ws_bytes = _lib.lib().come_merge_plan_workspace_bytes(frames)
    ws = torch.empty((ws_bytes,), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().come_merge_plan(ptr(mask_u8), frames, C.byref(layout), ptr(group_prefix), ptr(offsets),
                                              ptr(rev), ptr(weight), ptr(seg_max), ptr(ws), ws_bytes, stream_ptr(dev)))
    return group_prefix, offsets, rev, weight, seg_max


def co_me_token_merge_cuda(tokens: torch.Tensor, start_index: int, group_size: int, merge_mask: torch.Tensor):
    """Fused token merge: scan + scatter + rev_id.

    Args:
        tokens: ``[B, N, C]`` float tensor on CUDA (float32 / float16 / bfloat16).
        start_index: number of special prefix tokens per sample.
        group_size: ``G``, tokens per merge group.
        merge_mask: ``[B, M]`` bool tensor on CUDA.

    Returns:
        ``(out_flat [P, C], offsets [B+1] int32, rev_id [B*N] int64, weight [P] float32)``.
    """
    require_cuda(tokens, "tokens")
    require_cuda(merge_mask, "merge_mask")
    if tokens.dim() != 3:
        raise RuntimeError("tokens must be [B, N, C]")
    if merge_mask.dim() != 2:
        raise RuntimeError("merge_mask must be [B, M]")
    tokens_c = tokens.contiguous()
    mask_c = merge_mask.to(torch.bool).contiguous()
    B, N, Cc = tokens_c.shape
    M = mask_c.shape[1]
    if mask_c.shape[0] != B:
        raise RuntimeError("merge_mask batch != tokens batch")
    if N != start_index + M * group_size:
        raise RuntimeError("N != start_index + M * group_size")
    code = dtype_code(tokens_c.dtype, "tokens")
    layout = _lib.Layout.one_d(int(start_index), int(group_size), int(M))
    mask_u8 = mask_c.view(torch.uint8)
    group_prefix, offsets, rev, weight, _ = merge_plan_raw(mask_u8, layout, N)
    # The packed length decides the output shape, so it has to reach the host here (the reference reads
    # mask.sum() at the same point, kernel_token_merge.cu:265).
    P = int(offsets[-1].item()) if B > 0 else 0
    out = torch.empty((P, Cc), dtype=tokens_c.dtype, device=tokens_c.device)
    with torch.cuda.device(tokens_c.device):
        _lib.check(_lib.lib().come_merge(ptr(tokens_c), code, B, Cc, C.byref(layout), ptr(mask_u8), ptr(group_prefix),
                                         ptr(offsets), ptr(out), stream_ptr(tokens_c.device)))
    return out, offsets, rev, weight[:P]


def co_me_token_split_cuda(merged_flat: torch.Tensor, rev_id: torch.Tensor, C_: int) -> torch.Tensor:
    """Token split (inverse of merge): ``out[i] = merged_flat[rev_id[i]]``; returns ``[total, C]``."""
    require_cuda(merged_flat, "merged_flat")
    require_cuda(rev_id, "rev_id")
    if merged_flat.dim() != 2:
        raise RuntimeError("merged_flat must be [P, C]")
    if merged_flat.shape[1] != C_:
        raise RuntimeError("C mismatch")
    if rev_id.dtype != torch.int64:
        raise RuntimeError("rev_id must be int64")
    merged_c = merged_flat.contiguous()
    rev_c = rev_id.contiguous()
    total = rev_c.numel()
    code = dtype_code(merged_c.dtype, "merged_flat")
    out = torch.empty((total, C_), dtype=merged_c.dtype, device=merged_c.device)
    with torch.cuda.device(merged_c.device):
        _lib.check(_lib.lib().come_unmerge(ptr(merged_c), ptr(rev_c), total, C_, code, ptr(out),
                                           stream_ptr(merged_c.device)))
    return out
