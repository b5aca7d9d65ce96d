"""Host-side mirror of the reference's token-merger operator interface, on top of ``libcome_b200.so``.

* :class:`JaggedTokens` -- the packed variable-length container (``src/interface/token_merger.py:11-100``).
* :func:`func_token_merge`, :func:`func_token_split` -- ``src/accelerate/token_merger/co_me.py:152-254``.
* :func:`func_token_merge_2d` -- ``src/accelerate/token_merger/co_me_2d.py:174-211``; here the 2-D window gather
  runs inside the merge kernel (no permuted copy of the tokens) and grids that the windows do not tile exactly
  (37x37 with 3x3 windows) are accepted: uncovered patches are emitted right after the special tokens.
* :class:`MergePlan` -- everything of a merge that depends on the mask only, computed once per ``build_ctx``
  (one device->host read for the packed length) and reused by every merge / split / attention call.
* :func:`select_windows` -- the tensor code of ``build_ctx`` (``co_me_2d.py:268-298``, ``co_me.py:54-73``).
* :class:`CoMe2DTokenMerger`, :class:`CoMeTokenMerger` -- the 2-D and the 1-D ``ITokenMerger`` implementations with the
  reference's method names.

Argument validation raises ``ValueError`` with the reference's messages before anything is launched.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Any, Callable, Optional, Tuple

import torch

from . import _lib, co_me_cuext
from ._torch_util import dtype_code, ptr, require_cuda, stream_ptr

__all__ = [
    "JaggedTokens", "MergePlan", "func_token_merge", "func_token_split", "func_token_merge_2d", "select_windows",
    "CoMe2DTokenMerger", "CoMeTokenMerger",
]


# ---------------------------------------------------------------------------------------------------------
# JaggedTokens
# ---------------------------------------------------------------------------------------------------------
@dataclass
class JaggedTokens:
    """Packed variable-length tokens: ``tokens [1, P, C]``, ``weight [P]`` (tokens represented by each row),
    ``offset [M+1]`` int64 segment boundaries.

    Two optional fields, absent from the reference's container, let a caller that already knows the longest segment
    spare the attention modules their device-to-host read (``flash_attn/__init__.py:33``): ``max_seqlen`` (an upper
    bound on the host) and ``max_seqlen_dev`` (the exact value as a one-element int32 device tensor; it lets a launch
    sized for the bound skip the query blocks no segment reaches).  Both are None unless set.

    ``exchange`` (None unless set, also absent from the reference) marks tokens that are one rank's rows of a segment
    spread over several GPUs: a :class:`come_b200.dist.GlobalExchange`, which the attention modules use to attend these
    rows to the keys / values of all ranks."""
    tokens: torch.Tensor
    weight: torch.Tensor
    offset: torch.Tensor
    max_seqlen: Optional[int] = None
    max_seqlen_dev: Optional[torch.Tensor] = None
    exchange: Optional[Any] = None
    cu_seqlens: Optional[torch.Tensor] = None  # ``offset`` as int32, when the caller keeps it (spares a cast per block)

    def apply(self, func: Callable[[torch.Tensor], torch.Tensor]) -> "JaggedTokens":
        return JaggedTokens(tokens=func(self.tokens), weight=self.weight, offset=self.offset,
                            max_seqlen=self.max_seqlen, max_seqlen_dev=self.max_seqlen_dev, exchange=self.exchange,
                            cu_seqlens=self.cu_seqlens)

    def _on_device_path(self) -> bool:
        """The suffix kernels serve CUDA tensors in the library's layouts; anything else (CPU tensors, other weight or
        offset dtypes) takes the PyTorch indexing below, as in the reference."""
        return (self.tokens.is_cuda and self.weight.is_cuda and self.offset.is_cuda and self.weight.dtype == torch.float32
                and self.offset.dtype == torch.int64 and self.tokens.dtype in (torch.float32, torch.float16, torch.bfloat16))

    def add_suffix(self, suffix: torch.Tensor) -> "JaggedTokens":
        """Append ``T`` dense tokens (weight 1) to each of the ``M`` segments; ``suffix`` is ``(M, T, C)``
        (``src/interface/token_merger.py:23-58``).  CUDA tensors: one kernel (``come_suffix_add``)."""
        M = self.offset.shape[0] - 1
        if suffix.shape[0] != M:
            raise ValueError(f"suffix batch dim ({suffix.shape[0]}) must match segment count ({M})")
        T, Cc = suffix.shape[1], suffix.shape[2]
        P_old = self.tokens.shape[1]
        if self._on_device_path() and suffix.is_cuda and suffix.dtype == self.tokens.dtype and Cc == self.tokens.shape[2]:
            dev = self.tokens.device
            tokens, weight, offset = self.tokens[0].contiguous(), self.weight.contiguous(), self.offset.contiguous()
            suffix = suffix.contiguous()
            new_tokens = torch.empty(1, P_old + M * T, Cc, device=dev, dtype=tokens.dtype)
            new_weight = torch.empty(P_old + M * T, device=dev, dtype=torch.float32)
            new_offset = torch.empty_like(offset)
            with torch.cuda.device(dev):
                _lib.check(_lib.lib().come_suffix_add(ptr(tokens), ptr(weight), ptr(offset), M, P_old, Cc,
                                                      dtype_code(tokens.dtype, "tokens"), ptr(suffix), T, ptr(new_tokens),
                                                      ptr(new_weight), ptr(new_offset), stream_ptr(dev)))
            return JaggedTokens(tokens=new_tokens, weight=new_weight, offset=new_offset)
        dev = self.offset.device
        seg_len = self.offset[1:] - self.offset[:-1]
        seg_id = torch.repeat_interleave(torch.arange(M, device=dev), seg_len, output_size=P_old)
        new_pos = torch.arange(P_old, device=dev) + seg_id * T
        new_offset = self.offset + torch.arange(M + 1, device=dev, dtype=self.offset.dtype) * T
        new_tokens = torch.empty(1, P_old + M * T, Cc, device=self.tokens.device, dtype=self.tokens.dtype)
        new_weight = torch.ones(P_old + M * T, device=self.weight.device, dtype=self.weight.dtype)
        new_tokens[0, new_pos] = self.tokens[0]
        new_weight[new_pos] = self.weight
        tail = (new_offset[1:, None] - T + torch.arange(T, device=dev)[None, :]).reshape(-1)
        new_tokens[0, tail] = suffix.reshape(-1, Cc)
        return JaggedTokens(tokens=new_tokens, weight=new_weight, offset=new_offset)

    def split_suffix(self, count: int) -> Tuple["JaggedTokens", torch.Tensor]:
        """Remove the last ``count`` tokens of every segment (inverse of :meth:`add_suffix`,
        ``src/interface/token_merger.py:60-100``).  CUDA tensors: one kernel (``come_suffix_split``) after the
        reference's check of the segment lengths (a device-to-host read, as there)."""
        M = self.offset.shape[0] - 1
        T, Cc = count, self.tokens.shape[2]
        P_old = self.tokens.shape[1]
        P_new = P_old - M * T
        if P_new < 0:
            raise ValueError(f"Cannot strip {T} tokens from each of {M} segments (total tokens = {P_old})")
        dev = self.offset.device
        orig_offset = self.offset - torch.arange(M + 1, device=dev, dtype=self.offset.dtype) * T
        seg_len = orig_offset[1:] - orig_offset[:-1]
        if (seg_len < 0).any():
            raise ValueError(f"count={T} exceeds the length of at least one segment")
        if self._on_device_path():
            tdev = self.tokens.device
            tokens, weight, offset = self.tokens[0].contiguous(), self.weight.contiguous(), self.offset.contiguous()
            new_tokens = torch.empty(1, P_new, Cc, device=tdev, dtype=tokens.dtype)
            new_weight = torch.empty(P_new, device=tdev, dtype=torch.float32)
            new_offset = torch.empty_like(offset)
            suffix = torch.empty(M, T, Cc, device=tdev, dtype=tokens.dtype)
            with torch.cuda.device(tdev):
                _lib.check(_lib.lib().come_suffix_split(ptr(tokens), ptr(weight), ptr(offset), M, P_old, Cc,
                                                        dtype_code(tokens.dtype, "tokens"), T, ptr(new_tokens),
                                                        ptr(new_weight), ptr(new_offset), ptr(suffix), stream_ptr(tdev)))
            return JaggedTokens(tokens=new_tokens, weight=new_weight, offset=new_offset), suffix
        tail = (self.offset[1:, None] - T + torch.arange(T, device=dev)[None, :]).reshape(-1)
        suffix = self.tokens[0, tail].reshape(M, T, Cc)
        seg_id = torch.repeat_interleave(torch.arange(M, device=dev), seg_len, output_size=P_new)
        keep = torch.arange(P_new, device=dev) + seg_id * T
        return JaggedTokens(tokens=self.tokens[0, keep].unsqueeze(0), weight=self.weight[keep],
                            offset=orig_offset), suffix


# ---------------------------------------------------------------------------------------------------------
# validation (messages follow the reference so its tests read the same)
# ---------------------------------------------------------------------------------------------------------
def _validate_token_merge_args(tokens, start_index, group_size, merge_mask) -> None:
    if start_index < 0:
        raise ValueError(f"start_index must be >= 0, got {start_index}")
    if group_size <= 0:
        raise ValueError(f"group_size must be > 0, got {group_size}")
    if merge_mask.dtype != torch.bool:
        raise ValueError(f"merge_mask must be of dtype torch.bool, got {merge_mask.dtype}")
    B, N, _C = tokens.shape
    _Bm, M = merge_mask.shape
    if _Bm != B:
        raise ValueError(f"merge_mask batch ({_Bm}) must match tokens batch ({B})")
    if N != start_index + M * group_size:
        raise ValueError(
            f"Expected N = start_index + M * group_size = {start_index} + {M} * {group_size} = "
            f"{start_index + M * group_size}, got N = {N}")


def _validate_token_merge_2d_args(tokens, start_index, group_h, group_w, H, W, merge_mask, ragged) -> None:
    if start_index < 0:
        raise ValueError(f"start_index must be >= 0, got {start_index}")
    if group_h <= 0 or group_w <= 0:
        raise ValueError(f"group_h and group_w must be > 0, got ({group_h}, {group_w})")
    if not ragged:
        if H % group_h != 0:
            raise ValueError(f"H ({H}) must be divisible by group_h ({group_h})")
        if W % group_w != 0:
            raise ValueError(f"W ({W}) must be divisible by group_w ({group_w})")
    if merge_mask.dtype != torch.bool:
        raise ValueError(f"merge_mask must be of dtype torch.bool, got {merge_mask.dtype}")
    B, N, _C = tokens.shape
    _Bm, M = merge_mask.shape
    M_expected = (H // group_h) * (W // group_w)
    if _Bm != B:
        raise ValueError(f"merge_mask batch ({_Bm}) must match tokens batch ({B})")
    if N != start_index + H * W:
        raise ValueError(f"Expected N = start_index + H * W = {start_index} + {H * W} = {start_index + H * W}, got N = {N}")
    if M != M_expected:
        raise ValueError(f"Expected M = (H // group_h) * (W // group_w) = {M_expected}, got M = {M}")


# ---------------------------------------------------------------------------------------------------------
# MergePlan
# ---------------------------------------------------------------------------------------------------------
class MergePlan:
    """Index plan of a merge mask: packed offsets, ``rev_id``, ``weight``, per-key attention bias and the
    longest segment, built by one pair of small kernels and ONE device->host read.

    The reference recomputes all of this inside every ``merge`` call (114 times per forward in its direct
    mode); with a plan, ``merge`` and ``split`` are pure data movement and attention needs no
    ``max_seqlen`` read-back.
    """

    def __init__(self, merge_mask: torch.Tensor, layout: _lib.Layout):
        require_cuda(merge_mask, "merge_mask")
        if merge_mask.dtype != torch.bool or merge_mask.dim() != 2:
            raise ValueError(f"merge_mask must be a [frames, M] tensor of dtype torch.bool, got {merge_mask.dtype}")
        n_groups, n_tok, prefix = C.c_int64(), C.c_int64(), C.c_int64()
        _lib.check(_lib.lib().come_layout_info(C.byref(layout), C.byref(n_groups), C.byref(n_tok), C.byref(prefix)))
        if merge_mask.shape[1] != n_groups.value:
            raise ValueError(f"Expected M = {n_groups.value}, got M = {merge_mask.shape[1]}")
        self.layout = layout
        self.frames = int(merge_mask.shape[0])
        self.tokens_per_frame = int(n_tok.value)
        self.prefix_len = int(prefix.value)
        self.mask = merge_mask.contiguous()
        self._mask_u8 = self.mask.view(torch.uint8)
        self.group_prefix, self.offsets_i32, self.rev_id, weight_full, seg_max = co_me_cuext.merge_plan_raw(
            self._mask_u8, layout, self.tokens_per_frame)
        self.seg_max = seg_max  # [1] int32 on the device: the longest frame after merging
        if self.frames > 0:
            host = torch.stack([self.offsets_i32[-1], seg_max[0]]).tolist()  # the single synchronising read
            self.total, self.max_seqlen = int(host[0]), int(host[1])
        else:
            self.total, self.max_seqlen = 0, 0
        self.weight = weight_full[: self.total]
        self.offset = self.offsets_i32.long()
        self._bias = {}
        self._positions = None

    def load(self, other: "MergePlan", keep_derived: bool = False) -> None:
        """Overwrite this plan's device tensors with ``other``'s, keeping their addresses (a captured CUDA graph that
        reads this plan then sees the new scene).  Both plans must pack to the same number of rows.  The cached derived
        tensors (positions, bias) are dropped unless ``keep_derived``: a captured graph that recomputes them in place
        on every replay keeps them."""
        if (other.frames, other.tokens_per_frame, other.total) != (self.frames, self.tokens_per_frame, self.total):
            raise ValueError(f"plans differ in shape: {other.frames} frames / {other.total} rows against "
                             f"{self.frames} / {self.total}")
        for name in ("mask", "group_prefix", "offsets_i32", "rev_id", "weight", "offset", "seg_max"):
            getattr(self, name).copy_(getattr(other, name))
        self.max_seqlen = other.max_seqlen
        if not keep_derived:
            self._bias, self._positions = {}, None

    # -- derived, cached ---------------------------------------------------------------------------------
    def perkey_bias(self, dtype: torch.dtype) -> torch.Tensor:
        """``log(weight)`` in the run dtype (``src/accelerate/vggt/module/bias_attention.py:120``)."""
        if dtype not in self._bias:
            self._bias[dtype] = self.weight.log().to(dtype)
        return self._bias[dtype]

    def cu_seqlens(self, frames_per_segment: int = 1) -> torch.Tensor:
        """int32 segment boundaries; ``frames_per_segment = S`` concatenates the frames of a scene into one
        segment (global attention, ``src/accelerate/vggt/fused.py:136,149``)."""
        return self.offsets_i32 if frames_per_segment == 1 else self.offsets_i32[::frames_per_segment].contiguous()

    def positions(self) -> torch.Tensor:
        """``[P, 2]`` int64 (y, x) positions of the packed rows, computed from the plan alone
        (``come_packed_positions``): what the reference obtains by merging the bfloat16 position tensor and
        truncating it (``src/accelerate/vggt/fused.py:113-129``).  2-D layouts only."""
        if self._positions is None:
            pos = torch.empty(self.total, 2, dtype=torch.int64, device=self.mask.device)
            with torch.cuda.device(self.mask.device):
                _lib.check(_lib.lib().come_packed_positions(ptr(self._mask_u8), ptr(self.rev_id), self.frames,
                                                            C.byref(self.layout), ptr(pos),
                                                            stream_ptr(self.mask.device)))
            self._positions = pos
        return self._positions

    # -- data movement -----------------------------------------------------------------------------------
    def merge(self, tokens: torch.Tensor) -> torch.Tensor:
        """``tokens [frames, N, C]`` -> packed ``[P, C]``."""
        require_cuda(tokens, "tokens")
        if tokens.dim() != 3 or tokens.shape[0] != self.frames or tokens.shape[1] != self.tokens_per_frame:
            raise ValueError(f"Expected tokens [{self.frames}, {self.tokens_per_frame}, C], got {tuple(tokens.shape)}")
        tokens = tokens.contiguous()
        out = torch.empty((self.total, tokens.shape[2]), dtype=tokens.dtype, device=tokens.device)
        with torch.cuda.device(tokens.device):
            _lib.check(_lib.lib().come_merge(ptr(tokens), dtype_code(tokens.dtype, "tokens"), self.frames,
                                             tokens.shape[2], C.byref(self.layout), ptr(self._mask_u8),
                                             ptr(self.group_prefix), ptr(self.offsets_i32), ptr(out),
                                             stream_ptr(tokens.device)))
        return out

    def merge_layernorm(self, tokens: torch.Tensor, norm: torch.nn.LayerNorm) -> torch.Tensor:
        """``merge(norm(tokens))`` in one pass over the dense tokens (``come_merge_layernorm``): the block's ``norm1``
        followed by the merge of the per-layer mode (``src/thirdparty/vggt/layers/block.py:73``,
        ``src/accelerate/vggt/direct.py:97-101``).  ``tokens [frames, N, C]`` -> packed ``[P, C]``."""
        require_cuda(tokens, "tokens")
        if tokens.dim() != 3 or tokens.shape[0] != self.frames or tokens.shape[1] != self.tokens_per_frame:
            raise ValueError(f"Expected tokens [{self.frames}, {self.tokens_per_frame}, C], got {tuple(tokens.shape)}")
        Cc = tokens.shape[2]
        if not isinstance(norm, torch.nn.LayerNorm) or tuple(norm.normalized_shape) != (Cc,):
            raise NotImplementedError("merge_layernorm needs an nn.LayerNorm over the channel dimension")
        tokens = tokens.contiguous()
        dev, dt = tokens.device, tokens.dtype
        w = (norm.weight if norm.weight is not None else torch.ones(Cc, device=dev)).detach().to(device=dev, dtype=dt).contiguous()
        b = (norm.bias if norm.bias is not None else torch.zeros(Cc, device=dev)).detach().to(device=dev, dtype=dt).contiguous()
        out = torch.empty((self.total, Cc), dtype=dt, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().come_merge_layernorm(ptr(tokens), dtype_code(dt, "tokens"), self.frames, Cc,
                                                       C.byref(self.layout), ptr(w), ptr(b), float(norm.eps),
                                                       ptr(self._mask_u8), ptr(self.group_prefix), ptr(self.offsets_i32),
                                                       ptr(out), stream_ptr(dev)))
        return out

    def split(self, merged: torch.Tensor) -> torch.Tensor:
        """packed ``[P, C]`` -> ``[frames * N, C]``."""
        return co_me_cuext.co_me_token_split_cuda(merged, self.rev_id, merged.shape[-1])

    def split_add(self, merged: torch.Tensor, residual: torch.Tensor, scale: Optional[torch.Tensor] = None,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``residual + scale * split(merged)`` in one pass (``come_unmerge_residual``): the unmerge, the LayerScale
        and the residual add that close an attention block (``x = x + ls1(attn(norm1(x)))``,
        ``src/thirdparty/vggt/layers/block.py:73,90``).  ``residual`` is ``[frames * N, C]`` (any leading shape with that
        many rows), ``scale`` ``[C]`` or None; ``out`` may be ``residual`` itself."""
        require_cuda(merged, "merged")
        require_cuda(residual, "residual")
        rows = self.frames * self.tokens_per_frame
        Cc = merged.shape[-1]
        if merged.dim() != 2 or merged.shape[0] != self.total:
            raise ValueError(f"Expected merged [{self.total}, C], got {tuple(merged.shape)}")
        if residual.numel() != rows * Cc or residual.dtype != merged.dtype:
            raise ValueError(f"Expected residual with {rows} x {Cc} elements of {merged.dtype}, got {tuple(residual.shape)} {residual.dtype}")
        if scale is not None and (scale.shape != (Cc,) or scale.dtype != merged.dtype):
            raise ValueError(f"Expected scale [{Cc}] of {merged.dtype}")
        merged, residual = merged.contiguous(), residual.contiguous()
        if out is None:
            out = torch.empty_like(residual)
        elif out.shape != residual.shape or out.dtype != residual.dtype or not out.is_contiguous():
            raise ValueError("out must be contiguous and match residual")
        with torch.cuda.device(merged.device):
            _lib.check(_lib.lib().come_unmerge_residual(ptr(merged), ptr(self.rev_id), rows, Cc,
                                                        dtype_code(merged.dtype, "merged"), ptr(residual),
                                                        ptr(None if scale is None else scale.contiguous()), ptr(out),
                                                        stream_ptr(merged.device)))
        return out

    def split_concat(self, *merged: torch.Tensor) -> torch.Tensor:
        """Unmerge several packed ``[P, C_k]`` tensors side by side into one ``[frames * N, sum(C_k)]`` tensor:
        the ``torch.cat((split(frame_tokens), split(global_tokens)), dim=-1)`` of a retained layer
        (``src/accelerate/vggt/fused.py:157-167``) without materialising the separate splits."""
        if not merged:
            raise ValueError("split_concat needs at least one tensor")
        first = merged[0]
        for m in merged:
            require_cuda(m, "merged")
            if m.dim() != 2 or m.shape[0] != self.total or m.dtype != first.dtype or m.device != first.device:
                raise ValueError(f"Expected [{self.total}, C] tensors of one dtype on one device, got {tuple(m.shape)} {m.dtype}")
        width = sum(int(m.shape[1]) for m in merged)
        rows = self.frames * self.tokens_per_frame
        out = torch.empty((rows, width), dtype=first.dtype, device=first.device)
        code = dtype_code(first.dtype, "merged")
        col = 0
        with torch.cuda.device(first.device):
            for m in merged:
                m = m.contiguous()
                dst = out.data_ptr() + col * out.element_size()
                _lib.check(_lib.lib().come_unmerge_strided(ptr(m), ptr(self.rev_id), rows, m.shape[1], code, dst, width,
                                                           stream_ptr(first.device)))
                col += int(m.shape[1])
        return out

    def jagged(self, tokens: torch.Tensor) -> JaggedTokens:
        return JaggedTokens(tokens=self.merge(tokens).unsqueeze(0), weight=self.weight, offset=self.offset)


# ---------------------------------------------------------------------------------------------------------
# functional API
# ---------------------------------------------------------------------------------------------------------
def func_token_merge(tokens: torch.Tensor, start_index: int, group_size: int, merge_mask: torch.Tensor):
    """Merge token groups according to ``merge_mask``.

    Args:
        tokens:      ``[B, N, C]`` CUDA tensor.
        start_index: number of leading special tokens excluded from merging.
        group_size:  ``G`` tokens per merge group.
        merge_mask:  ``[B, M]`` bool; ``True`` merges the group into its mean, ``False`` keeps ``G`` tokens.

    Returns:
        ``(JaggedTokens, rev_id)``; ``rev_id[B*N]`` maps every original token to its packed row.
    """
    _validate_token_merge_args(tokens, start_index, group_size, merge_mask)
    out_flat, offsets, rev_id, weight = co_me_cuext.co_me_token_merge_cuda(tokens.contiguous(), start_index, group_size,
                                                                         merge_mask.contiguous())
    return JaggedTokens(tokens=out_flat.unsqueeze(0), weight=weight, offset=offsets.long()), rev_id


def func_token_split(tokens: JaggedTokens, rev_id: torch.Tensor, bsnc_shape: Tuple[int, int, int, int]) -> torch.Tensor:
    """Inverse of :func:`func_token_merge`: gather the packed rows back to ``[B*S, N, C]``."""
    B, S, N, Cc = bsnc_shape
    flat = tokens.tokens.squeeze(0)
    restored = co_me_cuext.co_me_token_split_cuda(flat.contiguous(), rev_id.contiguous(), Cc)
    return restored.reshape(B * S, N, Cc)


def func_token_merge_2d(tokens: torch.Tensor, start_index: int, group_h: int, group_w: int, H: int, W: int,
                        merge_mask: torch.Tensor, allow_ragged: bool = False):
    """Merge ``group_h x group_w`` windows of a row-major ``H x W`` patch grid (window order = raster order).

    Same results as the reference's rearrange-then-1-D path, produced by one gather kernel.  With
    ``allow_ragged`` the grid need not be a multiple of the window: windows tile the top-left part and the
    uncovered patches follow the special tokens, never merged.
    """
    _validate_token_merge_2d_args(tokens, start_index, group_h, group_w, H, W, merge_mask, allow_ragged)
    plan = MergePlan(merge_mask, _lib.Layout.two_d(start_index, H, W, group_h, group_w))
    return plan.jagged(tokens), plan.rev_id


_SELECT_MODES = {"pairwise-rank": _lib.COME_SELECT_RANK, "abs_mse": _lib.COME_SELECT_ABS, "mse": _lib.COME_SELECT_ZSCORE}


def select_windows(confidence: torch.Tensor, B: int, S: int, H: int, W: int, group_h: int, group_w: int,
                   threshold, mode: str = "pairwise-rank", scope: str = "batch") -> torch.Tensor:
    """Per-patch confidence ``[B, S*H*W]`` -> bool merge mask ``[B*S, M]``.

    ``mode``: ``"pairwise-rank"`` (``mean < quantile(mean, threshold)``), ``"abs_mse"`` (``mean < threshold``) or
    ``"mse"`` (the confidences of a batch element are z-normalised, ``(x - mean) / (std + 1e-3)``, before the window
    mean is compared with the threshold); ``scope``: ``"batch"`` ranks all windows of a batch element together (2-D
    merger class), ``"frame"`` ranks per frame (1-D merger class); only the ranking mode looks at it.
    """
    require_cuda(confidence, "confidence")
    if mode not in _SELECT_MODES:
        raise ValueError(f"unknown confidence mode {mode!r}")
    if scope not in ("batch", "frame"):
        raise ValueError(f"unknown scope {scope!r}")
    ratios = threshold if isinstance(threshold, torch.Tensor) else None  # one quantile level per batch element / frame
    if ratios is not None:
        if mode != "pairwise-rank":
            raise ValueError("per-group thresholds need the ranking mode")
        groups = B if scope == "batch" else B * S
        if ratios.numel() != groups or ratios.dtype != torch.float32 or not ratios.is_cuda:
            raise ValueError(f"Expected {groups} float32 CUDA ratios, got {tuple(ratios.shape)} {ratios.dtype}")
    elif mode == "pairwise-rank" and not (0.0 <= threshold <= 1.0):
        raise ValueError(f"Ranking mode requires threshold in [0, 1], got {threshold}")
    if confidence.numel() != B * S * H * W:
        raise ValueError(f"Expected {B * S * H * W} confidences, got {confidence.numel()}")
    conf = confidence.contiguous()
    M = (H // group_h) * (W // group_w)
    mask = torch.empty((B * S, M), dtype=torch.bool, device=conf.device)
    if ratios is not None:
        ratios = ratios.contiguous()
        with torch.cuda.device(conf.device):
            _lib.check(_lib.lib().come_select_windows_ratios(
                ptr(conf), dtype_code(conf.dtype, "confidence"), B, S, H, W, group_h, group_w, ptr(ratios),
                _lib.COME_SCOPE_BATCH if scope == "batch" else _lib.COME_SCOPE_FRAME, ptr(mask), stream_ptr(conf.device)))
        return mask
    with torch.cuda.device(conf.device):
        _lib.check(_lib.lib().come_select_windows(
            ptr(conf), dtype_code(conf.dtype, "confidence"), B, S, H, W, group_h, group_w, float(threshold),
            _SELECT_MODES[mode],
            _lib.COME_SCOPE_BATCH if scope == "batch" else _lib.COME_SCOPE_FRAME, ptr(mask), stream_ptr(conf.device)))
    return mask


# ---------------------------------------------------------------------------------------------------------
# ITokenMerger-style classes
# ---------------------------------------------------------------------------------------------------------
def _nvtx_range(name: str):
    """NVTX range on CUDA builds (the reference brackets its predictor the same way), a no-op context otherwise."""
    import contextlib
    try:
        return torch.cuda.nvtx.range(name)
    except Exception:  # noqa: BLE001  (no NVTX in this build of PyTorch)
        return contextlib.nullcontext()


class CoMe2DTokenMerger:
    """2-D Co-Me merger with the reference's ``ITokenMerger`` method names
    (``src/interface/token_merger.py:102-116``, ``src/accelerate/token_merger/co_me_2d.py:214-352``).

    ``predictor(feature_bshwc_bf16, BPHWC=(B, S, H, W, C)) -> confidence [B, S*H*W, 1]`` is any callable (the
    reference loads a distilled ``GlobalAttentionConfidence``; a seeded MLP head serves the synthetic
    benchmark configurations).  ``build_ctx`` returns ``(mask, (B, S, C, H, W), plan)``: the first two entries
    are the reference's context, the third is the cached :class:`MergePlan`.
    """

    def __init__(self, start_idx: int, group_h: int, group_w: int, threshold: float, predictor: Callable[..., torch.Tensor],
                 conf_mode: str = "pairwise-rank", allow_ragged: bool = True):
        self.start_idx = start_idx
        self.group_h = group_h
        self.group_w = group_w
        self.threshold = threshold
        self.predictor = predictor
        self.conf_mode = conf_mode
        self.allow_ragged = allow_ragged

    def build_ctx(self, feature: torch.Tensor) -> Any:
        B, S, Cc, H, W = feature.shape
        if not self.allow_ragged:
            if H % self.group_h != 0:
                raise ValueError(f"H ({H}) must be divisible by group_h ({self.group_h})")
            if W % self.group_w != 0:
                raise ValueError(f"W ({W}) must be divisible by group_w ({self.group_w})")
        with _nvtx_range("confidence_predictor"):  # the range name of the reference (co_me_2d.py:264)
            confidence = self.predictor(feature.permute(0, 1, 3, 4, 2).bfloat16(), BPHWC=(B, S, H, W, Cc)).squeeze(-1)
        mask = select_windows(confidence, B, S, H, W, self.group_h, self.group_w, self.threshold, self.conf_mode, "batch")
        plan = MergePlan(mask, _lib.Layout.two_d(self.start_idx, H, W, self.group_h, self.group_w))
        return (mask, (B, S, Cc, H, W), plan)

    def _plan_for(self, ctx, start_index: Optional[int]) -> MergePlan:
        mask, (B, S, Cc, H, W), plan = ctx
        if start_index is None or start_index == self.start_idx:
            return plan
        return MergePlan(mask, _lib.Layout.two_d(start_index, H, W, self.group_h, self.group_w))

    def merge(self, ctx, tokens: torch.Tensor, stub: Any = None, *, start_index: Optional[int] = None):
        plan = self._plan_for(ctx, start_index)
        return plan.jagged(tokens.flatten(0, 1)), (plan.rev_id, tokens.shape)

    def split(self, ctx, stub: Any, tokens: JaggedTokens) -> torch.Tensor:
        rev_id, shape_bsnc = stub
        B, S, N, Cc = shape_bsnc
        return func_token_split(tokens, rev_id, shape_bsnc).view(B, S, N, Cc)

    def build_infer_mask(self, ctx) -> torch.Tensor:
        mask, (B, S, _, H, W), _plan = ctx
        Mh, Mw = H // self.group_h, W // self.group_w
        m = mask.reshape(B * S, Mh, 1, Mw, 1).expand(-1, -1, self.group_h, -1, self.group_w)
        full = torch.zeros((B * S, H, W), dtype=torch.bool, device=mask.device)
        full[:, : Mh * self.group_h, : Mw * self.group_w] = m.reshape(B * S, Mh * self.group_h, Mw * self.group_w)
        return full.reshape(B, S, H, W)


class CoMeTokenMerger:
    """1-D Co-Me merger (``src/accelerate/token_merger/co_me.py:21-105``): groups of ``group_size`` CONSECUTIVE patch
    tokens behind ``start_idx`` special tokens, the ranking threshold taken per frame.  Same ``ITokenMerger`` method
    names and context layout as the reference: ``build_ctx`` returns ``(mask, (B, S, C, H, W), plan)`` -- the first two
    entries are the reference's context, the third the cached :class:`MergePlan`.

    ``predictor(feature_bshwc_bf16, BPHWC=(B, S, H, W, C)) -> confidence [B, S*H*W, 1]``.
    """

    def __init__(self, start_idx: int, group_size: int, threshold: float, predictor: Callable[..., torch.Tensor],
                 conf_mode: str = "pairwise-rank"):
        self.start_idx = start_idx
        self.group_size = group_size
        self.threshold = threshold
        self.predictor = predictor
        self.conf_mode = conf_mode

    def build_ctx(self, feature: torch.Tensor) -> Any:
        B, S, Cc, H, W = feature.shape
        if (H * W) % self.group_size != 0:
            raise ValueError(f"H * W ({H * W}) must be divisible by group_size ({self.group_size})")
        with _nvtx_range("confidence_predictor"):
            confidence = self.predictor(feature.permute(0, 1, 3, 4, 2).bfloat16(), BPHWC=(B, S, H, W, Cc)).squeeze(-1)
        # consecutive groups of a frame = 1 x group_size windows of a (H*W / group_size) x group_size grid
        M = (H * W) // self.group_size
        mask = select_windows(confidence, B, S, M, self.group_size, 1, self.group_size, self.threshold, self.conf_mode, "frame")
        plan = MergePlan(mask, _lib.Layout.one_d(self.start_idx, self.group_size, M))
        return (mask, (B, S, Cc, H, W), plan)

    def _plan_for(self, ctx, start_index: Optional[int]) -> MergePlan:
        mask, _shape, plan = ctx
        if start_index is None or start_index == self.start_idx:
            return plan
        return MergePlan(mask, _lib.Layout.one_d(start_index, self.group_size, mask.shape[1]))

    def merge(self, ctx, tokens: torch.Tensor, stub: Any = None, *, start_index: Optional[int] = None):
        """``tokens [B, S, N, C]`` -> ``(JaggedTokens, (rev_id, tokens.shape))``; ``stub`` is accepted and ignored, as in
        the reference (``co_me.py:88-93``)."""
        plan = self._plan_for(ctx, start_index)
        return plan.jagged(tokens.flatten(0, 1)), (plan.rev_id, tokens.shape)

    def split(self, ctx, stub: Any, tokens: JaggedTokens) -> torch.Tensor:
        rev_id, shape_bsnc = stub
        B, S, N, Cc = shape_bsnc
        return func_token_split(tokens, rev_id, shape_bsnc).view(B, S, N, Cc)

    def build_infer_mask(self, ctx) -> torch.Tensor:
        """Per-patch bool mask ``[B, S, H, W]`` of the merged groups (``co_me.py:101-105``)."""
        mask, (B, S, _, H, W), _plan = ctx
        return mask.unsqueeze(-1).expand(-1, -1, self.group_size).reshape(B, S, H, W)
