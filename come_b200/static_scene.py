"""A whole scene of the Co-Me operator chain as ONE CUDA graph, with no device->host read anywhere.

The reference reads the packed length back to the host inside every merge (``kernel_token_merge.cu:265``) and the
longest segment inside every attention call (``flash_attn/__init__.py:33``), because its output shapes depend on
them.  Here every buffer is allocated once for the worst case (nothing merged: ``frames * N`` packed rows) and every
kernel is launched for the worst case too: kernels read the real sizes (``offsets``, ``cu_seqlens``) from device
memory and the surplus CTAs exit at once.  The launch sequence therefore does not depend on the mask, is captured
once, and is replayed for every scene: selection -> plan -> per layer (merge, biased attention, unmerge).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from . import _lib
from ._torch_util import dtype_code, ptr, stream_ptr

__all__ = ["StaticScene"]


class StaticScene:
    """Fixed-shape scene runner: ``run(x, confidence, qkv)`` copies the inputs into its static buffers, replays the
    captured graph and returns the static output ``[frames, N, C]`` (valid until the next ``run``)."""

    def __init__(self, frames: int, channels: int = 1024, start_index: int = 5, grid_h: int = 37, grid_w: int = 37,
                 group_h: int = 3, group_w: int = 3, threshold: float = 0.5, num_heads: int = 16, head_dim: int = 64,
                 layer_kinds: Optional[Sequence[str]] = None, scope: str = "frame", dtype: torch.dtype = torch.bfloat16,
                 device: Optional[torch.device] = None, frames_per_scene: Optional[int] = None,
                 per_frame_ratios: bool = False):
        """``frames`` frames form ``frames / frames_per_scene`` independent scenes (default: one scene): frame layers
        attend inside a frame, global layers inside a scene.  With ``per_frame_ratios`` the merge ratio of every frame
        is read from the static buffer ``ratios [frames]`` (float32) instead of the single ``threshold``."""
        if num_heads * head_dim != channels:
            raise ValueError("channels must equal num_heads * head_dim (the attention output is unmerged as tokens)")
        self.dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.frames, self.C, self.H, self.D = frames, channels, num_heads, head_dim
        self.fps = frames if frames_per_scene is None else int(frames_per_scene)
        if self.fps <= 0 or frames % self.fps != 0:
            raise ValueError("frames must be a multiple of frames_per_scene")
        self.scenes = frames // self.fps
        if per_frame_ratios and scope != "frame":
            raise ValueError("per-frame ratios need scope='frame'")
        self.per_frame_ratios = per_frame_ratios
        self.grid = (grid_h, grid_w, group_h, group_w)
        self.threshold, self.scope, self.dtype = float(threshold), scope, dtype
        self.scale = head_dim ** -0.5
        self.layer_kinds: List[str] = list(layer_kinds) if layer_kinds is not None else ["frame", "global"] * 24
        self.layout = _lib.Layout.two_d(start_index, grid_h, grid_w, group_h, group_w)
        n_groups, n_tok, prefix = C.c_int64(), C.c_int64(), C.c_int64()
        _lib.check(_lib.lib().come_layout_info(C.byref(self.layout), C.byref(n_groups), C.byref(n_tok), C.byref(prefix)))
        self.M, self.N = int(n_groups.value), int(n_tok.value)
        rows = frames * self.N  # worst case: nothing merged
        self.rows_max = rows
        d, dt = self.dev, dtype
        e = torch.empty
        # inputs
        self.x = e((frames, self.N, channels), dtype=dt, device=d)
        self.conf = e((self.scenes, self.fps * grid_h * grid_w), dtype=dt, device=d)
        self.qkv = e((rows, 3, num_heads, head_dim), dtype=dt, device=d)
        # plan
        self.mask = e((frames, self.M), dtype=torch.uint8, device=d)
        self.group_prefix = e((frames, self.M), dtype=torch.int32, device=d)
        self.offsets = e((frames + 1,), dtype=torch.int32, device=d)
        self.rev = e((rows,), dtype=torch.int64, device=d)
        self.weight = torch.ones((rows,), dtype=torch.float32, device=d)
        self.seg_max = e((1,), dtype=torch.int32, device=d)
        self.bias = e((rows,), dtype=dt, device=d)
        self.cu_global = torch.zeros((self.scenes + 1,), dtype=torch.int32, device=d)
        self.global_max = e((1,), dtype=torch.int32, device=d)  # longest scene (global-attention segment), device side
        self.ratios = torch.full((frames,), float(threshold), dtype=torch.float32, device=d)
        self.ws_bytes = int(_lib.lib().come_merge_plan_workspace_bytes(frames))
        self.ws = e((self.ws_bytes,), dtype=torch.uint8, device=d)
        # per-layer scratch and output
        self.merged = e((rows, channels), dtype=dt, device=d)
        self.attn = e((rows, num_heads, head_dim), dtype=dt, device=d)
        self.lse = e((num_heads, rows), dtype=torch.float32, device=d)
        self.out = e((frames, self.N, channels), dtype=dt, device=d)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches_per_scene = 3 + 3 * len(self.layer_kinds)

    # -- the launch sequence (same for every mask) -----------------------------------------------------------
    def _enqueue(self) -> None:
        lib, st, code = _lib.lib(), stream_ptr(self.dev), dtype_code(self.dtype)
        H_, W_, gh, gw = self.grid
        if self.per_frame_ratios:
            _lib.check(lib.come_select_windows_ratios(ptr(self.conf), code, self.scenes, self.fps, H_, W_, gh, gw,
                                                      ptr(self.ratios), _lib.COME_SCOPE_FRAME, ptr(self.mask), st))
        else:
            _lib.check(lib.come_select_windows(ptr(self.conf), code, self.scenes, self.fps, H_, W_, gh, gw, self.threshold,
                                               _lib.COME_SELECT_RANK,
                                               _lib.COME_SCOPE_FRAME if self.scope == "frame" else _lib.COME_SCOPE_BATCH,
                                               ptr(self.mask), st))
        _lib.check(lib.come_merge_plan(ptr(self.mask), self.frames, C.byref(self.layout), ptr(self.group_prefix),
                                       ptr(self.offsets), ptr(self.rev), ptr(self.weight), ptr(self.seg_max), ptr(self.ws),
                                       self.ws_bytes, st))
        # per-key bias log(count) in the run dtype; rows past the packed length hold stale counts and are never read
        torch.log(self.weight, out=self._bias32)
        self.bias.copy_(self._bias32)
        self.cu_global.copy_(self.offsets[:: self.fps])  # scene boundaries = every frames_per_scene-th frame offset
        torch.amax(self.cu_global[1:] - self.cu_global[:-1], dim=0, keepdim=True, out=self.global_max)
        q, k, v = self.qkv[:, 0], self.qkv[:, 1], self.qkv[:, 2]
        for kind in self.layer_kinds:
            _lib.check(lib.come_merge(ptr(self.x), code, self.frames, self.C, C.byref(self.layout), ptr(self.mask),
                                      ptr(self.group_prefix), ptr(self.offsets), ptr(self.merged), st))
            # host-side bound = the unmerged worst case (the graph serves every mask); the true longest segment, which
            # the plan kernel left in device memory, trims the kernel's work list to the query blocks that exist
            if kind == "global":
                cu, nseg, max_len, max_dev = self.cu_global, self.scenes, self.fps * self.N, self.global_max
            else:
                cu, nseg, max_len, max_dev = self.offsets, self.frames, self.N, self.seg_max
            _lib.check(lib.come_attn_varlen_fwd_rows(ptr(q), ptr(k), ptr(v), code, self.rows_max, 0, self.rows_max, self.H,
                                                     self.D, q.stride(0), k.stride(0), v.stride(0), ptr(self.bias), ptr(cu),
                                                     nseg, max_len, ptr(max_dev), self.scale, ptr(self.attn),
                                                     self.attn.stride(0), ptr(self.lse), 0, st))
            _lib.check(lib.come_unmerge(ptr(self.attn), ptr(self.rev), self.rows_max, self.C, code, ptr(self.out), st))

    def capture(self) -> "StaticScene":
        """Run the sequence once eagerly (first-use set-up of the library happens outside the capture), then capture it."""
        self._bias32 = torch.empty((self.rows_max,), dtype=torch.float32, device=self.dev)
        with torch.cuda.device(self.dev):
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._enqueue()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._enqueue()
        return self

    def run(self, x: Optional[torch.Tensor] = None, confidence: Optional[torch.Tensor] = None,
            qkv: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Inputs may live on the host (pinned) or the device; ``None`` keeps what the static buffers hold.
        ``qkv`` may have fewer rows than the worst case (only the first ``P`` packed rows are read)."""
        if self.graph is None:
            self.capture()
        if x is not None:
            self.x.copy_(x, non_blocking=True)
        if confidence is not None:
            self.conf.copy_(confidence.reshape(self.conf.shape), non_blocking=True)
        if qkv is not None:
            self.qkv[: qkv.shape[0]].copy_(qkv, non_blocking=True)
        self.graph.replay()
        return self.out

    # -- pipelined host <-> device traffic -------------------------------------------------------------------
    def _pipe_init(self) -> None:
        d = self.dev
        self._copy_stream = torch.cuda.Stream(device=d)
        self._stage = [(torch.empty_like(self.x), torch.empty_like(self.conf), torch.empty_like(self.qkv)) for _ in range(2)]
        self._out_stage = [torch.empty_like(self.out) for _ in range(2)]
        self._staged = [torch.cuda.Event() for _ in range(2)]    # inputs of slot i are on the device
        self._consumed = [torch.cuda.Event() for _ in range(2)]  # slot i has been copied into the static inputs
        self._done = [torch.cuda.Event() for _ in range(2)]      # output of slot i is in its staging buffer
        self._drained = [torch.cuda.Event() for _ in range(2)]   # output staging buffer i has left for the host
        self._put = self._get = 0

    def stage(self, x_host: torch.Tensor, conf_host: torch.Tensor, qkv_host: torch.Tensor) -> None:
        """Start copying the NEXT scene's (pinned) host inputs to the device on a side stream; returns at once.  At
        most two scenes may be staged ahead of :meth:`run_staged`."""
        if not hasattr(self, "_copy_stream"):
            self._pipe_init()
        i = self._put % 2
        with torch.cuda.stream(self._copy_stream):
            if self._put >= 2:
                self._copy_stream.wait_event(self._consumed[i])
            sx, sc, sq = self._stage[i]
            sx.copy_(x_host, non_blocking=True)
            sc.copy_(conf_host.reshape(sc.shape), non_blocking=True)
            sq[: qkv_host.shape[0]].copy_(qkv_host, non_blocking=True)
            self._staged[i].record(self._copy_stream)
        self._put += 1

    def run_staged(self, out_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run the oldest staged scene on the current stream; with ``out_host`` (pinned) the result is sent to the
        host on the side stream while the next scene computes.  Returns the device staging buffer of the result."""
        if self.graph is None:
            self.capture()
        if self._get >= self._put:
            raise RuntimeError("run_staged() without a staged scene")
        i = self._get % 2
        cur = torch.cuda.current_stream(self.dev)
        cur.wait_event(self._staged[i])
        sx, sc, sq = self._stage[i]
        self.x.copy_(sx, non_blocking=True)
        self.conf.copy_(sc, non_blocking=True)
        self.qkv.copy_(sq, non_blocking=True)
        self._consumed[i].record(cur)
        self.graph.replay()
        if self._get >= 2:
            cur.wait_event(self._drained[i])
        self._out_stage[i].copy_(self.out, non_blocking=True)
        self._done[i].record(cur)
        if out_host is not None:
            with torch.cuda.stream(self._copy_stream):
                self._copy_stream.wait_event(self._done[i])
                out_host.copy_(self._out_stage[i], non_blocking=True)
                self._drained[i].record(self._copy_stream)
        else:
            self._drained[i].record(cur)
        self._get += 1
        return self._out_stage[i]

    def drain(self) -> None:
        """Wait for every outstanding copy of the pipeline."""
        if hasattr(self, "_copy_stream"):
            self._copy_stream.synchronize()

    def packed_rows(self) -> int:
        """Packed length of the last scene (reads one int back: for reporting, not needed to run)."""
        return int(self.offsets[-1].item())
