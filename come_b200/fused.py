"""The merged ("fused") forward pass of the alternating-attention aggregator, mirroring the forward the reference
patches into ``Aggregator`` (``src/accelerate/vggt/fused.py:95-167``): tokens are merged ONCE after the encoder, all
frame and global blocks run on the packed tokens, and only the retained layers are unmerged for the heads.

Against the reference's closure:

* the merge context is a :class:`~come_b200.token_merger.MergePlan` (one device-to-host read per scene); the packed
  positions come from the plan (``come_packed_positions``) instead of a second merge of a bfloat16 position tensor
  (``fused.py:113-129``);
* a retained layer is unmerged straight into its half of the concatenated ``[B, S, N, 2C]`` tensor
  (``come_unmerge_strided``) instead of two splits and a ``torch.cat`` (``fused.py:157-167``);
* when the token stream is already in the attention dtype, each ``LayerScale -> residual add -> LayerNorm`` between two
  GEMMs of the blocks (``module/block.py:66-79``) is one kernel (``come_residual_layernorm``) instead of three;
* every attention call gets the longest segment from the plan, so the block loop has no device-to-host read and can
  be captured in a CUDA graph (:class:`CapturedForward`), one graph per packed length.

The encoder, the heads and the confidence predictor are not part of this module: it starts from the dense tokens
``[B, S, N, C]`` the aggregator assembles (``fused.py:103-126``) and a merge mask.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .block import JaggedBlock, JaggedBlock_w_Bias, forward_fused, fusable, residual_layernorm
from .token_merger import JaggedTokens, MergePlan

__all__ = ["FusedAggregator", "ShardedFusedAggregator", "CapturedForward", "fused_accelerate", "FusedModel", "run_blocks"]


class FusedAggregator(torch.nn.Module):
    """``aggregator`` provides ``frame_blocks``, ``global_blocks``, ``aa_order``, ``aa_block_size``, ``aa_block_num``,
    ``retain_layers`` (None = all) and ``patch_start_idx`` (``src/thirdparty/vggt/models/aggregator.py:76-131``)."""

    def __init__(self, aggregator: torch.nn.Module, use_attn_bias_correction: bool = True, attn_dtype: str = "bf16",
                 fuse_elementwise: bool = True):
        """``fuse_elementwise``: run every ``LayerScale -> residual add -> LayerNorm`` of the blocks as one kernel
        (:func:`come_b200.block.forward_fused`) when the model allows it (token stream in the attention dtype, plain
        LayerNorm / LayerScale modules); otherwise, and when off, the blocks run module by module as in the reference."""
        super().__init__()
        self.fuse_elementwise = bool(fuse_elementwise)
        block_fn = JaggedBlock_w_Bias if use_attn_bias_correction else JaggedBlock
        self.aggregator = aggregator
        self.frame_blocks = torch.nn.ModuleList([block_fn(b, attn_dtype) for b in aggregator.frame_blocks])
        self.global_blocks = torch.nn.ModuleList([block_fn(b, attn_dtype) for b in aggregator.global_blocks])
        # the same blocks without the count bias, for tokens that were never merged
        self.plain_frame_blocks = torch.nn.ModuleList([JaggedBlock(b, attn_dtype) for b in aggregator.frame_blocks])
        self.plain_global_blocks = torch.nn.ModuleList([JaggedBlock(b, attn_dtype) for b in aggregator.global_blocks])
        self.aa_order = list(aggregator.aa_order)
        self.aa_block_size = int(aggregator.aa_block_size)
        self.aa_block_num = int(aggregator.aa_block_num)
        self.retain_layers = aggregator.retain_layers
        self.patch_start_idx = int(aggregator.patch_start_idx)

    # ------------------------------------------------------------------------------------------------------
    def _run(self, x: JaggedTokens, pos: torch.Tensor, frame_view, global_view, frame_blocks, global_blocks, unmerge):
        """The alternating loop (``fused.py:137-169``).  ``frame_view`` / ``global_view`` re-segment a JaggedTokens,
        ``unmerge(frame_tokens, global_tokens)`` produces a retained layer's output."""
        order = []  # the blocks in execution order (the fused path hands each block the next one's norm1)
        fi = gi = 0
        for _ in range(self.aa_block_num):
            for attn_type in self.aa_order:
                if attn_type not in ("frame", "global"):
                    raise ValueError(f"Unknown attention type: {attn_type}")
                for _ in range(self.aa_block_size):
                    if attn_type == "frame":
                        order.append(frame_blocks[fi])
                        fi += 1
                    else:
                        order.append(global_blocks[gi])
                        gi += 1
        fused = self.fuse_elementwise and bool(order) and all(fusable(w, x.tokens.dtype) for w in order)
        normed = None
        if fused:
            _, normed = residual_layernorm(x.tokens.squeeze(0), None, None, order[0].block.norm1)
        step = block_idx = 0
        output: Dict[int, torch.Tensor] = {}
        for _ in range(self.aa_block_num):
            frame_intermediate, globe_intermediate = [], []
            for attn_type in self.aa_order:
                x = frame_view(x) if attn_type == "frame" else global_view(x)
                for _ in range(self.aa_block_size):
                    if fused:
                        next_norm = order[step + 1].block.norm1 if step + 1 < len(order) else None
                        x, normed = forward_fused(order[step], x, normed, pos, next_norm)
                    else:
                        x = order[step](x, pos=pos)
                    (frame_intermediate if attn_type == "frame" else globe_intermediate).append(x)
                    step += 1
            for i in range(self.aa_block_size):
                if self.retain_layers is None or block_idx in self.retain_layers:
                    output[block_idx] = unmerge(frame_intermediate[i].tokens.squeeze(0),
                                                globe_intermediate[i].tokens.squeeze(0))
                block_idx += 1
        return output

    def forward(self, tokens: torch.Tensor, plan: MergePlan, static_shapes: bool = False
                ) -> Tuple[Dict[int, torch.Tensor], int]:
        """``tokens [B, S, N, C]`` dense; ``plan`` the merge plan of its ``B*S`` frames.  Returns the retained layers
        ``{block index: [B, S, N, 2C]}`` (frame and global tokens side by side) and ``patch_start_idx``.

        With ``static_shapes`` nothing launched depends on the segment lengths inside ``plan`` -- launches are sized
        for the unmerged lengths and read the real ones on the device -- so the same launch sequence serves every
        plan with the same packed length: the form a CUDA graph captures."""
        B, S, N, C = tokens.shape
        if plan.frames != B * S or plan.tokens_per_frame != N:
            raise ValueError(f"plan covers {plan.frames} frames of {plan.tokens_per_frame} tokens, tokens are {tuple(tokens.shape)}")
        merged = plan.merge(tokens.reshape(B * S, N, C))
        pos = plan.positions()
        frame_offset = plan.offset
        global_offset = plan.offset[::S].contiguous()
        if static_shapes:
            frame_max, frame_max_dev = N, plan.seg_max
            global_max = S * N
            global_max_dev = (global_offset[1:] - global_offset[:-1]).max().to(torch.int32).reshape(1)
        else:
            frame_max, frame_max_dev = plan.max_seqlen, None
            # several scenes: one read of the longest scene per forward pass (not one per global block)
            global_max = plan.total if B == 1 else int((global_offset[1:] - global_offset[:-1]).max().item())
            global_max_dev = None

        frame_cu, global_cu = plan.cu_seqlens(1), plan.cu_seqlens(S)  # the plan's int32 offsets: no cast per block

        def frame_view(x: JaggedTokens) -> JaggedTokens:
            return JaggedTokens(x.tokens, x.weight, frame_offset, frame_max, frame_max_dev, cu_seqlens=frame_cu)

        def global_view(x: JaggedTokens) -> JaggedTokens:
            return JaggedTokens(x.tokens, x.weight, global_offset, global_max, global_max_dev, cu_seqlens=global_cu)

        def unmerge(frame_tokens: torch.Tensor, global_tokens: torch.Tensor) -> torch.Tensor:
            return plan.split_concat(frame_tokens, global_tokens).view(B, S, N, 2 * C)

        x = JaggedTokens(tokens=merged.unsqueeze(0), weight=plan.weight, offset=frame_offset)
        output = self._run(x, pos, frame_view, global_view, self.frame_blocks, self.global_blocks, unmerge)
        return output, self.patch_start_idx

    def forward_unmerged(self, tokens: torch.Tensor, pos: Optional[torch.Tensor] = None
                         ) -> Tuple[Dict[int, torch.Tensor], int]:
        """The same stack on the dense tokens, nothing merged and no count bias: the model the accelerated one is
        compared with.  ``pos [B*S*N, 2]`` int64 (y, x); by default specials at (0, 0) and patch (y, x) at
        (y + 1, x + 1) on a square grid (``src/thirdparty/vggt/models/aggregator.py:217-229``)."""
        B, S, N, C = tokens.shape
        dev = tokens.device
        if pos is None:
            side = int(round((N - self.patch_start_idx) ** 0.5))
            if side * side != N - self.patch_start_idx:
                raise ValueError("pass pos for a patch grid that is not square")
            yy, xx = torch.meshgrid(torch.arange(1, side + 1, device=dev), torch.arange(1, side + 1, device=dev), indexing="ij")
            frame_pos = torch.cat([torch.zeros(self.patch_start_idx, 2, dtype=torch.int64, device=dev),
                                   torch.stack([yy.reshape(-1), xx.reshape(-1)], dim=-1)], dim=0)
            pos = frame_pos.repeat(B * S, 1)
        frame_offset = torch.arange(0, B * S * N + 1, N, device=dev, dtype=torch.int64)
        global_offset = frame_offset[::S].contiguous()
        weight = torch.ones(B * S * N, dtype=torch.float32, device=dev)

        def frame_view(x: JaggedTokens) -> JaggedTokens:
            return JaggedTokens(x.tokens, x.weight, frame_offset, N)

        def global_view(x: JaggedTokens) -> JaggedTokens:
            return JaggedTokens(x.tokens, x.weight, global_offset, S * N)

        def unmerge(frame_tokens: torch.Tensor, global_tokens: torch.Tensor) -> torch.Tensor:
            return torch.cat((frame_tokens, global_tokens), dim=-1).view(B, S, N, 2 * C)

        x = JaggedTokens(tokens=tokens.reshape(1, B * S * N, C), weight=weight, offset=frame_offset)
        output = self._run(x, pos, frame_view, global_view, self.plain_frame_blocks, self.plain_global_blocks, unmerge)
        return output, self.patch_start_idx


class ShardedFusedAggregator(FusedAggregator):
    """The merged forward pass of ONE scene whose frames are spread over the ranks of a process group (one process per
    GPU): every rank merges, runs and unmerges its own contiguous range of frames.  Everything row-wise (norms, GEMMs,
    MLP, LayerScale, residuals) and the frame blocks need no other rank; a global block all-gathers the prepared key /
    value rows of the packed tokens -- the only exchange -- and attends the local query rows to all of them
    (:class:`come_b200.dist.GlobalExchange`).  The merge mask of all frames is replicated, so every rank derives the
    packed row counts of all ranks without a collective.
    """

    def __init__(self, aggregator: torch.nn.Module, frames_total: int, world: int, rank: int, group=None, gather=None,
                 use_attn_bias_correction: bool = True, attn_dtype: str = "bf16", fuse_elementwise: bool = True,
                 overlap: bool = False):
        """``gather(local, rows, rank)`` replaces the process group's all-gather (single-process tests); by default the
        rows travel through :func:`come_b200.dist.gather_rows` over ``group``.  ``overlap``: hide that exchange behind
        attention to the local keys (:class:`come_b200.dist.GlobalExchange`)."""
        super().__init__(aggregator, use_attn_bias_correction, attn_dtype, fuse_elementwise)
        self.overlap = bool(overlap)
        self._exchange = None
        from .dist import shard_range
        self.frames_total, self.world, self.rank = int(frames_total), int(world), int(rank)
        self.group, self._gather = group, gather
        self.f_lo, self.f_hi = shard_range(self.frames_total, self.world, self.rank)

    def build_plans(self, mask_all: torch.Tensor, layout) -> Tuple[MergePlan, MergePlan]:
        """``mask_all [frames_total, M]`` (the same on every rank) -> (plan of the whole scene, plan of this rank's
        frames)."""
        if mask_all.shape[0] != self.frames_total:
            raise ValueError(f"mask covers {mask_all.shape[0]} frames, the scene has {self.frames_total}")
        return MergePlan(mask_all, layout), MergePlan(mask_all[self.f_lo:self.f_hi].contiguous(), layout)

    def forward(self, tokens_local: torch.Tensor, global_plan: MergePlan, local_plan: MergePlan
                ) -> Tuple[Dict[int, torch.Tensor], int]:
        """``tokens_local [1, frames_local, N, C]``: this rank's frames ``[f_lo, f_hi)``.  Returns the retained layers of
        those frames, ``{block index: [1, frames_local, N, 2C]}``."""
        from .dist import GlobalExchange, rows_per_rank
        B, S_local, N, C = tokens_local.shape
        if B != 1 or S_local != self.f_hi - self.f_lo or local_plan.frames != S_local or global_plan.frames != self.frames_total:
            raise ValueError(f"rank {self.rank} owns frames [{self.f_lo}, {self.f_hi}) of one scene, got tokens {tuple(tokens_local.shape)}")
        rows = rows_per_rank(global_plan.offset.tolist(), self.world)
        if rows[self.rank] != local_plan.total:
            raise ValueError("the local plan is not this rank's slice of the scene's plan")
        exchange = GlobalExchange(rows, self.rank, global_plan.weight, self.group, self._gather, overlap=self.overlap)
        keep = self._exchange
        if keep is not None and keep.rows == exchange.rows and keep._side is not None:  # keep the side stream and the buffer
            exchange._side, exchange._buf, exchange._cu_local = keep._side, keep._buf, keep._cu_local
        self._exchange = exchange
        merged = local_plan.merge(tokens_local.reshape(S_local, N, C))
        pos = local_plan.positions()
        frame_offset = local_plan.offset
        scene_offset = torch.tensor([0, local_plan.total], dtype=torch.int64, device=tokens_local.device)

        def frame_view(x: JaggedTokens) -> JaggedTokens:
            return JaggedTokens(x.tokens, x.weight, frame_offset, local_plan.max_seqlen)

        def global_view(x: JaggedTokens) -> JaggedTokens:
            return JaggedTokens(x.tokens, x.weight, scene_offset, exchange=exchange)

        def unmerge(frame_tokens: torch.Tensor, global_tokens: torch.Tensor) -> torch.Tensor:
            return local_plan.split_concat(frame_tokens, global_tokens).view(1, S_local, N, 2 * C)

        x = JaggedTokens(tokens=merged.unsqueeze(0), weight=local_plan.weight, offset=frame_offset)
        output = self._run(x, pos, frame_view, global_view, self.frame_blocks, self.global_blocks, unmerge)
        return output, self.patch_start_idx


def run_blocks(wrappers, x: JaggedTokens, pos: Optional[torch.Tensor], fuse: bool = True) -> JaggedTokens:
    """A plain sequence of jagged blocks (the patch encoder's), with the elementwise steps fused when the blocks allow it."""
    wrappers = list(wrappers)
    if not wrappers:
        return x
    if fuse and all(fusable(w, x.tokens.dtype) for w in wrappers):
        _, normed = residual_layernorm(x.tokens.squeeze(0), None, None, wrappers[0].block.norm1)
        for i, w in enumerate(wrappers):
            nxt = wrappers[i + 1].block.norm1 if i + 1 < len(wrappers) else None
            x, normed = forward_fused(w, x, normed, pos, nxt)
        return x
    for w in wrappers:
        x = w(x, pos=pos)
    return x


class FusedModel(torch.nn.Module):
    """The accelerated model from the images to the retained aggregator layers, in the shape of the reference's fused mode
    (``src/accelerate/vggt/fused.py:40-94``): the patch encoder runs dense up to block ``encoder_layer``; its output
    feeds the confidence predictor, the windows are selected and the tokens merged at once; the remaining encoder blocks
    run on the packed tokens with the count bias; the tokens are split after the last encoder block, normed, given the
    aggregator's camera and register tokens, merged again with the same plan, and the alternating-attention stack runs
    as :class:`FusedAggregator`.  The prediction heads are outside (they consume the retained layers).

    ``forward_unmerged`` runs the same weights with nothing merged: the model the accelerated one is compared with
    (``src/bench.py:13-46``, "Reference Model" against "Accelerated Model")."""

    def __init__(self, encoder: torch.nn.Module, aggregator: torch.nn.Module, predictor, encoder_layer: int = 14,
                 group_h: int = 3, group_w: int = 3, threshold: float = 0.5, conf_mode: str = "pairwise-rank",
                 use_attn_bias_correction: bool = True, attn_dtype: str = "bf16"):
        super().__init__()
        from .token_merger import CoMe2DTokenMerger
        if not (0 <= encoder_layer < len(encoder.blocks)):
            raise ValueError(f"encoder_layer {encoder_layer} outside the encoder's {len(encoder.blocks)} blocks")
        self.encoder, self.predictor, self.encoder_layer = encoder, predictor, int(encoder_layer)
        block_fn = JaggedBlock_w_Bias if use_attn_bias_correction else JaggedBlock
        self.enc_dense = torch.nn.ModuleList([JaggedBlock(b, attn_dtype) for b in encoder.blocks])
        self.enc_merged = torch.nn.ModuleList([block_fn(b, attn_dtype) for b in encoder.blocks[encoder_layer + 1:]])
        self.aggregator = FusedAggregator(aggregator, use_attn_bias_correction, attn_dtype)
        self.merger = CoMe2DTokenMerger(encoder.prefix_tokens, group_h, group_w, threshold, predictor, conf_mode)
        self.last_plan: Optional[MergePlan] = None

    def _dense_tokens(self, images: torch.Tensor):
        B, S = images.shape[:2]
        tokens = self.encoder.embed(images.flatten(0, 1))  # [B*S, N, C]
        N = tokens.shape[1]
        offset = torch.arange(0, B * S * N + 1, N, device=tokens.device, dtype=torch.int64)
        weight = torch.ones(B * S * N, dtype=torch.float32, device=tokens.device)
        x = JaggedTokens(tokens.reshape(1, B * S * N, -1), weight, offset, max_seqlen=N, cu_seqlens=offset.to(torch.int32))
        return x, B, S, N

    def forward(self, images: torch.Tensor) -> Tuple[Dict[int, torch.Tensor], int]:
        """``images [B, S, 3, H, W]`` -> (retained layers ``{block index: [B, S, N, 2C]}``, ``patch_start_idx``)."""
        enc = self.encoder
        x, B, S, N = self._dense_tokens(images)
        h, w = enc.grid
        x = run_blocks(self.enc_dense[: self.encoder_layer + 1], x, None)
        dense = x.tokens.reshape(B * S, N, -1)
        start = enc.prefix_tokens
        feature = dense[:, start:].permute(0, 2, 1).reshape(B, S, -1, h, w)  # [B, S, C, h, w] as the reference's hook builds it
        ctx = self.merger.build_ctx(feature)
        plan = ctx[2]
        self.last_plan = plan
        merged = plan.merge(dense)
        xm = JaggedTokens(merged.unsqueeze(0), plan.weight, plan.offset, max_seqlen=plan.max_seqlen, cu_seqlens=plan.cu_seqlens(1))
        xm = run_blocks(self.enc_merged, xm, None)
        dense = enc.norm(plan.split(xm.tokens.squeeze(0)).reshape(B * S, N, -1))
        tokens = self.aggregator.aggregator.assemble_tokens(dense[:, start:], B, S)
        if tokens.shape[2] != N:
            raise ValueError("the aggregator's special tokens must number the encoder's (one merge plan serves both)")
        return self.aggregator(tokens.contiguous(), plan)

    def forward_unmerged(self, images: torch.Tensor) -> Tuple[Dict[int, torch.Tensor], int]:
        enc = self.encoder
        x, B, S, N = self._dense_tokens(images)
        x = run_blocks(self.enc_dense, x, None)
        dense = enc.norm(x.tokens.reshape(B * S, N, -1))
        tokens = self.aggregator.aggregator.assemble_tokens(dense[:, enc.prefix_tokens:], B, S)
        h, w = enc.grid
        dev = tokens.device
        yy, xx = torch.meshgrid(torch.arange(1, h + 1, device=dev), torch.arange(1, w + 1, device=dev), indexing="ij")
        frame_pos = torch.cat([torch.zeros(enc.prefix_tokens, 2, dtype=torch.int64, device=dev),
                               torch.stack([yy.reshape(-1), xx.reshape(-1)], dim=-1)], dim=0)
        return self.aggregator.forward_unmerged(tokens.contiguous(), frame_pos.repeat(B * S, 1))


def fused_accelerate(aggregator: torch.nn.Module, use_attn_bias_correction: bool = True) -> FusedAggregator:
    """Counterpart of the reference's ``fused_accelerate(model, token_merger, encoder_layer, use_attn_bias_correction)``
    (``fused.py:18-21``) for the aggregator alone: wraps its blocks, bf16 attention as in ``fused.py:78,91,94``."""
    return FusedAggregator(aggregator, use_attn_bias_correction=use_attn_bias_correction, attn_dtype="bf16")


class CapturedForward:
    """Replays :meth:`FusedAggregator.forward` from CUDA graphs, one per (input shape, packed length).

    Per scene: the plan is built eagerly (two small kernels and its one host read, which yields the packed length and
    picks the graph), copied into the static plan the graph was captured with, the tokens are copied into the static
    input, and the graph is replayed.  The returned tensors are the graph's static outputs: valid until the next call
    with the same packed length.
    """

    def __init__(self, model: FusedAggregator, warmup: int = 2):
        self.model, self.warmup = model, int(warmup)
        self._graphs: Dict[tuple, tuple] = {}

    def __call__(self, tokens: torch.Tensor, plan: MergePlan) -> Tuple[Dict[int, torch.Tensor], int]:
        key = (tuple(tokens.shape), tokens.dtype, plan.total)
        entry = self._graphs.get(key)
        if entry is None:
            entry = self._capture(tokens, plan)
            self._graphs[key] = entry
        graph, static_tokens, static_plan, output = entry
        static_tokens.copy_(tokens)
        static_plan.load(plan, keep_derived=True)
        graph.replay()
        return output, self.model.patch_start_idx

    @torch.no_grad()
    def _capture(self, tokens: torch.Tensor, plan: MergePlan):
        static_tokens = tokens.clone()
        static_plan = MergePlan(plan.mask.clone(), plan.layout)
        side = torch.cuda.Stream(device=tokens.device)
        side.wait_stream(torch.cuda.current_stream(tokens.device))
        with torch.cuda.stream(side):  # warm-up outside the capture: lazy initialisations, cuBLAS workspaces
            for _ in range(self.warmup):
                self.model(static_tokens, static_plan, static_shapes=True)
        torch.cuda.current_stream(tokens.device).wait_stream(side)
        static_plan._positions = None  # recomputed inside the graph, into memory the graph owns
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            output, _ = self.model(static_tokens, static_plan, static_shapes=True)
        return graph, static_tokens, static_plan, output
