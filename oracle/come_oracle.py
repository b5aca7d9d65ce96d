"""CPU oracle for the Co-Me hot path (merge plan, merge, unmerge, window selection, biased attention).

TEST INFRASTRUCTURE ONLY.  This module is a plain numpy restatement of the reference algorithm and is
imported by the test-suite, by the smoke check and by the CPU-baseline leg of the benchmark — never by the
product package, which must fail loudly when its CUDA library is missing.

Every function cites the reference file (paths relative to the reference project root) it restates.
Pinned against the reference: the committed fixtures under ``tests/golden`` were produced by importing the
reference's own PyTorch implementation on CPU (``tests/golden/make_golden.py``: the merge / split functions, the
2-D merger, ``build_ctx``, ``prepare_packed_self_attention_qkv`` with the rotary module, the model's ``Block`` and the
``JaggedTokens`` suffix methods) and against the literal known-answer cases of the reference's test-suite
(``tests/golden/reference_cases.py``).
"""
from __future__ import annotations

import numpy as np

__all__ = [
    "merge_plan",
    "token_merge",
    "token_split",
    "token_split_residual",
    "block_perm_2d",
    "token_merge_2d",
    "ragged_layout_2d",
    "token_merge_2d_ragged",
    "window_means",
    "quantile_linear",
    "select_windows",
    "attention_bias",
    "attention_combine",
    "attention_combine_parts",
    "perkey_bias_from_weight",
    "max_seqlen",
    "rope_tables",
    "layer_norm_heads",
    "layer_norm_rows",
    "residual_layer_norm",
    "rope_2d",
    "qkv_prepare",
    "packed_positions",
    "jagged_add_suffix",
    "jagged_split_suffix",
    "gelu_erf",
    "jagged_block",
    "fused_aggregator",
]


# --------------------------------------------------------------------------------------------------------
# merge index plan
# --------------------------------------------------------------------------------------------------------
def merge_plan(mask: np.ndarray, group_size: int, start_index: int):
    """Index plan of one merge.

    Restates ``src/accelerate/token_merger/co_me.py:177-183,199-201`` (and the device twin
    ``src/cuda_extension/co_me/src/kernel_token_merge.cu:12-46,284-286``):
    a merged group emits one row, a kept group emits ``G`` rows, every frame starts with ``start_index``
    untouched rows.

    Returns ``(group_prefix[B,M] int64, offsets[B+1] int64, P)``.
    """
    mask = np.asarray(mask, dtype=bool)
    B, M = mask.shape
    G = int(group_size)
    group_len = np.where(mask, 1, G).astype(np.int64)
    group_prefix = np.cumsum(group_len, axis=1) - group_len
    k_b = mask.sum(axis=1, dtype=np.int64)
    L_b = start_index + (M - k_b) * G + k_b
    offsets = np.zeros(B + 1, dtype=np.int64)
    offsets[1:] = np.cumsum(L_b)
    return group_prefix, offsets, int(offsets[-1])


def _mean_rows_sequential(rows: np.ndarray) -> np.ndarray:
    """Mean over axis -2 accumulated g = 0, 1, ... in the array's own precision, then a true division.

    This is the rounding the reference's CPU path produces for ``img.mean(dim=2)``
    (``co_me.py:192-193``): a left-to-right sum in the element type followed by ``/ G``.
    float16 / bfloat16 inputs must be passed as float32 by the caller and rounded afterwards.
    """
    G = rows.shape[-2]
    acc = np.zeros(rows.shape[:-2] + rows.shape[-1:], dtype=rows.dtype)
    for g in range(G):
        acc = acc + rows[..., g, :]
    return acc / rows.dtype.type(G)


# --------------------------------------------------------------------------------------------------------
# 1-D merge / split
# --------------------------------------------------------------------------------------------------------
def token_merge(tokens: np.ndarray, start_index: int, group_size: int, mask: np.ndarray):
    """``func_token_merge`` (``src/accelerate/token_merger/co_me.py:152-222``).

    tokens ``[B, N, C]`` with ``N = start_index + M * G``; mask ``[B, M]`` bool.
    Returns ``(out[P,C], offsets[B+1] int64, rev_id[B*N] int64, weight[P] float32)``.
    """
    tokens = np.asarray(tokens)
    mask = np.asarray(mask, dtype=bool)
    B, N, C = tokens.shape
    _, M = mask.shape
    G = int(group_size)
    S = int(start_index)
    if N != S + M * G:
        raise ValueError(f"Expected N = start_index + M * group_size = {S + M * G}, got N = {N}")
    group_prefix, offsets, P = merge_plan(mask, G, S)

    out = np.empty((P, C), dtype=tokens.dtype)
    rev = np.empty((B, N), dtype=np.int64)
    weight = np.empty((P,), dtype=np.float32)
    base = offsets[:-1]

    special_pos = base[:, None] + np.arange(S, dtype=np.int64)[None, :]
    out[special_pos.reshape(-1)] = tokens[:, :S, :].reshape(-1, C)
    rev[:, :S] = special_pos
    weight[special_pos.reshape(-1)] = 1.0

    img = tokens[:, S:, :].reshape(B, M, G, C)
    merged = _mean_rows_sequential(img)
    group_base = base[:, None] + S + group_prefix  # [B, M]
    unmerged_pos = group_base[..., None] + np.arange(G, dtype=np.int64)

    merged_pos = group_base[mask]
    out[merged_pos] = merged[mask]
    weight[merged_pos] = float(G)

    keep = ~mask
    keep_pos = unmerged_pos[keep].reshape(-1)
    out[keep_pos] = img[keep].reshape(-1, C)
    weight[keep_pos] = 1.0

    rev[:, S:] = np.where(mask[..., None], group_base[..., None], unmerged_pos).reshape(B, M * G)
    return out, offsets, rev.reshape(-1), weight


def token_split(merged: np.ndarray, rev_id: np.ndarray) -> np.ndarray:
    """``func_token_split`` (``src/accelerate/token_merger/co_me.py:241-254``): ``out[i] = merged[rev_id[i]]``."""
    return np.asarray(merged)[np.asarray(rev_id, dtype=np.int64)]


# --------------------------------------------------------------------------------------------------------
# 2-D merge
# --------------------------------------------------------------------------------------------------------
def token_split_residual(merged: np.ndarray, rev_id: np.ndarray, residual: np.ndarray, scale=None, kind: str = "f32"):
    """``x + ls1(split(attn_out))``: the unmerge followed by LayerScale (``x * gamma``,
    ``src/thirdparty/vggt/layers/layer_scale.py:21-22``) and the residual add of the block
    (``src/thirdparty/vggt/layers/block.py:73,90``), each tensor operation rounded to the element type ``kind``."""
    u = np.asarray(merged, np.float32)[np.asarray(rev_id, np.int64)]
    if scale is not None:
        u = _round_like((u * np.asarray(scale, np.float32)[None, :]).astype(np.float32), kind)
    return _round_like((np.asarray(residual, np.float32).reshape(u.shape) + u).astype(np.float32), kind)


def block_perm_2d(H: int, W: int, gh: int, gw: int) -> np.ndarray:
    """Row-major patch index of every (window, in-window) slot, windows in raster order.

    Restates ``_build_2d_block_perm`` (``src/accelerate/token_merger/co_me_2d.py:26-35``).
    """
    idx = np.arange(H * W, dtype=np.int64).reshape(H // gh, gh, W // gw, gw)
    return idx.transpose(0, 2, 1, 3).reshape(-1)


def token_merge_2d(tokens, start_index, gh, gw, H, W, mask):
    """``func_token_merge_2d`` / ``naive_func_token_merge_2d``
    (``src/accelerate/token_merger/co_me_2d.py:77-211``): permute the patch grid into window order, run the
    1-D merge with ``G = gh * gw``, and report ``rev_id`` in the original row-major token order.
    """
    tokens = np.asarray(tokens)
    B, N, C = tokens.shape
    if H % gh or W % gw:
        raise ValueError("H and W must be divisible by the window size")
    if N != start_index + H * W:
        raise ValueError(f"Expected N = start_index + H * W = {start_index + H * W}, got N = {N}")
    perm = np.concatenate([np.arange(start_index, dtype=np.int64), block_perm_2d(H, W, gh, gw) + start_index])
    out, offsets, rev_perm, weight = token_merge(tokens[:, perm, :], start_index, gh * gw, mask)
    inv = np.empty(N, dtype=np.int64)
    inv[perm] = np.arange(N, dtype=np.int64)
    rev = rev_perm.reshape(B, N)[:, inv]
    return out, offsets, rev.reshape(-1), weight


def ragged_layout_2d(start_index: int, H: int, W: int, gh: int, gw: int):
    """Token order used when the patch grid is not a multiple of the window (e.g. 37x37 with 3x3 windows).

    The reference itself rejects such grids (``co_me_2d.py:255-258``); the extension keeps the reference's
    1-D semantics by moving the patches that no window covers (right columns and bottom rows, in row-major
    order) directly behind the special tokens, so that they become part of the never-merged prefix
    (``start_index' = start_index + #edge``), exactly as ``func_token_merge_2d`` permutes a divisible grid
    (``co_me_2d.py:193-211``).

    Returns ``(perm[N], prefix_len, M)`` with ``perm`` mapping merge order -> original token index.
    """
    Hc, Wc = (H // gh) * gh, (W // gw) * gw
    yy, xx = np.meshgrid(np.arange(H), np.arange(W), indexing="ij")
    covered = (yy < Hc) & (xx < Wc)
    edge = (yy * W + xx)[~covered].reshape(-1).astype(np.int64)  # row-major order
    idx = (np.arange(Hc, dtype=np.int64)[:, None] * W + np.arange(Wc, dtype=np.int64)[None, :])
    win = idx.reshape(Hc // gh, gh, Wc // gw, gw).transpose(0, 2, 1, 3).reshape(-1)
    perm = np.concatenate([np.arange(start_index, dtype=np.int64), edge + start_index, win + start_index])
    return perm, start_index + edge.size, (Hc // gh) * (Wc // gw)


def token_merge_2d_ragged(tokens, start_index, gh, gw, H, W, mask):
    """2-D merge over the top-left ``floor(H/gh)*gh x floor(W/gw)*gw`` region; see :func:`ragged_layout_2d`."""
    tokens = np.asarray(tokens)
    B, N, C = tokens.shape
    if N != start_index + H * W:
        raise ValueError(f"Expected N = start_index + H * W = {start_index + H * W}, got N = {N}")
    perm, prefix, M = ragged_layout_2d(start_index, H, W, gh, gw)
    if np.asarray(mask).shape != (B, M):
        raise ValueError(f"Expected M = {M}")
    out, offsets, rev_perm, weight = token_merge(tokens[:, perm, :], prefix, gh * gw, mask)
    inv = np.empty(N, dtype=np.int64)
    inv[perm] = np.arange(N, dtype=np.int64)
    rev = rev_perm.reshape(B, N)[:, inv]
    return out, offsets, rev.reshape(-1), weight


# --------------------------------------------------------------------------------------------------------
# window selection
# --------------------------------------------------------------------------------------------------------
def _round_like(x32: np.ndarray, kind: str) -> np.ndarray:
    """Round float32 values to the storage precision ``kind`` and return them as float32."""
    if kind == "f32":
        return x32.astype(np.float32)
    if kind == "f16":
        return x32.astype(np.float16).astype(np.float32)
    if kind == "bf16":
        u = x32.astype(np.float32).view(np.uint32).astype(np.uint64)
        nan = np.isnan(x32)
        r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16  # round to nearest even
        out = (r & 0xFFFFFFFF).astype(np.uint32).view(np.float32)
        return np.where(nan, np.float32(np.nan), out)
    raise ValueError(kind)


def window_means(conf: np.ndarray, H: int, W: int, gh: int, gw: int, kind: str = "f32") -> np.ndarray:
    """Per-window mean confidence ``[F, M]`` from per-patch confidence ``[F, H*W]``.

    Restates ``conf_blocks.mean(dim=-1)`` (``src/accelerate/token_merger/co_me_2d.py:270-272,291``).  Windows
    tile the top-left ``floor(H/gh)*gh x floor(W/gw)*gw`` region in raster order.  The sum runs over the window
    row by row (``g = 0 .. gh*gw-1``) in float32 and is divided by ``gh*gw``; the result is rounded to the
    confidence storage precision ``kind`` ("f32", "f16", "bf16") like a tensor of that dtype would be.
    """
    conf = np.asarray(conf, dtype=np.float32)
    F = conf.shape[0]
    Hm, Wm = H // gh, W // gw
    grid = conf.reshape(F, H, W)[:, : Hm * gh, : Wm * gw]
    blocks = grid.reshape(F, Hm, gh, Wm, gw).transpose(0, 1, 3, 2, 4).reshape(F, Hm * Wm, gh * gw)
    acc = np.zeros((F, Hm * Wm), dtype=np.float32)
    for g in range(gh * gw):
        acc = acc + blocks[:, :, g]
    return _round_like(acc / np.float32(gh * gw), kind)


def quantile_linear(values: np.ndarray, q: float) -> np.float32:
    """``torch.quantile(values.float(), q)`` with the default linear interpolation, restated.

    PyTorch 2.x (``aten/src/ATen/native/Sorting.cpp`` ``quantile_compute`` + ``cpu/LerpKernel.cpp``): sort
    ascending, ``rank = q * (n - 1)`` in float32, ``lo = floor(rank)``, ``hi = ceil(rank)``, ``w = rank - lo``
    and a fused-multiply-add lerp: ``fma(w, b - a, a)`` for ``w < 0.5`` and ``fma(w - 1, b - a, b)`` otherwise
    (one rounding; the product of two float32 is exact in float64, which stands in for the fused operation).
    Checked against ``torch.quantile`` itself in the CPU tests.
    """
    v = np.sort(np.asarray(values, dtype=np.float32).reshape(-1))
    n = v.size
    rank = np.float32(q) * np.float32(n - 1)
    lo = np.floor(rank)
    hi = np.ceil(rank)
    w = np.float32(rank - lo)
    a, b = v[int(lo)], v[int(hi)]
    d = np.float32(b - a)
    if w < np.float32(0.5):
        return np.float32(np.float64(w) * np.float64(d) + np.float64(a))
    return np.float32(np.float64(np.float32(w - np.float32(1.0))) * np.float64(d) + np.float64(b))


def z_normalise(conf: np.ndarray, kind: str = "f32") -> np.ndarray:
    """``(x - mean) / (std + 1e-3)`` per batch element, ``conf [B, n]`` (``co_me_2d.py:275-278``, ``co_me.py:56-57``).

    Every tensor operation of the expression rounds to the confidence dtype ``kind``: the mean, the unbiased
    standard deviation, ``std + 1e-3``, the difference and the quotient.  Mean and standard deviation are accumulated
    in float64 here (PyTorch sums a float32 tensor in float32 with a cascade whose order depends on the vector width and
    the thread count; both round to the same 16-bit value, a float32 result can differ in its last bits).
    """
    x = np.asarray(conf, dtype=np.float32)
    n = x.shape[-1]
    x64 = x.astype(np.float64)
    mean64 = x64.sum(axis=-1, keepdims=True) / n
    var64 = ((x64 - mean64) ** 2).sum(axis=-1, keepdims=True) / (n - 1) if n > 1 else np.full_like(mean64, np.nan)
    mean = _round_like(mean64.astype(np.float32), kind)
    std = _round_like(np.sqrt(var64).astype(np.float32), kind)
    den = _round_like(std + np.float32(1e-3), kind)
    return _round_like(_round_like(x - mean, kind) / den, kind)


def select_windows(conf, B, S, H, W, gh, gw, threshold, mode="pairwise-rank", scope="batch", kind="f32"):
    """Merge mask ``[B*S, M]`` from per-patch confidence ``[B, S*H*W]``.

    Restates the tensor code of ``_CoMe_2D_Base.build_ctx`` (``src/accelerate/token_merger/co_me_2d.py:268-298``)
    and of ``CoMe_TokenMerger.build_ctx`` (``src/accelerate/token_merger/co_me.py:54-73``):

    * ``pairwise-rank``: ``mask = mean < quantile(mean.float(), threshold)``; the quantile is taken over all
      ``S*M`` windows of a batch element (``scope="batch"``, the 2-D class) or over the ``M`` windows of a frame
      (``scope="frame"``, the 1-D class and the standalone op-chain configuration);
    * ``abs_mse``: ``mask = mean < threshold``;
    * ``mse``: confidences are z-normalised per batch element (unbiased std, ``+1e-3``) before the window mean.
    """
    conf = np.asarray(conf, dtype=np.float32).reshape(B, S * H * W)
    if mode == "mse":
        conf = z_normalise(conf, kind)
    means = window_means(conf.reshape(B * S, H * W), H, W, gh, gw, kind)  # [B*S, M]
    M = means.shape[1]
    if mode in ("abs_mse", "mse"):
        # a tensor compared with a Python number: the number is first rounded to the tensor's dtype
        return means < _round_like(np.float32(threshold), kind)
    if mode != "pairwise-rank":
        raise ValueError(mode)
    per_group = np.ndim(threshold) > 0  # one quantile level per group (per-frame merge ratios of the ragged batch)
    if not per_group and not (0.0 <= threshold <= 1.0):
        raise ValueError(f"Ranking mode requires threshold in [0, 1], got {threshold}")
    if scope == "batch":
        grouped = means.reshape(B, S * M)
    elif scope == "frame":
        grouped = means.reshape(B * S, M)
    else:
        raise ValueError(scope)
    levels = np.clip(np.asarray(threshold, np.float32), 0.0, 1.0) if per_group else np.full(len(grouped), threshold)
    thr = np.array([quantile_linear(row, q) for row, q in zip(grouped, levels)], dtype=np.float32)
    return (grouped < thr[:, None]).reshape(B * S, M)


# --------------------------------------------------------------------------------------------------------
# biased variable-length attention
# --------------------------------------------------------------------------------------------------------
def perkey_bias_from_weight(weight: np.ndarray, kind: str = "bf16") -> np.ndarray:
    """``log(weight)`` rounded to the run dtype (``src/accelerate/vggt/module/bias_attention.py:120``)."""
    return _round_like(np.log(np.asarray(weight, dtype=np.float32)), kind)


def max_seqlen(cu_seqlens: np.ndarray) -> int:
    """``infer_flash_attn_varlen_max_seqlen`` (``src/cuda_extension/flash_attn/__init__.py:21-33``)."""
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    return int((cu[1:] - cu[:-1]).max()) if cu.size > 1 else 0


def attention_bias(q, k, v, bias, cu_seqlens, scale):
    """fp32 biased softmax attention per segment and head.

    Restates the reference's test oracle ``_reference_attention_with_bias``
    (``test/auto_test/test_flex_attention_bias.py:26-36``):
    ``softmax(q @ k.T * scale + bias[None, :]) @ v`` for every packed segment ``[cu[i], cu[i+1])`` and head,
    which is what the device kernel computes (``src/cuda_extension/flash_attn/src/flash_fwd_kernel.h:30-55``).

    q, k, v ``[P, H, D]`` float32; bias ``[P]`` float32 or ``None``; returns ``(out[P,H,D], lse[H,P])`` float32.
    """
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k, dtype=np.float32)
    v = np.asarray(v, dtype=np.float32)
    P, Hh, D = q.shape
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    out = np.zeros((P, Hh, D), dtype=np.float32)
    lse = np.full((Hh, P), np.inf, dtype=np.float32)
    for i in range(cu.size - 1):
        s, e = int(cu[i]), int(cu[i + 1])
        if e <= s:
            continue
        b = np.zeros(e - s, np.float32) if bias is None else np.asarray(bias[s:e], dtype=np.float32)
        for h in range(Hh):
            logits = (q[s:e, h, :] @ k[s:e, h, :].T) * np.float32(scale) + b[None, :]
            m = logits.max(axis=-1, keepdims=True)
            p = np.exp(logits - m)
            l = p.sum(axis=-1, keepdims=True)
            out[s:e, h, :] = (p / l) @ v[s:e, h, :]
            lse[h, s:e] = (m + np.log(l))[:, 0]
    return out, lse


def attention_combine(out_a, lse_a, out_b, lse_b):
    """Merge of two attention results of the same query rows over disjoint key sets: with ``w_x = exp(lse_x - m)``,
    ``m = max(lse_a, lse_b)``: ``out = (w_a out_a + w_b out_b) / (w_a + w_b)``, ``lse = m + log(w_a + w_b)``.
    ``out_* [rows, H, D]``, ``lse_* [H, rows]``; float32.  (Identity of the softmax over a union of key sets; the
    reference has no such step, it never splits the keys.)"""
    la, lb = np.asarray(lse_a, np.float32).T[:, :, None], np.asarray(lse_b, np.float32).T[:, :, None]
    m = np.maximum(la, lb)
    wa, wb = np.exp(la - m, dtype=np.float32), np.exp(lb - m, dtype=np.float32)
    out = (wa * np.asarray(out_a, np.float32) + wb * np.asarray(out_b, np.float32)) / (wa + wb)
    return out.astype(np.float32), (m + np.log(wa + wb))[:, :, 0].T.astype(np.float32)


def attention_combine_parts(outs, lses):
    """The same merge for any number of results: ``outs [S, rows, H, D]``, ``lses [S, H, rows]`` -> ``(out [rows, H, D],
    lse [H, rows])`` with ``m = max_s lse_s``, ``w_s = exp(lse_s - m)``, ``out = sum_s w_s out_s / sum_s w_s`` (shares summed
    in index order), ``lse = m + log(sum_s w_s)``; float32."""
    outs, lses = np.asarray(outs, np.float32), np.asarray(lses, np.float32)
    l = np.transpose(lses, (0, 2, 1))[:, :, :, None]  # [S, rows, H, 1]
    m = l.max(axis=0)
    acc = np.zeros(outs.shape[1:], np.float32)
    wsum = np.zeros(m.shape, np.float32)
    for s in range(outs.shape[0]):
        w = np.exp(l[s] - m, dtype=np.float32)
        acc = acc + w * outs[s]
        wsum = wsum + w
    return (acc / wsum).astype(np.float32), (m + np.log(wsum))[:, :, 0].T.astype(np.float32)


# --------------------------------------------------------------------------------------------------------
# pre-attention preparation of the packed qkv tensor: q/k LayerNorm over the head dimension, 2-D rotary
# position embedding, per-key bias
# --------------------------------------------------------------------------------------------------------
def rope_tables(feature_dim: int, max_position: int, base_frequency: float = 100.0, kind: str = "bf16"):
    """cos / sin tables ``[max_position, feature_dim]`` of the 1-D rotary embedding, in the run dtype.

    ``RotaryPositionEmbedding2D._compute_frequency_components``
    (``src/thirdparty/vggt/layers/rope.py:87-114``): ``inv_freq = 1 / base ** (arange(0, dim, 2) / dim)`` in
    float32, ``angles = position * inv_freq`` in float32, ROUNDED TO THE RUN DTYPE, duplicated along the last
    axis, then cos / sin evaluated and rounded to the run dtype again.
    """
    exponents = np.arange(0, feature_dim, 2, dtype=np.float32) / np.float32(feature_dim)
    inv_freq = (np.float32(1.0) / np.power(np.float32(base_frequency), exponents, dtype=np.float32)).astype(np.float32)
    positions = np.arange(max_position, dtype=np.float32)
    angles = _round_like((positions[:, None] * inv_freq[None, :]).astype(np.float32), kind)
    angles = np.concatenate([angles, angles], axis=-1)
    return _round_like(np.cos(angles, dtype=np.float32), kind), _round_like(np.sin(angles, dtype=np.float32), kind)


def _sum_lanes_of_8(x: np.ndarray) -> np.ndarray:
    """Float32 sum over the last axis (a power of two >= 8) in a fixed order: inside each run of 8 consecutive
    elements the even-indexed and the odd-indexed elements are summed left to right as two chains and the two
    chains added; then a pairwise tree over the runs.  The order is part of the oracle's definition so that the
    CUDA kernel (8 elements per lane summed with packed two-lane adds, butterfly over lanes) can be compared bit
    for bit; any other order moves a result by at most one rounding."""
    D = x.shape[-1]
    r = x.reshape(x.shape[:-1] + (D // 8, 4, 2)).astype(np.float32)
    acc = r[..., 0, :].copy()
    for i in range(1, 4):
        acc = (acc + r[..., i, :]).astype(np.float32)
    acc = (acc[..., 0] + acc[..., 1]).astype(np.float32)
    while acc.shape[-1] > 1:
        acc = (acc[..., 0::2] + acc[..., 1::2]).astype(np.float32)
    return acc[..., 0]


def _fma32(a: np.ndarray, b: np.ndarray, c: np.ndarray) -> np.ndarray:
    """Fused multiply-add of float32 values: the product of two float32 is exact in float64, so only the final
    float64 -> float32 conversion can round twice (odds ~2^-29 per operation, and then by one float32 ulp)."""
    return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(np.float32)


def _sumsq_lanes_of_8(d: np.ndarray) -> np.ndarray:
    """Sum of squares in the order of :func:`_sum_lanes_of_8`, each chain accumulated with fused multiply-adds:
    ``acc = d0 * d0`` (rounded), then ``acc = fma(d_i, d_i, acc)``."""
    D = d.shape[-1]
    r = d.reshape(d.shape[:-1] + (D // 8, 4, 2)).astype(np.float32)
    acc = (r[..., 0, :] * r[..., 0, :]).astype(np.float32)
    for i in range(1, 4):
        acc = _fma32(r[..., i, :], r[..., i, :], acc)
    acc = (acc[..., 0] + acc[..., 1]).astype(np.float32)
    while acc.shape[-1] > 1:
        acc = (acc[..., 0::2] + acc[..., 1::2]).astype(np.float32)
    return acc[..., 0]


def layer_norm_heads(x: np.ndarray, gamma: np.ndarray, beta: np.ndarray, eps: float, kind: str = "bf16"):
    """``nn.LayerNorm(head_dim)`` applied to ``x[..., D]`` held in the run dtype (``q_norm`` / ``k_norm`` of
    the attention module, called at ``src/accelerate/common/qkv.py:30-31``).

    Statistics and the affine map are evaluated in float32 (as PyTorch does for 16-bit inputs):
    ``mean = sum(x) / D``, ``var = sum((x - mean)^2) / D`` (two passes), ``rstd = 1 / sqrt(var + eps)``,
    ``y = fma(gamma, rstd * (x - mean), beta)``, then rounded to the run dtype.  PyTorch's own kernels order the
    sums differently (and differently on CPU and GPU), which moves a result by at most one unit in the last place
    of the run dtype; the order chosen here is the CUDA kernel's, so that the two compare bit for bit.
    """
    x = x.astype(np.float32)
    D = x.shape[-1]
    inv_d = np.float32(1.0) / np.float32(D)  # exact: D is a power of two
    mean = (_sum_lanes_of_8(x) * inv_d).astype(np.float32)
    d = (x - mean[..., None]).astype(np.float32)
    var = (_sumsq_lanes_of_8(d) * inv_d).astype(np.float32)
    rstd = (np.float32(1.0) / np.sqrt((var + np.float32(eps)).astype(np.float32))).astype(np.float32)
    y = (rstd[..., None] * d).astype(np.float32)
    y = _fma32(np.broadcast_to(gamma.astype(np.float32), y.shape), y, np.broadcast_to(beta.astype(np.float32), y.shape))
    return _round_like(y, kind)


def _row_total(part: np.ndarray) -> np.ndarray:
    """Total of per-thread partial sums ``part[..., threads]`` (threads a multiple of 32) in the order of the fused
    LayerNorm + merge kernel: for every lane position the partials of the group's warps are added left to right, then a
    pairwise tree runs over the 32 lane positions (neighbours first)."""
    t = part.reshape(part.shape[:-1] + (part.shape[-1] // 32, 32)).astype(np.float32)
    acc = t[..., 0, :].copy()
    for w in range(1, t.shape[-2]):
        acc = (acc + t[..., w, :]).astype(np.float32)
    while acc.shape[-1] > 1:
        acc = (acc[..., 0::2] + acc[..., 1::2]).astype(np.float32)
    return acc[..., 0]


def layer_norm_rows(x: np.ndarray, gamma: np.ndarray, beta: np.ndarray, eps: float, kind: str = "bf16"):
    """``nn.LayerNorm(C)`` over the channels of dense tokens ``x[..., C]`` held in the element type ``kind`` -- the
    block's ``norm1`` in front of the attention (``src/thirdparty/vggt/layers/block.py:73``), whose output the per-layer
    mode merges (``src/accelerate/vggt/direct.py:97-101``).

    float32 statistics and affine map, result rounded to the element type: ``mean = sum(x) / C``,
    ``var = sum((x - mean)^2) / C`` (two passes, squares accumulated by fused multiply-adds),
    ``rstd = 1 / sqrt(var + eps)``, ``y = fma(gamma, rstd * (x - mean), beta)``.  The sums run in the fused CUDA kernel's
    order: a thread owns 16 bytes of consecutive channels, whose even and odd members are summed left to right as two
    chains and the chains added; threads are padded to a power of two >= 32, then :func:`_row_total`.  PyTorch's kernels
    use other orders, which moves a result by at most one unit in the last place of the element type.
    """
    x = x.astype(np.float32)
    C = x.shape[-1]
    vec = 4 if kind == "f32" else 8
    assert C % vec == 0
    cv = C // vec
    threads = 32
    while threads < cv:
        threads *= 2
    lead = x.shape[:-1]

    def per_thread(v, square):
        r = v.reshape(lead + (cv, vec // 2, 2))
        if square:
            acc = (r[..., 0, :] * r[..., 0, :]).astype(np.float32)
            for i in range(1, vec // 2):
                acc = _fma32(r[..., i, :], r[..., i, :], acc)
        else:
            acc = r[..., 0, :].copy()
            for i in range(1, vec // 2):
                acc = (acc + r[..., i, :]).astype(np.float32)
        out = np.zeros(lead + (threads,), np.float32)
        out[..., :cv] = (acc[..., 0] + acc[..., 1]).astype(np.float32)
        return out

    fC = np.float32(C)
    mean = (_row_total(per_thread(x, False)) / fC).astype(np.float32)
    d = (x - mean[..., None]).astype(np.float32)
    var = (_row_total(per_thread(d, True)) / fC).astype(np.float32)
    rstd = (np.float32(1.0) / np.sqrt((var + np.float32(eps)).astype(np.float32))).astype(np.float32)
    y = (rstd[..., None] * d).astype(np.float32)
    y = _fma32(np.broadcast_to(gamma.astype(np.float32), y.shape), y, np.broadcast_to(beta.astype(np.float32), y.shape))
    return _round_like(y, kind)


def residual_layer_norm(x, branch, scale, gamma, beta, eps: float, kind: str = "bf16"):
    """``x = x + ls(branch)`` followed by ``norm(x)`` on packed rows, the pair of steps between two sub-blocks of the
    jagged block (``src/accelerate/vggt/module/block.py:66-79``): LayerScale ``branch * scale``
    (``src/thirdparty/vggt/layers/layer_scale.py:21-22``) rounded to the element type, the residual sum rounded to the
    element type, then :func:`layer_norm_rows` of the result.  ``branch`` None: the norm of ``x`` alone; ``scale`` None:
    no LayerScale; ``gamma`` None: no norm.  Returns ``(x_out, normed)`` (``normed`` None without a norm)."""
    x_out = np.asarray(x, np.float32)
    if branch is not None:
        t = np.asarray(branch, np.float32)
        if scale is not None:
            t = _round_like((t * np.asarray(scale, np.float32)).astype(np.float32), kind)
        x_out = _round_like((x_out + t).astype(np.float32), kind)
    normed = None if gamma is None else layer_norm_rows(x_out, np.asarray(gamma, np.float32), np.asarray(beta, np.float32), eps, kind)
    return x_out, normed


def rope_2d(x: np.ndarray, pos: np.ndarray, cos_t: np.ndarray, sin_t: np.ndarray, kind: str = "bf16"):
    """2-D rotary embedding of ``x[P, H, D]`` with integer positions ``pos[P, 2]`` (y, x).

    ``RotaryPositionEmbedding2D.forward`` / ``_apply_1d_rope`` / ``_rotate_features``
    (``src/thirdparty/vggt/layers/rope.py:116-187``): the first ``D/2`` features rotate with the y position,
    the second ``D/2`` with the x position; inside a half, ``out = t * cos + rot(t) * sin`` with
    ``rot(t) = cat(-t[D/4:], t[:D/4])``.  All three operations happen in the run dtype, i.e. each result is
    rounded to it.
    """
    x = x.astype(np.float32)
    P, H, D = x.shape
    half, quarter = D // 2, D // 4
    out = np.empty_like(x)
    for axis in range(2):
        t = x[:, :, axis * half:(axis + 1) * half]
        rot = np.concatenate([-t[..., quarter:], t[..., :quarter]], axis=-1)
        c = cos_t[pos[:, axis]][:, None, :]
        s = sin_t[pos[:, axis]][:, None, :]
        a = _round_like((t * c).astype(np.float32), kind)
        b = _round_like((rot * s).astype(np.float32), kind)
        out[:, :, axis * half:(axis + 1) * half] = _round_like((a + b).astype(np.float32), kind)
    return out


def qkv_prepare(qkv, q_gamma, q_beta, k_gamma, k_beta, eps, pos, cos_t, sin_t, kind="bf16"):
    """``prepare_packed_self_attention_qkv`` without gradients (``src/accelerate/common/qkv.py:29-39``):
    q and k of the packed ``[P, 3, H, D]`` tensor are layer-normalised over ``D`` (skipped when ``gamma`` is
    None, the ``nn.Identity`` case), then rotated (skipped when ``pos`` is None); v is untouched."""
    out = np.array(qkv, dtype=np.float32, copy=True)
    for j, (g, b) in enumerate(((q_gamma, q_beta), (k_gamma, k_beta))):
        y = out[:, j]
        if g is not None:
            y = layer_norm_heads(y, g, b, eps, kind)
        if pos is not None:
            y = rope_2d(y, pos, cos_t, sin_t, kind)
        out[:, j] = y
    return out


def packed_positions(mask: np.ndarray, start_index: int, H: int, W: int, gh: int, gw: int) -> np.ndarray:
    """Integer (y, x) position of every packed row after the merge, ``[P, 2]`` int64.

    ``src/accelerate/vggt/fused.py:113-129``: special tokens sit at (0, 0), patch (y, x) at (y + 1, x + 1);
    the position tensor is merged like the features in bfloat16 and truncated with ``.long()``.  The mean of
    a ``gh x gw`` window of integer coordinates is ``first + (g - 1) / 2`` per axis; this function evaluates
    exactly what the reference evaluates (float32 sum, division by the window size, bfloat16 rounding,
    truncation) on the ragged layout.
    """
    mask = np.asarray(mask, dtype=bool)
    B = mask.shape[0]
    ys, xs = np.meshgrid(np.arange(H), np.arange(W), indexing="ij")
    p = np.zeros((start_index + H * W, 2), np.float32)
    p[start_index:, 0] = ys.reshape(-1) + 1
    p[start_index:, 1] = xs.reshape(-1) + 1
    pos = np.broadcast_to(p, (B,) + p.shape)
    merged, _off, _rev, _w = token_merge_2d_ragged(_round_like(pos, "bf16"), start_index, gh, gw, H, W, mask)
    return np.trunc(_round_like(merged, "bf16")).astype(np.int64)


# --------------------------------------------------------------------------------------------------------
# transformer block over packed tokens and the merged forward pass of the alternating-attention aggregator
# --------------------------------------------------------------------------------------------------------
def gelu_erf(x: np.ndarray) -> np.ndarray:
    """``nn.GELU()`` with its default exact form ``0.5 * x * (1 + erf(x / sqrt(2)))`` (the activation of the MLP,
    ``src/thirdparty/vggt/layers/mlp.py:18,31``), evaluated in float64 and returned as float32."""
    from math import erf
    x64 = np.asarray(x, dtype=np.float64)
    return (0.5 * x64 * (1.0 + np.vectorize(erf, otypes=[np.float64])(x64 / np.sqrt(2.0)))).astype(np.float32)


def _layer_norm_f32(x: np.ndarray, gamma: np.ndarray, beta: np.ndarray, eps: float) -> np.ndarray:
    x64 = np.asarray(x, dtype=np.float64)
    mean = x64.mean(axis=-1, keepdims=True)
    var = ((x64 - mean) ** 2).mean(axis=-1, keepdims=True)
    return ((x64 - mean) / np.sqrt(var + eps) * gamma.astype(np.float64) + beta.astype(np.float64)).astype(np.float32)


def jagged_block(x, weight, cu_seqlens, pos, p, num_heads, cos_t, sin_t, use_bias=True):
    """One transformer block on packed tokens ``x [P, C]``: ``JaggedBlock_w_Bias.forward``
    (``src/accelerate/vggt/module/block.py:58-81``) around ``JaggedAttention_w_Bias.forward``
    (``src/accelerate/vggt/module/bias_attention.py:100-137``):

        x = x + ls1 * proj(attention(prepare(qkv(norm1(x))), bias = log(weight)))
        x = x + ls2 * fc2(gelu(fc1(norm2(x))))

    in float32 throughout (the reference rounds the attention branch to bfloat16; the difference is what the
    tolerance of a comparison against this function has to cover).  ``p`` maps parameter names to float32 arrays:
    ``norm1.weight/bias, attn.qkv.weight/bias, attn.q_norm.weight/bias, attn.k_norm.weight/bias, attn.proj.weight/bias,
    ls1.gamma, norm2.weight/bias, mlp.fc1.weight/bias, mlp.fc2.weight/bias, ls2.gamma`` (the norm and LayerScale
    entries may be absent), plus ``eps`` values ``norm_eps`` and ``qk_norm_eps``.  ``cos_t`` / ``sin_t`` are the rotary
    tables of :func:`rope_tables` (None: no rotary embedding); ``use_bias=False`` gives the block without the count
    bias (``block.py:18-43``).
    """
    x = np.asarray(x, dtype=np.float32)
    P, C = x.shape
    D = C // num_heads
    eps = float(p.get("norm_eps", 1e-5))
    h = _layer_norm_f32(x, p["norm1.weight"], p["norm1.bias"], eps)
    qkv = (h @ p["attn.qkv.weight"].T + p["attn.qkv.bias"]).astype(np.float32).reshape(P, 3, num_heads, D)
    has_qk_norm = "attn.q_norm.weight" in p
    qkv = qkv_prepare(qkv, p.get("attn.q_norm.weight"), p.get("attn.q_norm.bias"), p.get("attn.k_norm.weight"),
                      p.get("attn.k_norm.bias"), float(p.get("qk_norm_eps", 1e-5)) if has_qk_norm else 0.0,
                      pos if cos_t is not None else None, cos_t, sin_t, kind="f32")
    bias = np.log(np.asarray(weight, dtype=np.float32)) if use_bias else None
    out, _ = attention_bias(qkv[:, 0], qkv[:, 1], qkv[:, 2], bias, cu_seqlens, D ** -0.5)
    out = (out.reshape(P, C) @ p["attn.proj.weight"].T + p["attn.proj.bias"]).astype(np.float32)
    x = x + out * p.get("ls1.gamma", np.float32(1.0))
    h = _layer_norm_f32(x, p["norm2.weight"], p["norm2.bias"], eps)
    h = gelu_erf(h @ p["mlp.fc1.weight"].T + p["mlp.fc1.bias"])
    h = (h @ p["mlp.fc2.weight"].T + p["mlp.fc2.bias"]).astype(np.float32)
    return (x + h * p.get("ls2.gamma", np.float32(1.0))).astype(np.float32)


def fused_aggregator(tokens, mask, start_index, H, W, gh, gw, frame_params, global_params, num_heads, retain_layers=None,
                     aa_order=("frame", "global"), aa_block_size=1, rope_base=100.0, rope_kind="bf16",
                     use_bias=True):
    """Merged forward pass of the aggregator (``src/accelerate/vggt/fused.py:95-167``): merge the dense tokens
    ``[B, S, N, C]`` once, run the alternating frame / global blocks on the packed tokens -- frame blocks attend inside
    a frame, global blocks inside a scene (``fused.py:141-149``) -- and unmerge the retained layers to
    ``[B, S, N, 2C]`` (frame tokens and global tokens side by side, ``fused.py:157-167``).  ``frame_params`` /
    ``global_params`` are lists of the dictionaries :func:`jagged_block` takes; ``rope_base <= 0`` disables the
    rotary embedding; its tables are built in ``rope_kind`` as the model does in its run dtype.
    Returns ``{block index: array}``."""
    tokens = np.asarray(tokens, dtype=np.float32)
    B, S, N, C = tokens.shape
    mask = np.asarray(mask, dtype=bool)
    x, offsets, rev, weight = token_merge_2d_ragged(tokens.reshape(B * S, N, C), start_index, gh, gw, H, W, mask)
    pos = packed_positions(mask, start_index, H, W, gh, gw)
    cos_t = sin_t = None
    if rope_base > 0:
        cos_t, sin_t = rope_tables(C // num_heads // 2, int(max(H, W)) + 2, rope_base, rope_kind)
    frame_cu = np.asarray(offsets, dtype=np.int64)
    global_cu = frame_cu[::S]
    depth = len(frame_params)
    block_idx = frame_idx = globe_idx = 0
    output = {}
    for _ in range(depth // aa_block_size):
        frame_mid, globe_mid = [], []
        for kind in aa_order:
            for _ in range(aa_block_size):
                if kind == "frame":
                    x = jagged_block(x, weight, frame_cu, pos, frame_params[frame_idx], num_heads, cos_t, sin_t, use_bias)
                    frame_mid.append(x)
                    frame_idx += 1
                elif kind == "global":
                    x = jagged_block(x, weight, global_cu, pos, global_params[globe_idx], num_heads, cos_t, sin_t, use_bias)
                    globe_mid.append(x)
                    globe_idx += 1
                else:
                    raise ValueError(f"Unknown attention type: {kind}")
        for i in range(aa_block_size):
            if retain_layers is None or block_idx in retain_layers:
                both = np.concatenate([token_split(frame_mid[i], rev), token_split(globe_mid[i], rev)], axis=-1)
                output[block_idx] = both.reshape(B, S, N, 2 * C)
            block_idx += 1
    return output


def patch_embed(images, proj_weight, proj_bias, cls_token, register_tokens, pos_embed, patch: int):
    """Patch embedding of a ViT with register tokens (``src/thirdparty/vggt/layers/vision_transformer.py``
    ``prepare_tokens_with_masks``): non-overlapping ``patch x patch`` convolution, class token in front, learned position
    embedding added to class + patch tokens, register tokens inserted behind the class token.
    ``images [F, 3, H, W]`` -> ``[F, 1 + R + h*w, C]`` float32."""
    images = np.asarray(images, np.float32)
    Fr, Cin, Hh, Ww = images.shape
    h, w = Hh // patch, Ww // patch
    x = images[:, :, : h * patch, : w * patch].reshape(Fr, Cin, h, patch, w, patch).transpose(0, 2, 4, 1, 3, 5).reshape(Fr, h * w, -1)
    Wm = np.asarray(proj_weight, np.float32).reshape(proj_weight.shape[0], -1)  # [C, 3 * patch * patch]
    tok = (x @ Wm.T + np.asarray(proj_bias, np.float32)).astype(np.float32)
    tok = np.concatenate([np.broadcast_to(cls_token, (Fr,) + cls_token.shape[1:]), tok], axis=1) + pos_embed
    reg = np.broadcast_to(register_tokens, (Fr,) + register_tokens.shape[1:])
    return np.concatenate([tok[:, :1], reg, tok[:, 1:]], axis=1).astype(np.float32)


def fused_model(images, enc, enc_params, encoder_layer, head, agg_tokens, frame_params, global_params, num_heads, gh, gw,
                threshold, retain_layers=None, rope_base=100.0, rope_kind="bf16", conf_kind="bf16", mask=None):
    """The accelerated model from images to the retained aggregator layers (``src/accelerate/vggt/fused.py:40-94`` around
    :func:`fused_aggregator`), float32: encoder blocks ``0 .. encoder_layer`` dense, confidence -> window selection over
    the scene (``co_me_2d.py:268-298``) -> merge, encoder blocks ``encoder_layer + 1 ..`` on the packed tokens with the
    count bias, split, final norm, camera / register tokens of the aggregator in front of the patch tokens, merged
    forward pass of the aggregator with the same mask.

    ``enc``: dict with ``proj.weight / proj.bias / cls_token / register_tokens / pos_embed / norm.weight / norm.bias``,
    ``patch``, ``norm_eps``; ``enc_params``: list of block dictionaries (:func:`jagged_block`); ``head``: the two-layer
    confidence MLP ``fc1.weight/bias, fc2.weight/bias``; ``agg_tokens``: ``camera_token [1,2,1,C]``, ``register_token
    [1,2,R,C]``.  ``mask`` (optional) overrides the selection (a device run may select in lower precision).
    Returns ``(layers, mask)``."""
    images = np.asarray(images, np.float32)
    B, S = images.shape[:2]
    x = patch_embed(images.reshape((B * S,) + images.shape[2:]), enc["proj.weight"], enc["proj.bias"], enc["cls_token"],
                    enc["register_tokens"], enc["pos_embed"], enc["patch"])
    Fr, N, C = x.shape
    start = 1 + enc["register_tokens"].shape[1]
    h, w = images.shape[3] // enc["patch"], images.shape[4] // enc["patch"]
    ones = np.ones(Fr * N, np.float32)
    cu = np.arange(0, Fr * N + 1, N, dtype=np.int64)
    flat = x.reshape(Fr * N, C)
    for p in enc_params[: encoder_layer + 1]:
        flat = jagged_block(flat, ones, cu, None, p, num_heads, None, None, use_bias=False)
    dense = flat.reshape(Fr, N, C)
    if mask is None:
        feat = _round_like(dense[:, start:], conf_kind)
        hid = gelu_erf(feat @ head["fc1.weight"].T + head["fc1.bias"])
        conf = (hid @ head["fc2.weight"].T + head["fc2.bias"]).reshape(B, S * h * w)
        mask = select_windows(_round_like(conf, conf_kind), B, S, h, w, gh, gw, threshold, "pairwise-rank", "batch", conf_kind)
    merged, offsets, rev, weight = token_merge_2d_ragged(dense, start, gh, gw, h, w, mask)
    for p in enc_params[encoder_layer + 1:]:
        merged = jagged_block(merged, weight, np.asarray(offsets, np.int64), None, p, num_heads, None, None, use_bias=True)
    dense = token_split(merged, rev).reshape(Fr, N, C)
    dense = _layer_norm_f32(dense, enc["norm.weight"], enc["norm.bias"], float(enc.get("norm_eps", 1e-6)))

    def expand(tok):  # [1, 2, X, C] -> [B*S, X, C]
        first = np.broadcast_to(tok[:, 0:1], (B, 1) + tok.shape[2:])
        rest = np.broadcast_to(tok[:, 1:2], (B, S - 1) + tok.shape[2:])
        return np.concatenate([first, rest], axis=1).reshape((B * S,) + tok.shape[2:])

    tokens = np.concatenate([expand(agg_tokens["camera_token"]), expand(agg_tokens["register_token"]), dense[:, start:]], axis=1)
    layers = fused_aggregator(tokens.reshape(B, S, N, C), mask, start, h, w, gh, gw, frame_params, global_params, num_heads,
                              retain_layers, rope_base=rope_base, rope_kind=rope_kind)
    return layers, mask


# --------------------------------------------------------------------------------------------------------
# suffix tokens of jagged segments
# --------------------------------------------------------------------------------------------------------
def jagged_add_suffix(tokens, weight, offset, suffix):
    """``JaggedTokens.add_suffix`` (``src/interface/token_merger.py:23-58``): segment ``m`` of the packed ``tokens [P, C]``
    is followed by its ``T`` rows of ``suffix [M, T, C]``, each with weight 1.  Returns ``(tokens, weight, offset)``."""
    tokens, weight = np.asarray(tokens), np.asarray(weight)
    offset = np.asarray(offset, dtype=np.int64)
    M, T = suffix.shape[0], suffix.shape[1]
    if M != offset.size - 1:
        raise ValueError(f"suffix batch dim ({M}) must match segment count ({offset.size - 1})")
    rows, wts = [], []
    for m in range(M):
        rows += [tokens[offset[m]:offset[m + 1]], np.asarray(suffix[m], dtype=tokens.dtype)]
        wts += [weight[offset[m]:offset[m + 1]], np.ones(T, dtype=weight.dtype)]
    C = tokens.shape[1]
    return (np.concatenate(rows, axis=0) if rows else np.zeros((0, C), tokens.dtype),
            np.concatenate(wts) if wts else np.zeros(0, weight.dtype), offset + np.arange(M + 1, dtype=np.int64) * T)


def jagged_split_suffix(tokens, weight, offset, count: int):
    """``JaggedTokens.split_suffix`` (``src/interface/token_merger.py:60-100``): the inverse of
    :func:`jagged_add_suffix`.  Returns ``(tokens, weight, offset, suffix [M, count, C])``; ``ValueError`` when a
    segment is shorter than ``count``."""
    tokens, weight = np.asarray(tokens), np.asarray(weight)
    offset = np.asarray(offset, dtype=np.int64)
    M, T, C = offset.size - 1, int(count), tokens.shape[1]
    if tokens.shape[0] - M * T < 0:
        raise ValueError(f"Cannot strip {T} tokens from each of {M} segments (total tokens = {tokens.shape[0]})")
    new_offset = offset - np.arange(M + 1, dtype=np.int64) * T
    if np.any(np.diff(new_offset) < 0):
        raise ValueError(f"count={T} exceeds the length of at least one segment")
    keep = [tokens[offset[m]:offset[m + 1] - T] for m in range(M)]
    wts = [weight[offset[m]:offset[m + 1] - T] for m in range(M)]
    suffix = np.stack([tokens[offset[m + 1] - T:offset[m + 1]] for m in range(M)]) if M else np.zeros((0, T, C), tokens.dtype)
    return (np.concatenate(keep, axis=0) if keep else np.zeros((0, C), tokens.dtype),
            np.concatenate(wts) if wts else np.zeros(0, weight.dtype), new_offset, suffix)
