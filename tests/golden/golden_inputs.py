"""Seeded input generators shared by ``make_golden.py`` (which runs the reference on them) and by the tests
(which feed the same inputs to the oracle and to the CUDA library and compare with the stored outputs).

All randomness comes from ``numpy.random.default_rng`` so that no reference checkout is needed to rebuild an
input.  Values meant for a 16-bit dtype are rounded here and carried as float32.
"""
from __future__ import annotations

import numpy as np


def round_bf16(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return (r & 0xFFFFFFFF).astype(np.uint32).view(np.float32)


def round_kind(x: np.ndarray, kind: str) -> np.ndarray:
    if kind == "f32":
        return np.ascontiguousarray(x, dtype=np.float32)
    if kind == "bf16":
        return round_bf16(x)
    if kind == "f16":
        return x.astype(np.float16).astype(np.float32)
    raise ValueError(kind)


def summarize_rows(a: np.ndarray, stride: int = 251) -> dict:
    """Compact fingerprint of a float matrix: exact per-row float64 sums, and every ``stride``-th row in full
    (small matrices are kept whole)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    if a.size <= 1 << 15:
        return {"full": a}
    return {"rowsum": a.astype(np.float64).sum(axis=1), "sample": a[::stride].copy(),
            "stride": np.asarray(stride)}


def check_rows(a: np.ndarray, store, prefix: str, rtol: float = 0.0, atol: float = 0.0) -> None:
    """Assert that ``a`` matches the fingerprint written by :func:`summarize_rows` (bit for bit by default;
    the row sums get the element tolerance times the row length)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    if prefix + "full" in store:
        np.testing.assert_allclose(a, store[prefix + "full"], rtol=rtol, atol=atol)
        return
    n = a.shape[1]
    np.testing.assert_allclose(a.astype(np.float64).sum(axis=1), store[prefix + "rowsum"], rtol=rtol,
                               atol=n * (atol + rtol * float(np.abs(a).max())))
    np.testing.assert_allclose(a[:: int(store[prefix + "stride"])], store[prefix + "sample"], rtol=rtol, atol=atol)


# ---- merge ------------------------------------------------------------------------------------------------
def merge1d_inputs(i: int, cfg, kind: str = "f32"):
    B, M, G, S, C = cfg
    rng = np.random.default_rng(4200 + i)
    tokens = round_kind(rng.standard_normal((B, S + M * G, C), dtype=np.float32), kind)
    ratio = rng.uniform(0.1, 0.9)
    mask = rng.random((B, M)) < ratio
    return tokens, mask


def merge2d_inputs(i: int, cfg):
    B, H, W, gh, gw, S, C = cfg
    rng = np.random.default_rng(4300 + i)
    tokens = rng.standard_normal((B, S + H * W, C), dtype=np.float32)
    mask = rng.random((B, (H // gh) * (W // gw))) < 0.5
    return tokens, mask


# ---- selection ---------------------------------------------------------------------------------------------
SELECT_CASES = {
    # name: batch, frames, grid, window, threshold, mode, merger class ("2d": quantile over the whole batch
    # element, "1d": per frame over consecutive groups), confidence dtype
    "rank2d_bf16": dict(B=1, S=8, H=36, W=36, gh=3, gw=3, thr=0.5, mode="pairwise-rank", cls="2d", kind="bf16"),
    "rank2d_b2_f32": dict(B=2, S=4, H=12, W=12, gh=3, gw=3, thr=0.3, mode="pairwise-rank", cls="2d", kind="f32"),
    "rank2d_2x3_bf16": dict(B=2, S=3, H=8, W=12, gh=2, gw=3, thr=0.75, mode="pairwise-rank", cls="2d", kind="bf16"),
    "rank2d_thr0": dict(B=1, S=2, H=6, W=6, gh=3, gw=3, thr=0.0, mode="pairwise-rank", cls="2d", kind="bf16"),
    "rank2d_thr1": dict(B=1, S=2, H=6, W=6, gh=3, gw=3, thr=1.0, mode="pairwise-rank", cls="2d", kind="bf16"),
    "rank2d_100f_bf16": dict(B=1, S=100, H=36, W=36, gh=3, gw=3, thr=0.5, mode="pairwise-rank", cls="2d", kind="bf16"),
    "abs2d_bf16": dict(B=2, S=2, H=9, W=9, gh=3, gw=3, thr=0.45, mode="abs_mse", cls="2d", kind="bf16"),
    # a threshold that is not a bfloat16 number: the comparison rounds it to the tensor's dtype first
    "abs2d_thr_rounded_bf16": dict(B=1, S=3, H=36, W=36, gh=3, gw=3, thr=0.501, mode="abs_mse", cls="2d", kind="bf16"),
    # z-normalised mode: (x - mean) / (std + 1e-3) per batch element, then the window mean against the threshold
    "mse2d_bf16": dict(B=2, S=4, H=36, W=36, gh=3, gw=3, thr=-0.2, mode="mse", cls="2d", kind="bf16"),
    "mse2d_f16": dict(B=1, S=5, H=12, W=18, gh=2, gw=3, thr=0.31, mode="mse", cls="2d", kind="f16"),
    "mse2d_f32": dict(B=2, S=3, H=12, W=12, gh=3, gw=3, thr=0.0, mode="mse", cls="2d", kind="f32"),
    "mse1d_bf16": dict(B=2, S=3, H=6, W=18, gh=1, gw=9, thr=0.1, mode="mse", cls="1d", kind="bf16"),
    "rank1d_bf16": dict(B=2, S=3, H=6, W=18, gh=1, gw=9, thr=0.5, mode="pairwise-rank", cls="1d", kind="bf16"),
    "rank1d_f16": dict(B=1, S=4, H=4, W=16, gh=1, gw=4, thr=0.25, mode="pairwise-rank", cls="1d", kind="f16"),
}


def select_inputs(name: str) -> np.ndarray:
    spec = SELECT_CASES[name]
    rng = np.random.default_rng(abs(hash_name(name)))
    conf = rng.random((spec["B"], spec["S"] * spec["H"] * spec["W"]), dtype=np.float32)
    return round_kind(conf, spec["kind"])


def hash_name(name: str) -> int:
    h = 2166136261
    for ch in name.encode():
        h = ((h ^ ch) * 16777619) & 0xFFFFFFFF
    return h


# ---- attention ---------------------------------------------------------------------------------------------
EXTRA_ATTENTION_CASES = [  # (seq_lens, H, D, dtype) beyond the reference's own list
    ([798, 300], 1, 64, "bf16"),   # one post-merge frame length of the headline configuration + a short one
    ([1, 7, 129], 2, 64, "bf16"),  # degenerate and just-over-a-tile segments
    ([257], 3, 64, "f16"),
]


def attention_inputs(i: int, case):
    seq_lens, H, D, kind = case
    P = int(sum(seq_lens))
    rng = np.random.default_rng(4400 + i)
    qkv = round_kind(rng.standard_normal((P, 3, H, D), dtype=np.float32), kind)
    weight = np.maximum(rng.random(P, dtype=np.float32), np.float32(1e-3))
    if i % 2 == 1:  # merge-count style weights {1, 9}
        weight = np.where(rng.random(P) < 0.25, np.float32(9.0), np.float32(1.0))
    bias = round_kind(np.log(weight.astype(np.float32)), kind)
    cu = np.zeros(len(seq_lens) + 1, np.int32)
    cu[1:] = np.cumsum(seq_lens)
    return qkv, bias, cu


# ---- headline standalone configuration -----------------------------------------------------------------------
def cfg1_inputs(frames: int = 8, channels: int = 1024):
    """8 frames x (5 special + 37x37 patch) tokens ~N(0,1), per-patch confidence ~U(0,1), seed 0."""
    rng = np.random.default_rng(0)
    tokens = rng.standard_normal((frames, 5 + 37 * 37, channels), dtype=np.float32)
    conf = rng.random((frames, 37 * 37), dtype=np.float32)
    return tokens, conf


# ---- pre-attention preparation (q/k LayerNorm + 2-D rotary embedding) -------------------------------------------
PREPARE_CASES = [  # (P, H, D, dtype, use_norm, use_rope)
    (150, 16, 64, "bf16", True, True),   # the attention shape of the headline configuration
    (129, 4, 32, "f16", True, True),
    (64, 2, 128, "bf16", True, True),
    (100, 16, 64, "bf16", False, True),  # nn.Identity norms
    (100, 16, 64, "f16", True, False),   # no rotary embedding
]
PREPARE_EPS = 1e-5          # nn.LayerNorm default, as the attention module builds q_norm / k_norm
PREPARE_MAX_POSITION = 38   # 37 x 37 patch grid + 1


def prepare_inputs(i: int, case):
    """qkv [P,3,H,D], (q_gamma, q_beta, k_gamma, k_beta) [D] and positions [P,2]; floats exactly representable in
    the case's dtype."""
    P, H, D, kind, _norm, _rope = case
    rng = np.random.default_rng(7700 + i)
    qkv = round_kind(rng.standard_normal((P, 3, H, D), dtype=np.float32) * np.float32(1.5) + np.float32(0.3), kind)
    params = [round_kind(np.float32(1.0) + np.float32(0.2) * rng.standard_normal(D, dtype=np.float32), kind),
              round_kind(np.float32(0.1) * rng.standard_normal(D, dtype=np.float32), kind),
              round_kind(np.float32(1.0) + np.float32(0.2) * rng.standard_normal(D, dtype=np.float32), kind),
              round_kind(np.float32(0.1) * rng.standard_normal(D, dtype=np.float32), kind)]
    pos = rng.integers(0, PREPARE_MAX_POSITION, size=(P, 2)).astype(np.int64)
    return qkv, params, pos


POSITION_CASES = [  # (frames, H, W, gh, gw, start_index): grids the reference's 2-D merger accepts (H % gh == 0)
    (3, 36, 36, 3, 3, 5),
    (2, 8, 12, 2, 3, 1),
]


def position_mask(i: int, case) -> np.ndarray:
    frames, H, W, gh, gw, _s = case
    rng = np.random.default_rng(7900 + i)
    return rng.random((frames, (H // gh) * (W // gw))) < 0.5


# ---- LayerNorm + merge (the block's norm1 followed by the merge of the per-layer mode) --------------------------
LN_MERGE_CASES = [  # (frames, H, W, gh, gw, start_index, C, dtype): grids the reference's 2-D merger accepts
    (2, 6, 6, 3, 3, 5, 1024, "bf16"),
    (2, 6, 9, 3, 3, 1, 256, "f32"),
    (1, 4, 6, 2, 2, 0, 1536, "f16"),
]
LN_MERGE_EPS = 1e-6  # the ViT blocks' LayerNorm eps


def ln_merge_inputs(i: int, case):
    frames, H, W, gh, gw, start, C, kind = case
    rng = np.random.default_rng(8100 + i)
    x = round_kind(rng.standard_normal((frames, start + H * W, C), dtype=np.float32) * np.float32(1.7) + np.float32(0.2), kind)
    gamma = round_kind(np.float32(1.0) + np.float32(0.2) * rng.standard_normal(C, dtype=np.float32), kind)
    beta = round_kind(np.float32(0.1) * rng.standard_normal(C, dtype=np.float32), kind)
    mask = rng.random((frames, (H // gh) * (W // gw))) < 0.5
    return x, gamma, beta, mask


def ln_merge_tolerance(kind: str) -> float:
    """Bound against the reference's CPU run: PyTorch sums the LayerNorm statistics in another order, which moves a
    normalised value by at most one unit in the last place of the element type."""
    return {"bf16": 2.0 ** -7, "f16": 2.0 ** -10, "f32": 4e-6}[kind]


# transformer block on unmerged tokens: the reference's own ``Block`` (float32, CPU) pins the block arithmetic of the
# oracle (norms, qkv order, q/k norm, rotary embedding, attention, projection, LayerScale, MLP with exact GELU)
BLOCK_CASES = [  # (frames, grid side, start_index, C, heads, mlp_ratio, qk_norm, rope, layer-scale init)
    (2, 6, 5, 128, 2, 4.0, True, True, 0.5),
    (3, 5, 1, 64, 1, 2.0, False, True, None),
    (1, 7, 5, 128, 4, 4.0, True, False, 1.0),
]
BLOCK_TOLERANCE = 2e-5  # float32 against float32, different summation orders
BLOCK_PARAM_NAMES = ("norm1.weight", "norm1.bias", "attn.qkv.weight", "attn.qkv.bias", "attn.q_norm.weight",
                     "attn.q_norm.bias", "attn.k_norm.weight", "attn.k_norm.bias", "attn.proj.weight", "attn.proj.bias",
                     "ls1.gamma", "norm2.weight", "norm2.bias", "mlp.fc1.weight", "mlp.fc1.bias", "mlp.fc2.weight",
                     "mlp.fc2.bias", "ls2.gamma")


def block_param_shapes(C: int, heads: int, mlp_ratio: float, qk_norm: bool, ls_init) -> dict:
    D, hidden = C // heads, int(C * mlp_ratio)
    shapes = {"norm1.weight": (C,), "norm1.bias": (C,), "attn.qkv.weight": (3 * C, C), "attn.qkv.bias": (3 * C,),
              "attn.proj.weight": (C, C), "attn.proj.bias": (C,), "norm2.weight": (C,), "norm2.bias": (C,),
              "mlp.fc1.weight": (hidden, C), "mlp.fc1.bias": (hidden,), "mlp.fc2.weight": (C, hidden), "mlp.fc2.bias": (C,)}
    if qk_norm:
        shapes.update({"attn.q_norm.weight": (D,), "attn.q_norm.bias": (D,), "attn.k_norm.weight": (D,), "attn.k_norm.bias": (D,)})
    if ls_init:
        shapes.update({"ls1.gamma": (C,), "ls2.gamma": (C,)})
    return {k: shapes[k] for k in BLOCK_PARAM_NAMES if k in shapes}


def block_params(rng, C: int, heads: int, mlp_ratio: float, qk_norm: bool, ls_init, kind: str = "f32") -> dict:
    """Seeded parameters of one block: weight matrices ~ N(0, 1/fan_in), norm gains around 1, LayerScale around its
    init value, small biases; rounded to ``kind``."""
    p = {}
    for name, shape in block_param_shapes(C, heads, mlp_ratio, qk_norm, ls_init).items():
        r = rng.standard_normal(shape, dtype=np.float32)
        if len(shape) == 2:
            v = r / np.float32(np.sqrt(shape[1]))
        elif name.endswith("gamma"):
            v = np.float32(ls_init) * (np.float32(1.0) + np.float32(0.1) * r)
        elif "norm" in name and name.endswith("weight"):
            v = np.float32(1.0) + np.float32(0.1) * r
        else:
            v = np.float32(0.05) * r
        p[name] = round_kind(v.astype(np.float32), kind)
    return p


def block_inputs(i: int, case):
    frames, side, start, C, heads, mlp_ratio, qk_norm, rope, ls_init = case
    rng = np.random.default_rng(9300 + i)
    N = start + side * side
    x = rng.standard_normal((frames, N, C), dtype=np.float32)
    params = block_params(rng, C, heads, mlp_ratio, qk_norm, ls_init)
    ys, xs = np.meshgrid(np.arange(side), np.arange(side), indexing="ij")
    pos = np.zeros((N, 2), np.int64)
    pos[start:, 0] = ys.reshape(-1) + 1
    pos[start:, 1] = xs.reshape(-1) + 1
    return x, params, np.broadcast_to(pos, (frames, N, 2)).copy()


# suffix tokens of jagged segments: (segment lengths, suffix length T, channels)
SUFFIX_CASES = [
    ([3], 1, 1),
    ([2, 1], 2, 1),
    ([1, 3, 2], 1, 2),
    ([5, 0, 7, 1], 3, 8),      # an empty segment
    ([40, 33, 61], 4, 136),    # rows of 17 sixteen-byte vectors in bfloat16
    ([9, 12], 0, 16),          # nothing appended
]


def suffix_inputs(i: int, case):
    lens, T, C = case
    rng = np.random.default_rng(9700 + i)
    P = int(sum(lens))
    tokens = rng.standard_normal((P, C), dtype=np.float32)
    weight = rng.choice(np.array([1.0, 4.0, 9.0], np.float32), size=P)
    offset = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    suffix = rng.standard_normal((len(lens), T, C), dtype=np.float32)
    return tokens, weight, offset, suffix
