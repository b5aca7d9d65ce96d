"""Known-answer cases of the reference's own test-suite, restated as plain data.

1-D cases: ``test/unit_test/test_token_merge_func.py:26-198`` (two hand-made, seven generated).
2-D cases: ``test/auto_test/test_token_merge_2d.py:46-121``.
Every case is a dict of nested lists; ``tokens`` carries a trailing channel axis unless given as 3-D.
"""

T, F = True, False


def _c(tokens, mask, start, group, out, offset, rev, weight, restored):
    return dict(tokens=tokens, mask=mask, start_index=start, group_size=group, out=out, offset=offset,
                rev=rev, weight=weight, restored=restored)


CASES_1D = [
    # hand-made, one special token, G = 2
    _c([[0, 1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11, 12, 13]], [[T, F, T], [F, F, T]], 1, 2,
       [0, 1.5, 3, 4, 5.5, 7, 8, 9, 10, 11, 12.5], [0, 5, 11],
       [0, 1, 1, 2, 3, 4, 4, 5, 6, 7, 8, 9, 10, 10], [1, 2, 1, 1, 2, 1, 1, 1, 1, 1, 2],
       [[0, 1.5, 1.5, 3, 4, 5.5, 5.5], [7, 8, 9, 10, 11, 12.5, 12.5]]),
    # hand-made, no special token
    _c([[1, 2, 3, 4, 5, 6], [8, 9, 10, 11, 12, 13]], [[T, F, T], [F, F, T]], 0, 2,
       [1.5, 3, 4, 5.5, 8, 9, 10, 11, 12.5], [0, 4, 9],
       [0, 0, 1, 2, 3, 3, 4, 5, 6, 7, 8, 8], [2, 1, 1, 2, 1, 1, 1, 1, 2],
       [[1.5, 1.5, 3, 4, 5.5, 5.5], [8, 9, 10, 11, 12.5, 12.5]]),
    # all groups merged
    _c([[1, 2, 3, 4, 5, 6]], [[T, T, T]], 0, 2, [1.5, 3.5, 5.5], [0, 3], [0, 0, 1, 1, 2, 2], [2, 2, 2],
       [[1.5, 1.5, 3.5, 3.5, 5.5, 5.5]]),
    # nothing merged
    _c([[1, 2, 3, 4, 5, 6]], [[F, F, F]], 0, 2, [1, 2, 3, 4, 5, 6], [0, 6], [0, 1, 2, 3, 4, 5],
       [1, 1, 1, 1, 1, 1], [[1, 2, 3, 4, 5, 6]]),
    # G = 3
    _c([[1, 2, 3, 4, 5, 6]], [[T, F]], 0, 3, [2, 4, 5, 6], [0, 4], [0, 0, 0, 1, 2, 3], [3, 1, 1, 1],
       [[2, 2, 2, 4, 5, 6]]),
    # two channels (tokens / out / restored given with their channel axis)
    _c([[[1, 10], [2, 20], [3, 30], [4, 40]]], [[T, F]], 0, 2, [[1.5, 15], [3, 30], [4, 40]], [0, 3],
       [0, 0, 1, 2], [2, 1, 1], [[[1.5, 15], [1.5, 15], [3, 30], [4, 40]]]),
    # three frames, varied patterns
    _c([[1, 2, 3, 4], [5, 6, 7, 8], [9, 10, 11, 12]], [[T, T], [F, F], [T, F]], 0, 2,
       [1.5, 3.5, 5, 6, 7, 8, 9.5, 11, 12], [0, 2, 6, 9], [0, 0, 1, 1, 2, 3, 4, 5, 6, 6, 7, 8],
       [2, 2, 1, 1, 1, 1, 2, 1, 1], [[1.5, 1.5, 3.5, 3.5], [5, 6, 7, 8], [9.5, 9.5, 11, 12]]),
    # G = 4 with two special tokens
    _c([[0, 1, 2, 3, 4, 5, 6, 7, 8, 9], [10, 11, 12, 13, 14, 15, 16, 17, 18, 19]], [[T, F], [F, T]], 2, 4,
       [0, 1, 3.5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 17.5], [0, 7, 14],
       [0, 1, 2, 2, 2, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 13, 13, 13],
       [1, 1, 4, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 4],
       [[0, 1, 3.5, 3.5, 3.5, 3.5, 6, 7, 8, 9], [10, 11, 12, 13, 14, 15, 17.5, 17.5, 17.5, 17.5]]),
    # G = 1: merging a single token is the identity
    _c([[10, 20, 30, 40]], [[T, F, T]], 1, 1, [10, 20, 30, 40], [0, 4], [0, 1, 2, 3], [1, 1, 1, 1],
       [[10, 20, 30, 40]]),
]


def _c2(tokens, mask, start, gh, gw, H, W, out, offset, rev, weight, restored):
    return dict(tokens=tokens, mask=mask, start_index=start, gh=gh, gw=gw, H=H, W=W, out=out, offset=offset,
                rev=rev, weight=weight, restored=restored)


CASES_2D = [
    # 4x4 grid, 2x2 windows, windows 0 and 2 merged
    _c2([list(range(16))], [[T, F, T, F]], 0, 2, 2, 4, 4,
        [2.5, 2, 3, 6, 7, 10.5, 10, 11, 14, 15], [0, 10],
        [0, 0, 1, 2, 0, 0, 3, 4, 5, 5, 6, 7, 5, 5, 8, 9], [4, 1, 1, 1, 1, 4, 1, 1, 1, 1],
        [[2.5, 2.5, 2, 3, 2.5, 2.5, 6, 7, 10.5, 10.5, 10, 11, 10.5, 10.5, 14, 15]]),
    # two frames, 2x4 grid, 2x2 windows, one special token
    _c2([[99, 0, 1, 2, 3, 4, 5, 6, 7], [100, 8, 9, 10, 11, 12, 13, 14, 15]], [[T, F], [F, T]], 1, 2, 2, 2, 4,
        [99, 2.5, 2, 3, 6, 7, 100, 8, 9, 12, 13, 12.5], [0, 6, 12],
        [0, 1, 1, 2, 3, 1, 1, 4, 5, 6, 7, 8, 11, 11, 9, 10, 11, 11], [1, 4, 1, 1, 1, 1, 1, 1, 1, 1, 1, 4],
        [[99, 2.5, 2.5, 2, 3, 2.5, 2.5, 6, 7], [100, 8, 9, 12.5, 12.5, 12, 13, 12.5, 12.5]]),
    # 4x6 grid, 2x3 windows, everything merged
    _c2([list(range(24))], [[T, T, T, T]], 0, 2, 3, 4, 6, [4, 7, 16, 19], [0, 4],
        [0, 0, 0, 1, 1, 1, 0, 0, 0, 1, 1, 1, 2, 2, 2, 3, 3, 3, 2, 2, 2, 3, 3, 3], [6, 6, 6, 6],
        [[4, 4, 4, 7, 7, 7, 4, 4, 4, 7, 7, 7, 16, 16, 16, 19, 19, 19, 16, 16, 16, 19, 19, 19]]),
]

# Shapes of the reference's randomised parity sweeps.
RANDOM_CONFIGS_1D = [  # (B, M, G, start_index, C)  test/auto_test/test_token_merge_cuda.py:77-88
    (1, 4, 2, 0, 8), (2, 8, 2, 1, 16), (4, 16, 4, 2, 32), (8, 32, 4, 0, 64), (2, 64, 8, 4, 128),
    (16, 128, 2, 0, 256), (1, 256, 4, 1, 512), (4, 512, 2, 0, 1024), (2, 1024, 4, 2, 512),
]
RANDOM_CONFIGS_2D = [  # (B, H, W, gh, gw, start_index, C)  test/auto_test/test_token_merge_2d.py:218-228
    (1, 4, 4, 2, 2, 0, 8), (2, 4, 6, 2, 3, 1, 16), (4, 8, 8, 4, 4, 0, 32), (2, 6, 6, 2, 3, 2, 64),
    (8, 8, 16, 4, 4, 0, 128), (1, 16, 16, 4, 8, 1, 256), (4, 8, 12, 2, 4, 0, 64), (2, 12, 12, 4, 6, 3, 32),
]
# Segment-length sets and head shapes of the biased attention tests (test/auto_test/test_flex_attention_bias.py:247-331).
ATTENTION_CASES = [  # (seq_lens, H, D, dtype)
    ([32, 48, 24, 24], 2, 32, "f16"), ([56, 49, 23], 2, 32, "f16"), ([128], 2, 32, "f16"),
    ([60, 40], 2, 32, "f16"), ([50], 1, 64, "f16"), ([64, 64], 4, 64, "f16"), ([64, 64], 4, 64, "bf16"),
    ([128, 256], 4, 64, "f16"), ([100, 150, 50], 4, 64, "f16"), ([64, 64, 64, 64], 4, 64, "f16"),
]
ATTENTION_ATOL = 1e-2  # test/auto_test/test_flex_attention_bias.py:20-21
ATTENTION_RTOL = 1e-2


def as_arrays(case):
    """Convert one case dict into numpy arrays (tokens/out/restored get their channel axis)."""
    import numpy as np

    tok = np.asarray(case["tokens"], dtype=np.float32)
    if tok.ndim == 2:
        tok = tok[..., None]
    out = np.asarray(case["out"], dtype=np.float32)
    if out.ndim == 1:
        out = out[:, None]
    res = np.asarray(case["restored"], dtype=np.float32)
    if res.ndim == 2:
        res = res[..., None]
    d = dict(case)
    d.update(tokens=tok, mask=np.asarray(case["mask"], dtype=bool), out=out,
             offset=np.asarray(case["offset"], dtype=np.int64), rev=np.asarray(case["rev"], dtype=np.int64),
             weight=np.asarray(case["weight"], dtype=np.float32), restored=res)
    return d
