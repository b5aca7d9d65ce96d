"""ctypes front end of the C oracle (``come_oracle.c``).  Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from .build import LIB, build

_KIND = {"f32": 0, "f16": 1, "bf16": 2}
_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build()
        _lib = C.CDLL(LIB)
        _lib.orc_merge.restype = C.c_int64
        _lib.orc_layout2d.restype = C.c_int64
        _lib.orc_select.restype = C.c_int
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    """OpenMP threads of the following calls."""
    lib().orc_set_num_threads(C.c_int(int(n)))


def layout2d(start, H, W, gh, gw):
    src = np.empty(start + H * W, np.int64)
    prefix = lib().orc_layout2d(C.c_int64(start), C.c_int64(H), C.c_int64(W), C.c_int64(gh), C.c_int64(gw), _p(src))
    return src, int(prefix)


def token_merge(tokens, start_index, group_size, mask, kind="f32", src_of=None):
    tokens = np.ascontiguousarray(tokens, np.float32)
    mask8 = np.ascontiguousarray(mask, np.uint8)
    B, N, Cc = tokens.shape
    M = mask8.shape[1]
    out = np.empty((B * N, Cc), np.float32)
    offsets = np.empty(B + 1, np.int64)
    rev = np.empty(B * N, np.int64)
    weight = np.empty(B * N, np.float32)
    src = None if src_of is None else np.ascontiguousarray(src_of, np.int64)
    P = lib().orc_merge(_p(tokens), C.c_int64(B), C.c_int64(N), C.c_int64(Cc), C.c_int64(start_index),
                        C.c_int64(group_size), C.c_int64(M), _p(mask8), _p(src), C.c_int(_KIND[kind]),
                        _p(out), _p(offsets), _p(rev), _p(weight))
    return out[:P], offsets, rev, weight[:P]


def token_merge_2d(tokens, start_index, gh, gw, H, W, mask, kind="f32"):
    src, prefix = layout2d(start_index, H, W, gh, gw)
    return token_merge(tokens, prefix, gh * gw, mask, kind, src)


def token_split(merged, rev):
    merged = np.ascontiguousarray(merged, np.float32)
    rev = np.ascontiguousarray(rev, np.int64)
    out = np.empty((rev.size, merged.shape[1]), np.float32)
    lib().orc_split(_p(merged), _p(rev), C.c_int64(rev.size), C.c_int64(merged.shape[1]), _p(out))
    return out


def select_windows(conf, B, S, H, W, gh, gw, threshold, mode="pairwise-rank", scope="batch", kind="f32"):
    conf = np.ascontiguousarray(conf, np.float32)
    M = (H // gh) * (W // gw)
    mask = np.empty((B * S, M), np.uint8)
    rc = lib().orc_select(_p(conf), C.c_int64(B), C.c_int64(S), C.c_int64(H), C.c_int64(W), C.c_int64(gh),
                          C.c_int64(gw), C.c_float(threshold), C.c_int({"pairwise-rank": 0, "abs_mse": 1, "mse": 2}[mode]),
                          C.c_int({"batch": 0, "frame": 1}[scope]), C.c_int(_KIND[kind]), None, _p(mask))
    if rc != 0:
        raise MemoryError("orc_select")
    return mask.astype(bool)


def attention_bias(qkv, bias, cu_seqlens, scale, q_lo=0, q_hi=-1):
    """qkv [P, 3, H, D] float32 packed; returns (out [P,H,D], lse [H,P]).  ``q_lo/q_hi`` restrict the query rows
    of every segment (bounded benchmark samples); rows outside stay uninitialised."""
    qkv = np.ascontiguousarray(qkv, np.float32)
    P, _, Hh, D = qkv.shape
    cu = np.ascontiguousarray(cu_seqlens, np.int32)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    out = np.empty((P, Hh, D), np.float32)
    lse = np.full((Hh, P), np.inf, np.float32)
    base = qkv.ctypes.data
    hd = Hh * D * 4
    lib().orc_attention(C.c_void_p(base), C.c_void_p(base + hd), C.c_void_p(base + 2 * hd), C.c_int64(3 * Hh * D),
                        _p(b), _p(cu), C.c_int64(cu.size - 1), C.c_int64(P), C.c_int64(Hh), C.c_int64(D),
                        C.c_float(scale), _p(out), _p(lse), C.c_int64(q_lo), C.c_int64(q_hi))
    return out, lse
