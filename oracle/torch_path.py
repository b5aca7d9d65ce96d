"""The biased attention of the reference's CPU path restated with PyTorch CPU operators -- the form the reference's own
test oracle has (``test/auto_test/test_flex_attention_bias.py:26-36``: ``softmax(q k^T * scale + log_w[None, :]) @ v`` per
segment and head, float32).  TEST INFRASTRUCTURE ONLY: it is the timed CPU baseline of the benchmark (the reference's
fallback path is PyTorch, whose matrix products run on the BLAS library PyTorch ships; the plain C loops of
``come_oracle.c`` are about five times slower on the same cores) and is itself checked against ``come_oracle.c`` by the
CPU tests.  The product library never imports it.
"""
from __future__ import annotations

import numpy as np
import torch


def attention_bias(qkv: np.ndarray, bias, cu_seqlens, scale: float, q_lo: int = 0, q_hi: int = -1):
    """``qkv [P, 3, H, D]`` float32 packed; returns ``(out [P, H, D], lse [H, P])`` as numpy arrays.  ``q_lo / q_hi``
    restrict the query rows of every segment (bounded benchmark samples); rows outside stay zero / +inf."""
    t = torch.from_numpy(np.ascontiguousarray(qkv, np.float32))
    P, _, H, D = t.shape
    b = None if bias is None else torch.from_numpy(np.ascontiguousarray(bias, np.float32))
    out = torch.zeros((P, H, D), dtype=torch.float32)
    lse = torch.full((H, P), float("inf"), dtype=torch.float32)
    cu = [int(c) for c in cu_seqlens]
    for a, e in zip(cu[:-1], cu[1:]):
        lo = a + q_lo
        hi = e if (q_hi < 0 or a + q_hi > e) else a + q_hi
        if hi <= lo:
            continue
        k = t[a:e, 1].transpose(0, 1)            # [H, L, D]
        v = t[a:e, 2].transpose(0, 1)
        # the expression materialises the score matrix: walk the query rows in blocks that keep it under ~1.5 GB
        step = max(1, int(1.5e9 // (4 * H * max(e - a, 1))))
        for r0 in range(lo, hi, step):
            r1 = min(r0 + step, hi)
            q = t[r0:r1, 0].transpose(0, 1)      # [H, rows, D]
            s = q @ k.transpose(1, 2) * scale
            if b is not None:
                s = s + b[a:e][None, None, :]
            lse[:, r0:r1] = torch.logsumexp(s, dim=-1)
            out[r0:r1] = (torch.softmax(s, dim=-1) @ v).transpose(0, 1)
    return out.numpy(), lse.numpy()


def set_num_threads(n: int) -> None:
    torch.set_num_threads(max(int(n), 1))


def num_threads() -> int:
    return int(torch.get_num_threads())
