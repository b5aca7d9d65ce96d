"""Times the reference's own PyTorch fallback path on the host cores beside the C port of this folder, on the standalone
op-chain configuration (8 frames x 1374 tokens x 1024 channels, 3x3 windows, 50 % merged, 16 heads x 64).

Usage (only where a checkout of the reference is available):

    python oracle/time_reference_cpu.py --reference /path/to/CoMe

The reference rejects a 37x37 grid with 3x3 windows, so its merge runs in the form the 2-D operator reduces to: the 1-D
operator with the 73 uncovered patches moved behind the 5 special tokens (start_index 78, 144 groups of 9).  Attention is
the float32 biased softmax of the reference's test suite (test/auto_test/test_flex_attention_bias.py:26-36).
Test infrastructure: prints one JSON object, used to relate the `port` CPU baseline of the benchmark to the reference's
CPU path.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))


def best_of(fn, n=3):
    best = 1e30
    for _ in range(n):
        t0 = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t0)
    return best * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    import torch
    from make_golden import import_reference
    import_reference(args.reference)
    from src.accelerate.token_merger.co_me import func_token_merge, func_token_split
    from src.utility.feature import CUDAExtension
    from oracle import clib

    frames, start, G, M, C, H, D = 8, 78, 9, 144, 1024, 16, 64
    N = start + M * G
    rng = np.random.default_rng(0)
    tokens = rng.standard_normal((frames, N, C), dtype=np.float32)
    means = rng.random((frames, M), dtype=np.float32)
    mask = means < np.quantile(means, 0.5, axis=1, keepdims=True)
    t_tokens, t_mask = torch.from_numpy(tokens), torch.from_numpy(mask)
    res = {"threads_torch": torch.get_num_threads(), "threads_openmp": clib.num_threads(), "config": "8 x 1374 x 1024 fp32, 72 of 144 windows merged per frame"}
    with CUDAExtension.disable():
        jag, rev = func_token_merge(t_tokens, start, G, t_mask)
        res["reference_merge_ms"] = best_of(lambda: func_token_merge(t_tokens, start, G, t_mask))
        res["reference_split_ms"] = best_of(lambda: func_token_split(jag, rev, (1, frames, N, C)))
    res["port_merge_ms"] = best_of(lambda: clib.token_merge(tokens, start, G, mask))
    out, off, rev_np, w = clib.token_merge(tokens, start, G, mask)
    res["port_split_ms"] = best_of(lambda: clib.token_split(out, rev_np))
    assert np.array_equal(jag.offset.numpy(), off) and np.array_equal(rev.numpy(), rev_np)
    assert np.abs(jag.tokens[0].numpy() - out).max() <= 1e-6
    # frame attention of the 8 merged frames, 16 heads, float32
    P = out.shape[0]
    qkv = rng.standard_normal((P, 3, H, D), dtype=np.float32)
    bias = np.log(w)
    cu = off.astype(np.int32)
    tq, tb = torch.from_numpy(qkv), torch.from_numpy(bias)

    def torch_attention():  # softmax(q k^T * scale + log_w[None, :]) @ v per segment and head
        outs = []
        for s in range(frames):
            a, e = int(cu[s]), int(cu[s + 1])
            q, k, v = (tq[a:e, i].transpose(0, 1) for i in range(3))  # [H, L, D]
            att = torch.softmax(q @ k.transpose(1, 2) * D ** -0.5 + tb[a:e][None, None, :], dim=-1)
            outs.append((att @ v).transpose(0, 1))
        return torch.cat(outs)

    want = torch_attention().numpy()
    res["reference_frame_attention_ms"] = best_of(torch_attention)
    got, _ = clib.attention_bias(qkv, bias, cu, D ** -0.5)
    res["port_frame_attention_ms"] = best_of(lambda: clib.attention_bias(qkv, bias, cu, D ** -0.5))
    assert np.abs(got - want).max() <= 1e-4
    print(json.dumps(res))


if __name__ == "__main__":
    main()
