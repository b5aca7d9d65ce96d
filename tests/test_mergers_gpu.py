"""The merger objects with the reference's ``ITokenMerger`` contract (``src/interface/token_merger.py:102-116``) and the
MLP half of the per-layer mode, on the GPU, against the oracle."""
import numpy as np
import pytest
import torch

import golden_inputs as gi
from gpu_util import to_dev, to_np
from oracle import come_oracle as orc

pytestmark = pytest.mark.gpu


def _predictor_for(conf: torch.Tensor):
    """Stand-in for the distilled confidence predictor: returns a fixed confidence ``[B, S*H*W, 1]`` and records what it
    was called with."""
    seen = {}

    def predictor(feature, BPHWC):
        seen["shape"], seen["dtype"], seen["BPHWC"] = tuple(feature.shape), feature.dtype, BPHWC
        return conf.unsqueeze(-1)

    return predictor, seen


@pytest.mark.parametrize("mode,thr", [("pairwise-rank", 0.5), ("abs_mse", 0.4), ("mse", -0.1)])
def test_one_dimensional_merger_object(mode, thr):
    """``CoMeTokenMerger`` (``src/accelerate/token_merger/co_me.py:21-105``): build_ctx ranks the groups of consecutive
    tokens per frame, merge / split / build_infer_mask follow the reference's shapes; every result against the oracle."""
    from come_b200.token_merger import CoMeTokenMerger
    B, S, H, W, C, G, start = 2, 3, 6, 6, 32, 9, 5
    rng = np.random.default_rng(3)
    conf = gi.round_kind(rng.random((B, S * H * W), dtype=np.float32), "bf16")
    predictor, seen = _predictor_for(to_dev(conf, "bf16"))
    merger = CoMeTokenMerger(start, G, thr, predictor, conf_mode=mode)
    feature = torch.zeros((B, S, 4, H, W), device="cuda")
    ctx = merger.build_ctx(feature)
    mask, shape = ctx[0], ctx[1]
    assert shape == (B, S, 4, H, W) and seen["shape"] == (B, S, H, W, 4) and seen["dtype"] == torch.bfloat16
    M = H * W // G
    want_mask = orc.select_windows(conf, B, S, M, G, 1, G, thr, mode, "frame", "bf16")
    np.testing.assert_array_equal(to_np(mask), want_mask)
    tokens = rng.standard_normal((B, S, start + H * W, C), dtype=np.float32)
    jag, stub = merger.merge(ctx, to_dev(tokens))
    out, off, rev, w = orc.token_merge(tokens.reshape(B * S, -1, C), start, G, want_mask)
    np.testing.assert_array_equal(to_np(jag.tokens[0]), out)
    np.testing.assert_array_equal(to_np(jag.offset), off)
    np.testing.assert_array_equal(to_np(jag.weight), w)
    np.testing.assert_array_equal(to_np(stub[0]), rev)
    back = merger.split(ctx, stub, jag)
    assert tuple(back.shape) == (B, S, start + H * W, C)
    np.testing.assert_array_equal(to_np(back).reshape(-1, C), orc.token_split(out, rev))
    infer = merger.build_infer_mask(ctx)
    assert tuple(infer.shape) == (B, S, H, W) and infer.dtype == torch.bool
    np.testing.assert_array_equal(to_np(infer).reshape(B * S, M, G), np.repeat(want_mask[:, :, None], G, axis=2))
    # another number of special tokens for the same mask (what the reference's merge(..., start_index=...) does)
    jag0, stub0 = merger.merge(ctx, to_dev(tokens[:, :, start:]), start_index=0)
    out0, off0, rev0, _ = orc.token_merge(tokens[:, :, start:].reshape(B * S, -1, C), 0, G, want_mask)
    np.testing.assert_array_equal(to_np(jag0.tokens[0]), out0)
    np.testing.assert_array_equal(to_np(jag0.offset), off0)
    with pytest.raises(ValueError, match="divisible"):
        merger.build_ctx(torch.zeros((B, S, 4, 5, 5), device="cuda"))


def test_two_dimensional_merger_object_z_normalised_mode():
    """``CoMe2DTokenMerger`` in the reference's third confidence mode (``co_me_2d.py:274-281``)."""
    from come_b200.token_merger import CoMe2DTokenMerger
    B, S, H, W, C = 1, 4, 9, 12, 16
    rng = np.random.default_rng(4)
    conf = gi.round_kind(rng.random((B, S * H * W), dtype=np.float32) * 2 - 0.5, "bf16")
    predictor, _ = _predictor_for(to_dev(conf, "bf16"))
    merger = CoMe2DTokenMerger(5, 3, 3, 0.2, predictor, conf_mode="mse")
    mask, shape, plan = merger.build_ctx(torch.zeros((B, S, 2, H, W), device="cuda"))
    want = orc.select_windows(conf, B, S, H, W, 3, 3, 0.2, "mse", "batch", "bf16")
    np.testing.assert_array_equal(to_np(mask), want)
    assert 0 < int(want.sum()) < want.size and plan.frames == B * S


class _Mlp(torch.nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.fc1, self.act, self.fc2 = torch.nn.Linear(dim, 4 * dim), torch.nn.GELU(), torch.nn.Linear(4 * dim, dim)

    def forward(self, x):
        return self.fc2(self.act(self.fc1(x)))


@pytest.mark.parametrize("global_shape", [False, True])
def test_direct_mlp(global_shape):
    """The per-layer replacement of block.mlp.forward (``src/accelerate/vggt/direct.py:148-168``): the MLP on the merged
    tokens, split back -- against merge (oracle) -> the same module -> split (oracle); and the fused residual branch
    ``x + ls2(mlp(norm2(x)))`` against the oracle chain around the same module."""
    from come_b200 import _lib
    from come_b200.direct import DirectMlp
    from come_b200.token_merger import MergePlan
    torch.manual_seed(7)
    dim, S, Hg, Wg = 128, 3, 7, 8
    rng = np.random.default_rng(41)
    mask = rng.random((S, 4)) < 0.5
    plan = MergePlan(torch.from_numpy(mask).cuda(), _lib.Layout.two_d(5, Hg, Wg, 3, 3))
    N = 5 + Hg * Wg
    mlp = _Mlp(dim).cuda().bfloat16().eval()
    mod = DirectMlp(mlp)
    xb = gi.round_kind(rng.standard_normal((S, N, dim), dtype=np.float32), "bf16")
    x = to_dev(xb, "bf16")
    x_in = x.reshape(1, S * N, dim) if global_shape else x
    with torch.no_grad():
        y = mod(x_in, plan)
    assert y.shape == x_in.shape and y.dtype == torch.bfloat16
    merged, off, rev, w = orc.token_merge_2d_ragged(xb, 5, 3, 3, Hg, Wg, mask)
    merged = gi.round_kind(merged, "bf16")
    with torch.no_grad():
        hidden = mlp(torch.from_numpy(merged).cuda().bfloat16())
    want = orc.token_split(to_np(hidden), rev).reshape(x_in.shape)
    np.testing.assert_array_equal(to_np(y), want)  # same module on the same merged rows: bit for bit
    # residual branch
    norm2 = torch.nn.LayerNorm(dim, eps=1e-6).cuda().bfloat16()
    gamma = torch.from_numpy(gi.round_kind(0.5 * rng.random(dim, dtype=np.float32), "bf16")).cuda().bfloat16()
    with torch.no_grad():
        z = mod.forward_residual(x_in, plan, norm2, gamma)
    normed = orc.layer_norm_rows(xb, to_np(norm2.weight), to_np(norm2.bias), 1e-6, "bf16")
    merged2, _, rev2, _ = orc.token_merge_2d_ragged(normed, 5, 3, 3, Hg, Wg, mask)
    with torch.no_grad():
        hidden2 = mlp(torch.from_numpy(gi.round_kind(merged2, "bf16")).cuda().bfloat16())
    want2 = orc.token_split_residual(to_np(hidden2), rev2, xb.reshape(-1, dim), to_np(gamma), "bf16").reshape(x_in.shape)
    np.testing.assert_array_equal(to_np(z), want2)
