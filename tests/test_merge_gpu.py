"""Merge / unmerge parity on the GPU, through the C ABI (come_b200.co_me_cuext / token_merger).

Mirrors the reference's suites: literal known-answer cases (test/unit_test/test_token_merge_func.py:26-198,
test/auto_test/test_token_merge_2d.py:46-121), the randomised sweeps (test_token_merge_cuda.py:77-155,
test_token_merge_2d.py:218-285) and the validation errors (test_token_merge_func.py:298-318,
test_token_merge_2d.py:288-321).  Bar: indices, offsets and counts bit-exact; float32 features bit-exact against
the oracle and within 1e-6 of the fixtures written by the reference.
"""
import os

import numpy as np
import pytest
import torch

import golden_inputs as gi
import reference_cases as rc
from gpu_util import TORCH_DTYPE, to_dev, to_np
from oracle import clib, come_oracle as orc

pytestmark = pytest.mark.gpu

FEATURE_TOL = dict(rtol=1e-6, atol=1e-6)


@pytest.fixture(scope="module")
def tm():
    from come_b200 import token_merger
    return token_merger


def _merge(tm, tokens, start, G, mask, kind="f32"):
    jag, rev = tm.func_token_merge(to_dev(tokens, kind), start, G, torch.from_numpy(mask).cuda())
    return jag, rev


@pytest.mark.parametrize("idx", range(len(rc.CASES_1D)))
def test_literals_1d(tm, idx):
    c = rc.as_arrays(rc.CASES_1D[idx])
    jag, rev = _merge(tm, c["tokens"], c["start_index"], c["group_size"], c["mask"])
    assert jag.tokens.shape[0] == 1 and jag.offset.dtype == torch.int64 and rev.dtype == torch.int64
    assert jag.weight.dtype == torch.float32
    np.testing.assert_array_equal(to_np(jag.tokens[0]), c["out"])
    np.testing.assert_array_equal(to_np(jag.offset), c["offset"])
    np.testing.assert_array_equal(to_np(jag.weight), c["weight"])
    np.testing.assert_array_equal(to_np(rev), c["rev"])
    B, N, C = c["tokens"].shape
    restored = tm.func_token_split(jag, rev, (1, B, N, C))
    assert tuple(restored.shape) == (B, N, C)
    np.testing.assert_array_equal(to_np(restored), c["restored"])


@pytest.mark.parametrize("idx", range(len(rc.CASES_2D)))
@pytest.mark.parametrize("ragged", [False, True])
def test_literals_2d(tm, idx, ragged):
    c = rc.as_arrays(rc.CASES_2D[idx])
    jag, rev = tm.func_token_merge_2d(to_dev(c["tokens"]), c["start_index"], c["gh"], c["gw"], c["H"], c["W"],
                                      torch.from_numpy(c["mask"]).cuda(), allow_ragged=ragged)
    np.testing.assert_array_equal(to_np(jag.tokens[0]), c["out"])
    np.testing.assert_array_equal(to_np(jag.offset), c["offset"])
    np.testing.assert_array_equal(to_np(jag.weight), c["weight"])
    np.testing.assert_array_equal(to_np(rev), c["rev"])
    B, N, C = c["tokens"].shape
    np.testing.assert_array_equal(to_np(tm.func_token_split(jag, rev, (1, B, N, C))), c["restored"])


@pytest.mark.parametrize("idx", range(len(rc.RANDOM_CONFIGS_1D)))
@pytest.mark.parametrize("kind", ["f32", "bf16"])
def test_random_1d_vs_oracle_and_fixture(tm, golden_dir, idx, kind):
    z = np.load(os.path.join(golden_dir, "merge_1d.npz"))
    cfg = rc.RANDOM_CONFIGS_1D[idx]
    B, M, G, S, C = cfg
    tokens, mask = gi.merge1d_inputs(idx, cfg, kind)
    jag, rev = _merge(tm, tokens, S, G, mask, kind)
    out = to_np(jag.tokens[0])
    o_out, o_off, o_rev, o_w = clib.token_merge(tokens, S, G, mask, kind=kind)
    np.testing.assert_array_equal(to_np(jag.offset), o_off)
    np.testing.assert_array_equal(to_np(rev), o_rev)
    np.testing.assert_array_equal(to_np(jag.weight), o_w)
    np.testing.assert_array_equal(out, o_out)  # same left-to-right float32 sum and one rounding: bit-exact
    key = f"c{idx}_{kind}_"
    tol = FEATURE_TOL if kind == "f32" else dict(rtol=8e-3, atol=8e-3)
    np.testing.assert_array_equal(to_np(rev), z[key + "rev"].astype(np.int64))
    np.testing.assert_array_equal(to_np(jag.offset), z[key + "offset"])
    gi.check_rows(out, z, key + "out_", **tol)
    restored = to_np(tm.func_token_split(jag, rev, (1, B, S + M * G, C))).reshape(-1, C)
    np.testing.assert_array_equal(restored, o_out[o_rev])
    gi.check_rows(restored, z, key + "res_", **tol)


@pytest.mark.parametrize("idx", range(len(rc.RANDOM_CONFIGS_2D)))
def test_random_2d_vs_oracle_and_fixture(tm, golden_dir, idx):
    z = np.load(os.path.join(golden_dir, "merge_2d.npz"))
    cfg = rc.RANDOM_CONFIGS_2D[idx]
    B, H, W, gh, gw, S, C = cfg
    tokens, mask = gi.merge2d_inputs(idx, cfg)
    jag, rev = tm.func_token_merge_2d(to_dev(tokens), S, gh, gw, H, W, torch.from_numpy(mask).cuda())
    o_out, o_off, o_rev, o_w = clib.token_merge_2d(tokens, S, gh, gw, H, W, mask)
    np.testing.assert_array_equal(to_np(jag.tokens[0]), o_out)
    np.testing.assert_array_equal(to_np(jag.offset), o_off)
    np.testing.assert_array_equal(to_np(rev), o_rev)
    np.testing.assert_array_equal(to_np(jag.weight), o_w)
    key = f"c{idx}_"
    np.testing.assert_array_equal(to_np(rev), z[key + "rev"].astype(np.int64))
    gi.check_rows(to_np(jag.tokens[0]), z, key + "out_", **FEATURE_TOL)
    restored = to_np(tm.func_token_split(jag, rev, (1, B, S + H * W, C))).reshape(-1, C)
    np.testing.assert_array_equal(restored, o_out[o_rev])


@pytest.mark.parametrize("mask_val", [True, False])
@pytest.mark.parametrize("kind", ["f32", "f16", "bf16"])
def test_uniform_mask(tm, mask_val, kind):
    B, M, G, S, C = 4, 32, 4, 2, 64
    rng = np.random.default_rng(11)
    tokens = gi.round_kind(rng.standard_normal((B, S + M * G, C), dtype=np.float32), kind)
    mask = np.full((B, M), mask_val)
    jag, rev = _merge(tm, tokens, S, G, mask, kind)
    o_out, o_off, o_rev, o_w = clib.token_merge(tokens, S, G, mask, kind=kind)
    np.testing.assert_array_equal(to_np(jag.tokens[0]), o_out)
    np.testing.assert_array_equal(to_np(jag.offset), o_off)
    np.testing.assert_array_equal(to_np(rev), o_rev)
    np.testing.assert_array_equal(to_np(jag.weight), o_w)


def test_group_size_1(tm):
    B, M, S, C = 2, 16, 1, 32
    rng = np.random.default_rng(12)
    tokens = rng.standard_normal((B, S + M, C), dtype=np.float32)
    mask = rng.random((B, M)) < 0.5
    jag, rev = _merge(tm, tokens, S, 1, mask)
    o_out, o_off, o_rev, o_w = orc.token_merge(tokens, S, 1, mask)
    np.testing.assert_array_equal(to_np(jag.tokens[0]), o_out)
    np.testing.assert_array_equal(to_np(rev), o_rev)
    np.testing.assert_array_equal(to_np(jag.weight), o_w)


@pytest.mark.parametrize("C,kind", [(1, "f32"), (2, "bf16"), (3, "f16"), (6, "f32"), (10, "bf16"), (1028, "f32")])
def test_odd_channel_counts(tm, C, kind):
    """Rows that are not 16-byte multiples take the scalar path (the reference merges 2-channel bf16 positions)."""
    B, M, G, S = 3, 7, 9, 5
    rng = np.random.default_rng(13 + C)
    tokens = gi.round_kind(rng.standard_normal((B, S + M * G, C), dtype=np.float32), kind)
    mask = rng.random((B, M)) < 0.5
    jag, rev = _merge(tm, tokens, S, G, mask, kind)
    o_out, o_off, o_rev, o_w = clib.token_merge(tokens, S, G, mask, kind=kind)
    np.testing.assert_array_equal(to_np(jag.tokens[0]), o_out)
    np.testing.assert_array_equal(to_np(rev), o_rev)
    restored = to_np(tm.func_token_split(jag, rev, (1, B, S + M * G, C))).reshape(-1, C)
    np.testing.assert_array_equal(restored, o_out[o_rev])


def test_large_group_and_many_frames(tm):
    """G above the in-flight batch (12 rows) and more frames than a plan tile."""
    B, M, G, S, C = 300, 5, 25, 3, 8
    rng = np.random.default_rng(14)
    tokens = rng.standard_normal((B, S + M * G, C), dtype=np.float32)
    mask = rng.random((B, M)) < 0.4
    jag, rev = _merge(tm, tokens, S, G, mask)
    o_out, o_off, o_rev, o_w = clib.token_merge(tokens, S, G, mask)
    np.testing.assert_array_equal(to_np(jag.tokens[0]), o_out)
    np.testing.assert_array_equal(to_np(jag.offset), o_off)
    np.testing.assert_array_equal(to_np(rev), o_rev)


def test_many_groups_per_frame(tm):
    """M above one scan tile (256 groups) exercises the carried prefix."""
    B, M, G, S, C = 2, 1000, 3, 1, 4
    rng = np.random.default_rng(15)
    tokens = rng.standard_normal((B, S + M * G, C), dtype=np.float32)
    mask = rng.random((B, M)) < 0.6
    jag, rev = _merge(tm, tokens, S, G, mask)
    o_out, o_off, o_rev, o_w = clib.token_merge(tokens, S, G, mask)
    np.testing.assert_array_equal(to_np(jag.tokens[0]), o_out)
    np.testing.assert_array_equal(to_np(rev), o_rev)
    np.testing.assert_array_equal(to_np(jag.weight), o_w)


def test_empty_inputs(tm):
    tok = torch.zeros((0, 7, 4), device="cuda")
    jag, rev = tm.func_token_merge(tok, 1, 2, torch.zeros((0, 3), dtype=torch.bool, device="cuda"))
    assert jag.tokens.shape == (1, 0, 4) and rev.numel() == 0 and jag.offset.tolist() == [0]
    # no groups at all: only special tokens
    tok = torch.arange(6, dtype=torch.float32, device="cuda").reshape(2, 3, 1)
    jag, rev = tm.func_token_merge(tok, 3, 2, torch.zeros((2, 0), dtype=torch.bool, device="cuda"))
    assert jag.offset.tolist() == [0, 3, 6] and rev.tolist() == [0, 1, 2, 3, 4, 5]
    np.testing.assert_array_equal(to_np(jag.tokens[0, :, 0]), np.arange(6, dtype=np.float32))


def test_non_default_stream(tm):
    rng = np.random.default_rng(16)
    tokens = rng.standard_normal((2, 1 + 8 * 4, 64), dtype=np.float32)
    mask = rng.random((2, 8)) < 0.5
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        jag, rev = _merge(tm, tokens, 1, 4, mask)
        restored = tm.func_token_split(jag, rev, (1, 2, 33, 64))
    s.synchronize()
    o_out, _, o_rev, _ = orc.token_merge(tokens, 1, 4, mask)
    np.testing.assert_array_equal(to_np(restored).reshape(-1, 64), o_out[o_rev])


def test_cfg1_chain_merge_unmerge(tm, golden_dir):
    """Headline standalone configuration: 8 x 1374 tokens x 1024 channels, ragged 37x37 grid, 3x3 windows."""
    z = np.load(os.path.join(golden_dir, "cfg1_chain.npz"))
    tokens, conf = gi.cfg1_inputs()
    mask = tm.select_windows(to_dev(conf), 8, 1, 37, 37, 3, 3, 0.5, "pairwise-rank", "frame")
    want_mask = np.unpackbits(z["mask"])[: 8 * 144].reshape(8, 144).astype(bool)
    np.testing.assert_array_equal(to_np(mask), want_mask)
    jag, rev = tm.func_token_merge_2d(to_dev(tokens), 5, 3, 3, 37, 37, mask, allow_ragged=True)
    assert jag.tokens.shape == (1, 8 * 798, 1024)
    np.testing.assert_array_equal(to_np(jag.offset), z["offset"])
    np.testing.assert_array_equal(to_np(rev), z["rev"].astype(np.int64))
    np.testing.assert_array_equal(to_np(jag.weight), z["weight"].astype(np.float32))
    out = to_np(jag.tokens[0])
    gi.check_rows(out, z, "out_", **FEATURE_TOL)
    o_out, _, o_rev, _ = clib.token_merge_2d(tokens, 5, 3, 3, 37, 37, want_mask)
    np.testing.assert_array_equal(out, o_out)
    restored = to_np(tm.func_token_split(jag, rev, (1, 8, 1374, 1024))).reshape(-1, 1024)
    gi.check_rows(restored, z, "res_", **FEATURE_TOL)
    np.testing.assert_array_equal(restored, o_out[o_rev])


def test_plan_reuse_and_properties(tm):
    """One plan serves many merges; size-independent properties at 100 frames: unmerge(merge(x)) keeps every
    never-merged token bit-exact, merged windows carry their mean, counts sum to the token count."""
    from come_b200 import _lib
    frames, C = 100, 256
    rng = np.random.default_rng(17)
    x = torch.from_numpy(rng.standard_normal((frames, 1374, C), dtype=np.float32)).cuda()
    mask = torch.from_numpy(rng.random((frames, 144)) < 0.5).cuda()
    plan = tm.MergePlan(mask, _lib.Layout.two_d(5, 37, 37, 3, 3))
    assert plan.total == int(frames * 1374 - 8 * mask.sum().item())
    assert plan.max_seqlen == int((plan.offset[1:] - plan.offset[:-1]).max().item())
    assert float(plan.weight.sum().item()) == frames * 1374
    merged = plan.merge(x)
    back = plan.split(merged).reshape(frames, 1374, C)
    same = plan.weight[plan.rev_id] == 1.0
    assert torch.equal(back.reshape(-1, C)[same], x.reshape(-1, C)[same])
    # a second tensor through the same plan (bf16, as the direct mode feeds it)
    y = x[:, :, :64].bfloat16().contiguous()
    back_y = plan.split(plan.merge(y)).reshape(frames, 1374, 64)
    assert torch.equal(back_y.reshape(-1, 64)[same], y.reshape(-1, 64)[same])
    # idempotence: merging the restored grid gives the same packed rows for kept tokens and the same mean
    # (mean of 9 equal values may round once) for merged windows
    again = plan.merge(back)
    kept_rows = plan.weight == 1.0
    assert torch.equal(again[kept_rows], merged[kept_rows])
    torch.testing.assert_close(again, merged, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("tokens,mask,start,G,msg", [
    (torch.randn(2, 7, 4), torch.ones(2, 3, dtype=torch.bool), 0, 2, "Expected N = start_index"),
    (torch.randn(2, 6, 4), torch.ones(3, 3, dtype=torch.bool), 0, 2, "merge_mask batch"),
    (torch.randn(1, 6, 4), torch.ones(1, 3, dtype=torch.bool), -1, 2, "start_index"),
    (torch.randn(1, 6, 4), torch.ones(1, 3, dtype=torch.bool), 0, 0, "group_size"),
    (torch.randn(1, 6, 4), torch.ones(1, 3, dtype=torch.float32), 0, 2, "torch.bool"),
])
def test_validation_1d(tm, tokens, mask, start, G, msg):
    with pytest.raises(ValueError, match=msg):
        tm.func_token_merge(tokens.cuda(), start, G, mask.cuda())


@pytest.mark.parametrize("tokens,mask,start,gh,gw,H,W,msg", [
    (torch.randn(1, 15, 4), torch.ones(1, 3, dtype=torch.bool), 0, 2, 3, 3, 5, "H.*divisible"),
    (torch.randn(1, 12, 4), torch.ones(1, 2, dtype=torch.bool), 0, 2, 5, 4, 3, "W.*divisible"),
    (torch.randn(2, 16, 4), torch.ones(3, 4, dtype=torch.bool), 0, 2, 2, 4, 4, "merge_mask batch"),
    (torch.randn(1, 10, 4), torch.ones(1, 4, dtype=torch.bool), 0, 2, 2, 4, 4, "Expected N"),
    (torch.randn(1, 16, 4), torch.ones(1, 2, dtype=torch.bool), 0, 2, 2, 4, 4, "Expected M"),
    (torch.randn(1, 16, 4), torch.ones(1, 4, dtype=torch.bool), -1, 2, 2, 4, 4, "start_index"),
    (torch.randn(1, 16, 4), torch.ones(1, 4, dtype=torch.bool), 0, 0, 2, 4, 4, "group_h.*group_w.*> 0"),
    (torch.randn(1, 16, 4), torch.ones(1, 4, dtype=torch.float32), 0, 2, 2, 4, 4, "torch.bool"),
])
def test_validation_2d(tm, tokens, mask, start, gh, gw, H, W, msg):
    with pytest.raises(ValueError, match=msg):
        tm.func_token_merge_2d(tokens.cuda(), start, gh, gw, H, W, mask.cuda())


def test_extension_errors_are_runtime_errors():
    from come_b200 import co_me_cuext
    with pytest.raises(RuntimeError, match="on CUDA"):
        co_me_cuext.co_me_token_merge_cuda(torch.randn(1, 6, 4), 0, 2, torch.ones(1, 3, dtype=torch.bool))
    with pytest.raises(RuntimeError, match="N != start_index"):
        co_me_cuext.co_me_token_merge_cuda(torch.randn(1, 7, 4).cuda(), 0, 2, torch.ones(1, 3, dtype=torch.bool).cuda())
    with pytest.raises(RuntimeError, match="C mismatch"):
        co_me_cuext.co_me_token_split_cuda(torch.randn(3, 4).cuda(), torch.zeros(3, dtype=torch.int64).cuda(), 5)


@pytest.mark.parametrize("kind,widths", [("f32", (1024, 1024)), ("bf16", (1024, 1024)), ("f32", (6, 10)), ("f16", (3, 5, 8))])
def test_split_concat(kind, widths):
    """Unmerging several packed tensors side by side equals concatenating the oracle's separate unmerges
    (the [frame | global] concatenation of a retained layer)."""
    import torch
    from come_b200 import _lib
    from come_b200.token_merger import MergePlan
    from gpu_util import TORCH_DTYPE, to_dev, to_np
    import golden_inputs as gi
    from oracle import come_oracle as orc
    rng = np.random.default_rng(sum(widths))
    mask = rng.random((3, 144)) < 0.5
    plan = MergePlan(torch.from_numpy(mask).cuda(), _lib.Layout.two_d(5, 37, 37, 3, 3))
    _o, _off, rev, _w = orc.token_merge_2d_ragged(np.zeros((3, 1374, 1), np.float32), 5, 3, 3, 37, 37, mask)
    parts = [gi.round_kind(rng.standard_normal((plan.total, c), dtype=np.float32), kind) for c in widths]
    got = to_np(plan.split_concat(*[to_dev(p, kind) for p in parts]))
    want = np.concatenate([orc.token_split(p, rev) for p in parts], axis=1)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("kind,C,with_scale", [("bf16", 1024, True), ("f32", 1024, True), ("f16", 1024, False),
                                                ("bf16", 24, True), ("f32", 7, True), ("bf16", 2048 + 8, True)])
def test_split_add_residual(kind, C, with_scale):
    """Unmerge fused with LayerScale and the residual add, bit for bit against the oracle's three separate tensor
    operations in the element type; also in place (out = residual)."""
    import torch
    from come_b200 import _lib
    from come_b200.token_merger import MergePlan
    from gpu_util import TORCH_DTYPE, to_dev, to_np
    import golden_inputs as gi
    from oracle import come_oracle as orc
    rng = np.random.default_rng(C)
    mask = rng.random((3, 144)) < 0.5
    plan = MergePlan(torch.from_numpy(mask).cuda(), _lib.Layout.two_d(5, 37, 37, 3, 3))
    _o, _off, rev, _w = orc.token_merge_2d_ragged(np.zeros((3, 1374, 1), np.float32), 5, 3, 3, 37, 37, mask)
    merged = gi.round_kind(rng.standard_normal((plan.total, C), dtype=np.float32), kind)
    x = gi.round_kind(rng.standard_normal((3 * 1374, C), dtype=np.float32), kind)
    gamma = gi.round_kind(0.01 + 0.5 * rng.random(C, dtype=np.float32), kind) if with_scale else None
    want = orc.token_split_residual(merged, rev, x, gamma, kind)
    xd = to_dev(x, kind)
    got = plan.split_add(to_dev(merged, kind), xd.reshape(3, 1374, C), None if gamma is None else to_dev(gamma, kind))
    assert got.shape == (3, 1374, C)
    np.testing.assert_array_equal(to_np(got).reshape(-1, C), want)
    plan.split_add(to_dev(merged, kind), xd, None if gamma is None else to_dev(gamma, kind), out=xd)  # in place
    np.testing.assert_array_equal(to_np(xd), want)


@pytest.mark.parametrize("idx", range(3))
def test_merge_layernorm_fixture_and_oracle(golden_dir, idx):
    """LayerNorm fused into the merge: bit for bit against the oracle (same summation order), within one unit in the last
    place against nn.LayerNorm + the reference's merge (fixture)."""
    import torch
    from come_b200 import _lib
    from come_b200.token_merger import MergePlan
    from gpu_util import TORCH_DTYPE, to_dev, to_np
    import golden_inputs as gi
    from oracle import come_oracle as orc
    z = np.load(os.path.join(golden_dir, "ln_merge.npz"))
    case = gi.LN_MERGE_CASES[idx]
    frames, H, W, gh, gw, start, C, kind = case
    x, gamma, beta, mask = gi.ln_merge_inputs(idx, case)
    ln = torch.nn.LayerNorm(C, eps=gi.LN_MERGE_EPS).cuda().to(TORCH_DTYPE[kind])
    with torch.no_grad():
        ln.weight.copy_(to_dev(gamma, kind))
        ln.bias.copy_(to_dev(beta, kind))
    plan = MergePlan(torch.from_numpy(mask).cuda(), _lib.Layout.two_d(start, H, W, gh, gw))
    got = to_np(plan.merge_layernorm(to_dev(x, kind), ln))
    want, _off, _rev, _w = orc.token_merge_2d(orc.layer_norm_rows(x, gamma, beta, gi.LN_MERGE_EPS, kind), start, gh, gw, H, W, mask)
    np.testing.assert_array_equal(got, orc._round_like(want, kind))
    tol = gi.ln_merge_tolerance(kind)
    gi.check_rows(got, z, f"l{idx}_out_", rtol=tol, atol=tol)


def test_merge_layernorm_headline_shape():
    """8 x 1374 x 1024 bfloat16 on the ragged 37 x 37 grid: fused kernel == LayerNorm oracle + merge oracle, bit for bit;
    shapes the fused kernel does not take are refused."""
    import torch
    from come_b200 import _lib
    from come_b200.token_merger import MergePlan
    from gpu_util import TORCH_DTYPE, to_dev, to_np
    import golden_inputs as gi
    from oracle import come_oracle as orc
    rng = np.random.default_rng(77)
    frames, C = 3, 1024
    x = gi.round_kind(rng.standard_normal((frames, 1374, C), dtype=np.float32) * 3 - 1, "bf16")
    gamma = gi.round_kind(1 + 0.3 * rng.standard_normal(C, dtype=np.float32), "bf16")
    beta = gi.round_kind(0.2 * rng.standard_normal(C, dtype=np.float32), "bf16")
    mask = rng.random((frames, 144)) < 0.5
    ln = torch.nn.LayerNorm(C, eps=1e-6).cuda().bfloat16()
    with torch.no_grad():
        ln.weight.copy_(to_dev(gamma, "bf16"))
        ln.bias.copy_(to_dev(beta, "bf16"))
    plan = MergePlan(torch.from_numpy(mask).cuda(), _lib.Layout.two_d(5, 37, 37, 3, 3))
    got = to_np(plan.merge_layernorm(to_dev(x, "bf16"), ln))
    want, _off, _rev, _w = orc.token_merge_2d_ragged(orc.layer_norm_rows(x, gamma, beta, 1e-6, "bf16"), 5, 3, 3, 37, 37, mask)
    np.testing.assert_array_equal(got, orc._round_like(want, "bf16"))
    wide = torch.zeros(frames, 1374, 4096, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError):
        plan.merge_layernorm(wide, torch.nn.LayerNorm(4096).cuda().bfloat16())


# ---- suffix tokens of jagged segments (come_suffix_add / come_suffix_split) ----------------------------------------
@pytest.mark.parametrize("kind", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("idx", range(len(gi.SUFFIX_CASES)))
def test_suffix_kernels_against_fixture(golden_dir, idx, kind):
    from come_b200.token_merger import JaggedTokens
    z = np.load(os.path.join(golden_dir, "suffix.npz"))
    case = gi.SUFFIX_CASES[idx]
    tokens, weight, offset, suffix = gi.suffix_inputs(idx, case)
    tokens, suffix = gi.round_kind(tokens, kind), gi.round_kind(suffix, kind)
    jag = JaggedTokens(tokens=to_dev(tokens, kind)[None], weight=to_dev(weight), offset=torch.from_numpy(offset).cuda())
    ext = jag.add_suffix(to_dev(suffix, kind))
    ref_tok, ref_w, ref_off = orc.jagged_add_suffix(tokens, weight, offset, suffix)
    assert ext.tokens.dtype == TORCH_DTYPE[kind] and ext.offset.dtype == torch.int64
    assert np.array_equal(to_np(ext.tokens[0]), ref_tok) and np.array_equal(to_np(ext.weight), ref_w)
    assert np.array_equal(to_np(ext.offset), ref_off)
    assert np.array_equal(to_np(ext.weight), z[f"s{idx}_weight"].astype(np.float32))
    assert np.array_equal(to_np(ext.offset), z[f"s{idx}_offset"].astype(np.int64))
    if kind == "f32":
        assert np.array_equal(to_np(ext.tokens[0]), z[f"s{idx}_tokens"])
    back, suf = ext.split_suffix(case[1])
    assert np.array_equal(to_np(back.tokens[0]), tokens) and np.array_equal(to_np(back.weight), weight)
    assert np.array_equal(to_np(back.offset), offset) and np.array_equal(to_np(suf), suffix)
    assert suf.shape == suffix.shape


def test_suffix_kernels_large_and_errors():
    """Frame-sized segments (the packed tokens of 8 half-merged frames + 4 suffix tokens each) against the PyTorch
    indexing path of the same container on CPU; errors as in the reference."""
    from come_b200 import _lib
    from come_b200.token_merger import JaggedTokens
    rng = np.random.default_rng(3)
    lens = [1374 - 8 * int(k) for k in rng.integers(0, 73, size=8)]
    P, C, T = sum(lens), 1024, 4
    tokens = gi.round_kind(rng.standard_normal((P, C), dtype=np.float32), "bf16")
    weight = rng.choice(np.array([1.0, 9.0], np.float32), size=P)
    offset = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    suffix = gi.round_kind(rng.standard_normal((8, T, C), dtype=np.float32), "bf16")
    cpu = JaggedTokens(torch.from_numpy(tokens).bfloat16()[None], torch.from_numpy(weight), torch.from_numpy(offset))
    gpu = JaggedTokens(cpu.tokens.cuda(), cpu.weight.cuda(), cpu.offset.cuda())
    ext_cpu, ext_gpu = cpu.add_suffix(torch.from_numpy(suffix).bfloat16()), gpu.add_suffix(torch.from_numpy(suffix).bfloat16().cuda())
    for a, b in ((ext_cpu.tokens, ext_gpu.tokens), (ext_cpu.weight, ext_gpu.weight), (ext_cpu.offset, ext_gpu.offset)):
        assert torch.equal(a, b.cpu())
    back_gpu, suf_gpu = ext_gpu.split_suffix(T)
    assert torch.equal(back_gpu.tokens.cpu(), cpu.tokens) and torch.equal(suf_gpu.cpu(), torch.from_numpy(suffix).bfloat16())
    assert torch.equal(back_gpu.offset.cpu(), cpu.offset) and torch.equal(back_gpu.weight.cpu(), cpu.weight)
    with pytest.raises(ValueError):
        gpu.add_suffix(torch.zeros(7, T, C, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        gpu.split_suffix(P)  # more than the total
    short = JaggedTokens(gpu.tokens[:, :6], gpu.weight[:6], torch.tensor([0, 5, 6], device="cuda"))
    with pytest.raises(ValueError):
        short.split_suffix(2)  # 4 <= 6 in total, but the second segment holds one token
    assert _lib.device_status() == 0
