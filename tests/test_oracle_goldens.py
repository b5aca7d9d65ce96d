"""The CPU oracle against the reference: literal known-answer cases of the reference's tests and fixtures
written by running the reference itself (tests/golden/make_golden.py).  No GPU needed."""
import os

import numpy as np
import pytest

import golden_inputs as gi
import reference_cases as rc
from oracle import clib, come_oracle as orc

FEATURE_TOL = dict(rtol=1e-6, atol=1e-6)  # the reference's vectorised CPU sum may round once differently


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


@pytest.mark.parametrize("idx", range(len(rc.CASES_1D)))
@pytest.mark.parametrize("impl", ["numpy", "c"])
def test_reference_literals_1d(idx, impl):
    c = rc.as_arrays(rc.CASES_1D[idx])
    merge = orc.token_merge if impl == "numpy" else clib.token_merge
    split = orc.token_split if impl == "numpy" else clib.token_split
    out, off, rev, w = merge(c["tokens"], c["start_index"], c["group_size"], c["mask"])
    np.testing.assert_array_equal(out, c["out"])
    np.testing.assert_array_equal(off, c["offset"])
    np.testing.assert_array_equal(rev, c["rev"])
    np.testing.assert_array_equal(w, c["weight"])
    B, N, C = c["tokens"].shape
    np.testing.assert_array_equal(split(out, rev).reshape(B, N, C), c["restored"])


@pytest.mark.parametrize("idx", range(len(rc.CASES_2D)))
@pytest.mark.parametrize("impl", ["numpy", "numpy-ragged", "c"])
def test_reference_literals_2d(idx, impl):
    c = rc.as_arrays(rc.CASES_2D[idx])
    fn = {"numpy": orc.token_merge_2d, "numpy-ragged": orc.token_merge_2d_ragged, "c": clib.token_merge_2d}[impl]
    out, off, rev, w = fn(c["tokens"], c["start_index"], c["gh"], c["gw"], c["H"], c["W"], c["mask"])
    np.testing.assert_array_equal(out, c["out"])
    np.testing.assert_array_equal(off, c["offset"])
    np.testing.assert_array_equal(rev, c["rev"])
    np.testing.assert_array_equal(w, c["weight"])
    B, N, C = c["tokens"].shape
    np.testing.assert_array_equal(orc.token_split(out, rev).reshape(B, N, C), c["restored"])


@pytest.mark.parametrize("idx", range(len(rc.RANDOM_CONFIGS_1D)))
@pytest.mark.parametrize("kind", ["f32", "bf16"])
def test_merge_1d_fixture(golden_dir, idx, kind):
    z = _load(golden_dir, "merge_1d.npz")
    cfg = rc.RANDOM_CONFIGS_1D[idx]
    tokens, mask = gi.merge1d_inputs(idx, cfg, kind)
    B, M, G, S, C = cfg
    key = f"c{idx}_{kind}_"
    tol = FEATURE_TOL if kind == "f32" else dict(rtol=8e-3, atol=8e-3)
    for name, impl in (("numpy", orc.token_merge), ("c", lambda *a: clib.token_merge(*a, kind=kind))):
        out, off, rev, w = impl(tokens, S, G, mask)
        if name == "numpy" and kind != "f32":
            out = orc._round_like(out, kind)
        np.testing.assert_array_equal(off, z[key + "offset"])
        np.testing.assert_array_equal(rev, z[key + "rev"].astype(np.int64))
        np.testing.assert_array_equal(w, z[key + "weight"].astype(np.float32))
        gi.check_rows(out, z, key + "out_", **tol)
        gi.check_rows(orc.token_split(out, rev), z, key + "res_", **tol)
        if name == "numpy":
            first = out
        else:
            np.testing.assert_array_equal(out, first)  # the two oracles agree bit for bit


@pytest.mark.parametrize("idx", range(len(rc.RANDOM_CONFIGS_2D)))
def test_merge_2d_fixture(golden_dir, idx):
    z = _load(golden_dir, "merge_2d.npz")
    cfg = rc.RANDOM_CONFIGS_2D[idx]
    tokens, mask = gi.merge2d_inputs(idx, cfg)
    B, H, W, gh, gw, S, C = cfg
    key = f"c{idx}_"
    a = orc.token_merge_2d(tokens, S, gh, gw, H, W, mask)
    b = clib.token_merge_2d(tokens, S, gh, gw, H, W, mask)
    c = orc.token_merge_2d_ragged(tokens, S, gh, gw, H, W, mask)
    for out, off, rev, w in (a, b, c):
        np.testing.assert_array_equal(off, z[key + "offset"])
        np.testing.assert_array_equal(rev, z[key + "rev"].astype(np.int64))
        np.testing.assert_array_equal(w, z[key + "weight"].astype(np.float32))
        gi.check_rows(out, z, key + "out_", **FEATURE_TOL)
        np.testing.assert_array_equal(out, a[0])


@pytest.mark.parametrize("name", sorted(gi.SELECT_CASES))
def test_select_fixture(golden_dir, name):
    z = _load(golden_dir, "select.npz")
    spec = gi.SELECT_CASES[name]
    conf = gi.select_inputs(name)
    shape = tuple(z[name + "_shape"])
    want = np.unpackbits(z[name + "_mask"])[: shape[0] * shape[1]].reshape(shape).astype(bool)
    scope = "batch" if spec["cls"] == "2d" else "frame"
    args = (conf, spec["B"], spec["S"], spec["H"], spec["W"], spec["gh"], spec["gw"], spec["thr"], spec["mode"], scope,
            spec["kind"])
    np.testing.assert_array_equal(orc.select_windows(*args), want)
    np.testing.assert_array_equal(clib.select_windows(*args), want)


def test_quantile_matches_torch():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(7)
    for n in (1, 2, 3, 7, 144, 145, 1152, 14400):
        for q in (0.0, 0.1, 0.25, 0.5, 0.75, 0.9, 1.0, 0.333):
            v = rng.random(n, dtype=np.float32)
            want = torch.quantile(torch.from_numpy(v), q).item()
            assert float(orc.quantile_linear(v, q)) == want, (n, q)


@pytest.mark.parametrize("idx", range(len(rc.ATTENTION_CASES) + len(gi.EXTRA_ATTENTION_CASES)))
def test_attention_fixture(golden_dir, idx):
    z = _load(golden_dir, "attention.npz")
    case = (list(rc.ATTENTION_CASES) + list(gi.EXTRA_ATTENTION_CASES))[idx]
    seq_lens, H, D, kind = case
    qkv, bias, cu = gi.attention_inputs(idx, case)
    scale = 1.0 / (D ** 0.5)
    want = z[f"a{idx}_out"]
    out, lse = orc.attention_bias(qkv[:, 0], qkv[:, 1], qkv[:, 2], bias, cu, scale)
    np.testing.assert_allclose(out, want, rtol=1e-5, atol=2e-6)
    out_c, lse_c = clib.attention_bias(qkv, bias, cu, scale)
    np.testing.assert_allclose(out_c, want, rtol=1e-4, atol=5e-6)
    np.testing.assert_allclose(lse_c, lse, rtol=1e-5, atol=1e-5)


def test_cfg1_chain_fixture(golden_dir):
    """Standalone op chain of the headline configuration: 8 x (5 + 37x37) tokens, 3x3 windows, 50 % per frame."""
    z = _load(golden_dir, "cfg1_chain.npz")
    tokens, conf = gi.cfg1_inputs()
    mask = orc.select_windows(conf, 8, 1, 37, 37, 3, 3, 0.5, "pairwise-rank", "frame", "f32")
    want_mask = np.unpackbits(z["mask"])[: 8 * 144].reshape(8, 144).astype(bool)
    np.testing.assert_array_equal(mask, want_mask)
    assert (mask.sum(axis=1) == 72).all()
    np.testing.assert_array_equal(clib.select_windows(conf, 8, 1, 37, 37, 3, 3, 0.5, "pairwise-rank", "frame"), want_mask)
    out, off, rev, w = clib.token_merge_2d(tokens, 5, 3, 3, 37, 37, mask)
    assert out.shape == (8 * 798, 1024)
    np.testing.assert_array_equal(off, z["offset"])
    np.testing.assert_array_equal(rev, z["rev"].astype(np.int64))
    np.testing.assert_array_equal(w, z["weight"].astype(np.float32))
    gi.check_rows(out, z, "out_", **FEATURE_TOL)
    gi.check_rows(clib.token_split(out, rev), z, "res_", **FEATURE_TOL)
    # numpy twin on a channel slice (keeps the CPU suite fast)
    o2 = orc.token_merge_2d_ragged(tokens[:, :, :64], 5, 3, 3, 37, 37, mask)
    np.testing.assert_array_equal(o2[0], out[:, :64])
    np.testing.assert_array_equal(o2[2], rev)


def _prepare_fixture(z, i, kind):
    """q, k of the fixture (stored as 16-bit patterns of the run dtype) as float32."""
    raw = z[f"p{i}_qk"]
    if kind == "f16":
        return raw.view(np.float16).astype(np.float32)
    return (raw.astype(np.uint32) << 16).view(np.float32)


def prepare_tolerance(ref, kind):
    """Bound used for LayerNorm + rotation against the reference: the reference's CPU LayerNorm sums its
    statistics in another order, so a normalised value next to a rounding boundary may move by one unit in the
    last place of the run dtype, and the rotation mixes two such values: 2 ulp at the head vector's largest
    magnitude (bfloat16 ulp 2^-7 relative, float16 2^-10)."""
    return 2.0 * np.abs(ref).max(axis=-1, keepdims=True) * (2.0 ** -7 if kind == "bf16" else 2.0 ** -10)


@pytest.mark.parametrize("idx", range(len(gi.PREPARE_CASES)))
def test_prepare_fixture(golden_dir, idx):
    z = _load(golden_dir, "prepare.npz")
    case = gi.PREPARE_CASES[idx]
    P, H, D, kind, use_norm, use_rope = case
    qkv, params, pos = gi.prepare_inputs(idx, case)
    cos_t, sin_t = orc.rope_tables(D // 2, gi.PREPARE_MAX_POSITION, 100.0, kind)
    out = orc.qkv_prepare(qkv, *(params if use_norm else [None] * 4), gi.PREPARE_EPS, pos if use_rope else None,
                          cos_t, sin_t, kind)
    ref = _prepare_fixture(z, idx, kind)
    assert np.all(np.abs(out[:, :2] - ref) <= prepare_tolerance(ref, kind))
    mismatched = np.mean(out[:, :2] != ref)
    assert mismatched < (1e-3 if use_norm else 1e-12), mismatched  # rotation alone is bit-exact
    np.testing.assert_array_equal(out[:, 2], qkv[:, 2])


@pytest.mark.parametrize("idx", range(len(gi.POSITION_CASES)))
def test_positions_fixture(golden_dir, idx):
    z = _load(golden_dir, "prepare.npz")
    case = gi.POSITION_CASES[idx]
    frames, H, W, gh, gw, start = case
    got = orc.packed_positions(gi.position_mask(idx, case), start, H, W, gh, gw)
    np.testing.assert_array_equal(got, z[f"pos{idx}"].astype(np.int64))


def test_positions_are_window_centres():
    """Specials at (0, 0), kept patches at (y + 1, x + 1), a merged 3x3 window at its centre; ragged 37x37 grid."""
    rng = np.random.default_rng(3)
    mask = rng.random((2, 144)) < 0.5
    pos = orc.packed_positions(mask, 5, 37, 37, 3, 3)
    _out, off, rev, w = orc.token_merge_2d_ragged(np.zeros((2, 1374, 1), np.float32), 5, 3, 3, 37, 37, mask)
    assert pos.shape == (off[-1], 2)
    rev = rev.reshape(2, 1374)
    for b in range(2):
        assert (pos[rev[b, :5]] == 0).all()
        for y, x in ((0, 0), (36, 36), (10, 36), (36, 3), (17, 20)):
            row = rev[b, 5 + y * 37 + x]
            if y < 36 and x < 36 and mask[b, (y // 3) * 12 + x // 3]:
                assert tuple(pos[row]) == (3 * (y // 3) + 2, 3 * (x // 3) + 2) and w[row] == 9
            else:
                assert tuple(pos[row]) == (y + 1, x + 1) and w[row] == 1


@pytest.mark.parametrize("idx", range(len(gi.LN_MERGE_CASES)))
def test_ln_merge_fixture(golden_dir, idx):
    """LayerNorm over the channels followed by the 2-D merge, against nn.LayerNorm + the reference's merge on CPU."""
    z = _load(golden_dir, "ln_merge.npz")
    case = gi.LN_MERGE_CASES[idx]
    frames, H, W, gh, gw, start, C, kind = case
    x, gamma, beta, mask = gi.ln_merge_inputs(idx, case)
    out, _off, _rev, _w = orc.token_merge_2d(orc.layer_norm_rows(x, gamma, beta, gi.LN_MERGE_EPS, kind), start, gh, gw, H, W, mask)
    tol = gi.ln_merge_tolerance(kind)
    gi.check_rows(orc._round_like(out, kind), z, f"l{idx}_out_", rtol=tol, atol=tol)


@pytest.mark.parametrize("idx", range(len(gi.BLOCK_CASES)))
def test_block_fixture(golden_dir, idx):
    """One transformer block on unmerged tokens against the reference model's own Block (float32, CPU)."""
    z = _load(golden_dir, "block.npz")
    case = gi.BLOCK_CASES[idx]
    frames, side, start, C, heads, mlp_ratio, qk_norm, use_rope, ls_init = case
    x, params, pos = gi.block_inputs(idx, case)
    N = x.shape[1]
    cos_t = sin_t = None
    if use_rope:
        cos_t, sin_t = orc.rope_tables(C // heads // 2, side + 1, 100.0, "f32")
    cu = np.arange(frames + 1, dtype=np.int64) * N
    out = orc.jagged_block(x.reshape(-1, C), np.ones(frames * N, np.float32), cu, pos.reshape(-1, 2),
                           dict(params, norm_eps=1e-5, qk_norm_eps=1e-5), heads, cos_t, sin_t)
    gi.check_rows(out, z, f"b{idx}_out_", rtol=gi.BLOCK_TOLERANCE, atol=gi.BLOCK_TOLERANCE)


def test_fused_aggregator_without_merging_is_the_block_chain():
    """With an all-False mask the merged forward pass is the plain alternating chain of blocks on the dense tokens
    (in the ragged layout's order), and a retained layer is [frame tokens | global tokens]."""
    rng = np.random.default_rng(77)
    B, S, side, start, C, heads = 1, 2, 4, 2, 32, 1
    N = start + side * side
    tokens = rng.standard_normal((B, S, N, C), dtype=np.float32)
    fp = [gi.block_params(rng, C, heads, 2.0, True, 0.5) for _ in range(2)]
    gp = [gi.block_params(rng, C, heads, 2.0, True, 0.5) for _ in range(2)]
    mask = np.zeros((B * S, 4), bool)
    out = orc.fused_aggregator(tokens, mask, start, side, side, 2, 2, fp, gp, heads, retain_layers={1})
    assert sorted(out) == [1] and out[1].shape == (B, S, N, 2 * C)
    # the same chain by hand, in the dense order (the attention is permutation-equivariant given the positions)
    ys, xs = np.meshgrid(np.arange(side), np.arange(side), indexing="ij")
    pos = np.zeros((N, 2), np.int64)
    pos[start:, 0], pos[start:, 1] = ys.reshape(-1) + 1, xs.reshape(-1) + 1
    pos = np.tile(pos, (B * S, 1))
    cos_t, sin_t = orc.rope_tables(C // heads // 2, side + 2, 100.0, "bf16")
    ones = np.ones(B * S * N, np.float32)
    frame_cu = np.arange(B * S + 1) * N
    global_cu = np.arange(B + 1) * S * N
    x = tokens.reshape(-1, C)
    for layer in range(2):
        x = orc.jagged_block(x, ones, frame_cu, pos, fp[layer], heads, cos_t, sin_t)
        frame_x = x
        x = orc.jagged_block(x, ones, global_cu, pos, gp[layer], heads, cos_t, sin_t)
    expect = np.concatenate([frame_x, x], axis=-1).reshape(B, S, N, 2 * C)
    np.testing.assert_allclose(out[1], expect, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("idx", range(len(gi.SUFFIX_CASES)))
def test_suffix_fixture(golden_dir, idx):
    """add_suffix / split_suffix of the jagged container against the reference's own class on CPU."""
    z = _load(golden_dir, "suffix.npz")
    case = gi.SUFFIX_CASES[idx]
    tokens, weight, offset, suffix = gi.suffix_inputs(idx, case)
    tok, w, off = orc.jagged_add_suffix(tokens, weight, offset, suffix)
    assert np.array_equal(tok, z[f"s{idx}_tokens"]) and np.array_equal(w, z[f"s{idx}_weight"].astype(np.float32))
    assert np.array_equal(off, z[f"s{idx}_offset"].astype(np.int64))
    b_tok, b_w, b_off, b_suf = orc.jagged_split_suffix(tok, w, off, case[1])
    assert np.array_equal(b_tok, tokens) and np.array_equal(b_w, weight)
    assert np.array_equal(b_off, offset) and np.array_equal(b_suf, suffix)


def test_suffix_known_answers_and_errors():
    """The literal cases of the reference's suffix test (two segments [a, b | c], T = 2) and its error conditions."""
    tok, w, off = orc.jagged_add_suffix(np.array([[1.], [2.], [3.]], np.float32), np.array([4., 1., 1.], np.float32), [0, 2, 3],
                                        np.array([[[10.], [20.]], [[30.], [40.]]], np.float32))
    assert tok[:, 0].tolist() == [1., 2., 10., 20., 3., 30., 40.]
    assert w.tolist() == [4., 1., 1., 1., 1., 1., 1.] and off.tolist() == [0, 4, 7]
    with pytest.raises(ValueError):
        orc.jagged_add_suffix(tok, w, off, np.zeros((3, 1, 1), np.float32))
    with pytest.raises(ValueError):
        orc.jagged_split_suffix(tok, w, off, 4)       # more than the total
    with pytest.raises(ValueError):  # 4 <= 6 in total, but the second segment holds one token
        orc.jagged_split_suffix(np.zeros((6, 1), np.float32), np.ones(6, np.float32), [0, 5, 6], 2)


def test_attention_combine_is_attention_over_the_union_of_keys():
    """The oracle's merge of two partial attention results reproduces attention over all keys (float32)."""
    rng = np.random.default_rng(8)
    P, rows, H, D = 90, 40, 2, 16
    qkv = rng.standard_normal((P, 3, H, D), dtype=np.float32)
    bias = np.log(np.where(rng.random(P) < 0.3, 9.0, 1.0)).astype(np.float32)
    scale = D ** -0.5
    full, full_lse = orc.attention_bias(qkv[:, 0], qkv[:, 1], qkv[:, 2], bias, np.array([0, P], np.int32), scale)
    parts = []
    for lo, hi in ((0, rows), (rows, P)):  # the first `rows` queries against each block of keys
        s = np.einsum("ihd,jhd->hij", qkv[:rows, 0], qkv[lo:hi, 1]) * scale + bias[None, None, lo:hi]
        m = s.max(-1, keepdims=True)
        p = np.exp(s - m)
        l = p.sum(-1, keepdims=True)
        parts.append((np.einsum("hij,jhd->ihd", p / l, qkv[lo:hi, 2]).astype(np.float32), (m + np.log(l))[:, :, 0].astype(np.float32)))
    out, lse = orc.attention_combine(parts[0][0], parts[0][1], parts[1][0], parts[1][1])
    np.testing.assert_allclose(out, full[:rows], atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(lse, full_lse[:, :rows], atol=2e-6, rtol=1e-5)


def test_torch_cpu_attention_matches_the_c_oracle():
    """The PyTorch-operator restatement of the biased attention (the timed CPU baseline) against the C oracle."""
    from oracle import torch_path
    rng = np.random.default_rng(12)
    lengths = [5, 130, 64, 1]
    P, H, D = sum(lengths), 3, 64
    qkv = rng.standard_normal((P, 3, H, D), dtype=np.float32)
    bias = np.log(np.where(rng.random(P) < 0.3, 9.0, 1.0)).astype(np.float32)
    cu = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    for b in (bias, None):
        want, want_lse = clib.attention_bias(qkv, b, cu, D ** -0.5)
        got, got_lse = torch_path.attention_bias(qkv, b, cu, D ** -0.5)
        np.testing.assert_allclose(got, want, atol=2e-6, rtol=1e-5)
        np.testing.assert_allclose(got_lse, want_lse, atol=2e-6, rtol=1e-5)
    part, part_lse = torch_path.attention_bias(qkv, bias, cu[:2 + 1][1:], D ** -0.5, 10, 50)  # rows 10..49 of the 130-row segment
    full, full_lse = clib.attention_bias(qkv, bias, cu, D ** -0.5)
    np.testing.assert_allclose(part[5 + 10:5 + 50], full[5 + 10:5 + 50], atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(part_lse[:, 5 + 10:5 + 50], full_lse[:, 5 + 10:5 + 50], atol=2e-6, rtol=1e-5)


def test_n_way_attention_merge_agrees_with_the_pairwise_one():
    """``attention_combine_parts`` with two shares is ``attention_combine``; with more shares it reproduces attention over the
    union of the key sets (numpy float64 reference on a small case)."""
    from oracle import come_oracle as orc
    rng = np.random.default_rng(11)
    rows, H, D, kv, S = 7, 2, 8, 40, 4
    q = rng.standard_normal((rows, H, D)).astype(np.float32)
    k = rng.standard_normal((kv, H, D)).astype(np.float32)
    v = rng.standard_normal((kv, H, D)).astype(np.float32)

    def attend(lo, hi):
        s = np.einsum("ihd,jhd->hij", q.astype(np.float64), k[lo:hi].astype(np.float64))
        m = s.max(-1, keepdims=True)
        p = np.exp(s - m)
        l = p.sum(-1, keepdims=True)
        return np.einsum("hij,jhd->ihd", p / l, v[lo:hi].astype(np.float64)).astype(np.float32), (m + np.log(l))[:, :, 0].astype(np.float32)

    parts = [attend(i * 10, (i + 1) * 10) for i in range(S)]
    outs, lses = np.stack([p[0] for p in parts]), np.stack([p[1] for p in parts])
    out, lse = orc.attention_combine_parts(outs, lses)
    want, want_lse = attend(0, kv)
    np.testing.assert_allclose(out, want, atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(lse, want_lse, atol=2e-6, rtol=1e-6)
    two, two_lse = orc.attention_combine_parts(outs[:2], lses[:2])
    ref, ref_lse = orc.attention_combine(outs[0], lses[0], outs[1], lses[1])
    np.testing.assert_allclose(two, ref, atol=1e-7, rtol=1e-6)
    np.testing.assert_allclose(two_lse, ref_lse, atol=1e-6, rtol=1e-6)
