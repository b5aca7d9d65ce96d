"""Pre-attention preparation on the GPU (come_qkv_prepare, come_packed_positions) against the oracle, bit for bit,
and against fixtures written by the reference's prepare_packed_self_attention_qkv + rotary module on CPU."""
import os

import numpy as np
import pytest
import torch

import golden_inputs as gi
from gpu_util import TORCH_DTYPE, to_dev, to_np
from oracle import come_oracle as orc
from test_oracle_goldens import _prepare_fixture, prepare_tolerance

pytestmark = pytest.mark.gpu


def _norm(D, gamma, beta, kind):
    n = torch.nn.LayerNorm(D, eps=gi.PREPARE_EPS).cuda().to(TORCH_DTYPE[kind])
    with torch.no_grad():
        n.weight.copy_(to_dev(gamma, kind))
        n.bias.copy_(to_dev(beta, kind))
    return n


def _run(qkv, params, pos, kind, use_norm, use_rope, weight=None, max_position=gi.PREPARE_MAX_POSITION):
    from come_b200.qkv import RotaryPositionEmbedding2D, prepare_packed_self_attention_qkv
    D = qkv.shape[-1]
    qn = _norm(D, params[0], params[1], kind) if use_norm else torch.nn.Identity()
    kn = _norm(D, params[2], params[3], kind) if use_norm else torch.nn.Identity()
    rope = RotaryPositionEmbedding2D(100.0, max_position=max_position) if use_rope else None
    t = to_dev(qkv, kind)
    p = torch.from_numpy(pos).cuda()[None] if use_rope else None
    w = None if weight is None else torch.from_numpy(weight).cuda()
    res = prepare_packed_self_attention_qkv(t, qn, kn, rope, p, TORCH_DTYPE[kind], weight=w)
    if weight is None:
        assert res is t  # in place, like the reference's inference branch
        return to_np(t), None
    assert res[0] is t
    return to_np(t), to_np(res[1])


@pytest.mark.parametrize("idx", range(len(gi.PREPARE_CASES)))
def test_prepare_fixture_and_oracle(golden_dir, idx):
    z = np.load(os.path.join(golden_dir, "prepare.npz"))
    case = gi.PREPARE_CASES[idx]
    P, H, D, kind, use_norm, use_rope = case
    qkv, params, pos = gi.prepare_inputs(idx, case)
    got, _ = _run(qkv, params, pos, kind, use_norm, use_rope)
    cos_t, sin_t = orc.rope_tables(D // 2, gi.PREPARE_MAX_POSITION, 100.0, kind)
    want = orc.qkv_prepare(qkv, *(params if use_norm else [None] * 4), gi.PREPARE_EPS, pos if use_rope else None,
                           cos_t, sin_t, kind)
    np.testing.assert_array_equal(got, want)  # same order of float32 operations and roundings: bit-exact
    ref = _prepare_fixture(z, idx, kind)
    assert np.all(np.abs(got[:, :2] - ref) <= prepare_tolerance(ref, kind))
    assert np.mean(got[:, :2] != ref) < (1e-3 if use_norm else 1e-12)


@pytest.mark.parametrize("P,H,D,kind", [(6384, 16, 64, "bf16"), (1, 16, 64, "bf16"), (5, 8, 128, "f16"),
                                        (1031, 12, 64, "f16"), (77, 16, 32, "bf16")])
def test_prepare_oracle_sizes(P, H, D, kind):
    rng = np.random.default_rng(P + H)
    qkv = gi.round_kind(rng.standard_normal((P, 3, H, D), dtype=np.float32) * 2 - 0.5, kind)
    params = [gi.round_kind(1 + 0.3 * rng.standard_normal(D, dtype=np.float32), kind),
              gi.round_kind(0.2 * rng.standard_normal(D, dtype=np.float32), kind),
              gi.round_kind(1 + 0.3 * rng.standard_normal(D, dtype=np.float32), kind),
              gi.round_kind(0.2 * rng.standard_normal(D, dtype=np.float32), kind)]
    pos = rng.integers(0, 38, size=(P, 2)).astype(np.int64)
    weight = np.where(rng.random(P) < 0.3, np.float32(9), np.float32(1)).astype(np.float32)
    got, bias = _run(qkv, params, pos, kind, True, True, weight=weight)
    cos_t, sin_t = orc.rope_tables(D // 2, 38, 100.0, kind)
    want = orc.qkv_prepare(qkv, *params, gi.PREPARE_EPS, pos, cos_t, sin_t, kind)
    np.testing.assert_array_equal(got, want)
    np.testing.assert_array_equal(bias, orc.perkey_bias_from_weight(weight, kind))


def test_prepare_empty_and_errors():
    from come_b200 import _lib
    from come_b200.qkv import RotaryPositionEmbedding2D, prepare_packed_self_attention_qkv
    empty = torch.empty(0, 3, 16, 64, device="cuda", dtype=torch.bfloat16)
    ln = torch.nn.LayerNorm(64).cuda().bfloat16()
    assert prepare_packed_self_attention_qkv(empty, ln, ln, None, None, torch.bfloat16) is empty
    with pytest.raises(RuntimeError):  # run dtype mismatch
        prepare_packed_self_attention_qkv(torch.zeros(4, 3, 16, 64, device="cuda"), ln, ln, None, None, torch.bfloat16)
    with pytest.raises(NotImplementedError):  # float32 is not an attention dtype
        prepare_packed_self_attention_qkv(torch.zeros(4, 3, 16, 64, device="cuda"), torch.nn.Identity(),
                                          torch.nn.Identity(), None, None, torch.float32)
    with pytest.raises(NotImplementedError):  # head_dim outside the supported set
        prepare_packed_self_attention_qkv(torch.zeros(4, 3, 16, 48, device="cuda", dtype=torch.bfloat16),
                                          torch.nn.Identity(), torch.nn.Identity(), None, None, torch.bfloat16)
    with pytest.raises(RuntimeError):  # not contiguous
        prepare_packed_self_attention_qkv(torch.zeros(4, 6, 16, 64, device="cuda", dtype=torch.bfloat16)[:, ::2],
                                          ln, ln, None, None, torch.bfloat16)
    # a position beyond the rotary table is clamped and reported through the device status word
    _lib.device_status(clear=True)
    t = torch.zeros(4, 3, 16, 64, device="cuda", dtype=torch.bfloat16)
    pos = torch.tensor([[0, 1], [2, 99], [3, 3], [1, 1]], device="cuda")
    prepare_packed_self_attention_qkv(t, ln, ln, RotaryPositionEmbedding2D(100.0, max_position=16), pos, torch.bfloat16)
    assert _lib.device_status(clear=True) == 1 << 16
    assert _lib.device_status(clear=True) == 0


@pytest.mark.parametrize("idx", range(len(gi.POSITION_CASES)))
def test_positions_fixture(golden_dir, idx):
    from come_b200 import _lib
    from come_b200.token_merger import MergePlan
    z = np.load(os.path.join(golden_dir, "prepare.npz"))
    case = gi.POSITION_CASES[idx]
    frames, H, W, gh, gw, start = case
    mask = gi.position_mask(idx, case)
    plan = MergePlan(torch.from_numpy(mask).cuda(), _lib.Layout.two_d(start, H, W, gh, gw))
    np.testing.assert_array_equal(to_np(plan.positions()), z[f"pos{idx}"].astype(np.int64))


def test_positions_ragged_grid():
    from come_b200 import _lib
    from come_b200.token_merger import MergePlan
    rng = np.random.default_rng(11)
    mask = rng.random((8, 144)) < 0.5
    plan = MergePlan(torch.from_numpy(mask).cuda(), _lib.Layout.two_d(5, 37, 37, 3, 3))
    np.testing.assert_array_equal(to_np(plan.positions()), orc.packed_positions(mask, 5, 37, 37, 3, 3))


class _Attention(torch.nn.Module):
    """Stand-in for the model's attention block: the attributes the reference's wrapper reads."""

    def __init__(self, dim, heads):
        super().__init__()
        self.num_heads, self.head_dim = heads, dim // heads
        self.scale = self.head_dim ** -0.5
        self.qkv = torch.nn.Linear(dim, 3 * dim)
        self.q_norm = torch.nn.LayerNorm(self.head_dim)
        self.k_norm = torch.nn.LayerNorm(self.head_dim)
        self.attn_drop = torch.nn.Dropout(0.0)
        self.proj = torch.nn.Linear(dim, dim)
        self.proj_drop = torch.nn.Dropout(0.0)
        self.rope = type("Rope", (), {"base_frequency": 100.0})()


def test_jagged_attention_module():
    """JaggedAttention_w_Bias = qkv GEMM -> prepare kernel -> biased attention kernel -> proj GEMM; checked against the
    oracle's prepare + attention applied to the same GEMM output (bfloat16, 2e-2 absolute on the attention output)."""
    from come_b200.bias_attention import JaggedAttention_w_Bias
    from come_b200.token_merger import JaggedTokens
    torch.manual_seed(3)
    dim, heads = 128, 2
    mod = JaggedAttention_w_Bias(_Attention(dim, heads).cuda(), "bf16").eval()
    seq = [130, 57, 300]
    P = sum(seq)
    rng = np.random.default_rng(8)
    tokens = torch.from_numpy(rng.standard_normal((1, P, dim), dtype=np.float32)).cuda().bfloat16()
    weight = torch.from_numpy(np.where(rng.random(P) < 0.3, 9.0, 1.0).astype(np.float32)).cuda()
    offset = torch.tensor(np.concatenate([[0], np.cumsum(seq)]), dtype=torch.int64, device="cuda")
    pos = torch.from_numpy(rng.integers(0, 38, size=(1, P, 2))).cuda()
    with torch.no_grad():
        out = mod(JaggedTokens(tokens=tokens, weight=weight, offset=offset), pos=pos)
        qkv = mod.attn.qkv(tokens[0]).reshape(P, 3, heads, dim // heads)
    assert out.tokens.shape == (1, P, dim) and out.weight is weight and out.offset is offset
    a = mod.attn
    cos_t, sin_t = orc.rope_tables(dim // heads // 2, 256, 100.0, "bf16")
    prepared = orc.qkv_prepare(to_np(qkv), to_np(a.q_norm.weight), to_np(a.q_norm.bias), to_np(a.k_norm.weight),
                               to_np(a.k_norm.bias), a.q_norm.eps, to_np(pos)[0], cos_t, sin_t, "bf16")
    bias = orc.perkey_bias_from_weight(to_np(weight), "bf16")
    want, _lse = orc.attention_bias(prepared[:, 0], prepared[:, 1], prepared[:, 2], bias, to_np(offset).astype(np.int32),
                                    a.scale)
    with torch.no_grad():
        want_out = a.proj(torch.from_numpy(want.reshape(P, dim)).cuda().bfloat16())
    err = (out.tokens[0].float() - want_out.float()).abs().max().item()
    assert err <= 2e-2, err
    with pytest.raises(ValueError):
        JaggedAttention_w_Bias(_Attention(dim, heads), "fp32")


@pytest.mark.parametrize("is_global", [False, True])
def test_direct_attention_block(is_global):
    """The per-layer replacement of block.attn.forward: merge -> jagged biased attention -> split, against the oracle
    chain (merge, prepare, attention, split) around the same two GEMMs."""
    from come_b200 import _lib
    from come_b200.direct import DirectAttention
    from come_b200.token_merger import MergePlan
    torch.manual_seed(5)
    dim, heads, S, Hg, Wg = 128, 2, 3, 7, 8  # 3 frames of 5 + 7x8 tokens, 3x3 windows tile the top-left 6x6
    rng = np.random.default_rng(21)
    mask = rng.random((S, 4)) < 0.5
    plan = MergePlan(torch.from_numpy(mask).cuda(), _lib.Layout.two_d(5, Hg, Wg, 3, 3))
    N = 5 + Hg * Wg
    mod = DirectAttention(_Attention(dim, heads).cuda(), is_global=is_global).eval()
    x32 = rng.standard_normal((S, N, dim), dtype=np.float32)
    x = torch.from_numpy(x32).cuda()
    x_in = x.reshape(1, S * N, dim) if is_global else x
    with torch.no_grad():
        y = mod(x_in, plan, frames_per_scene=S)
    assert y.shape == x_in.shape and y.dtype == x.dtype
    # oracle chain
    a = mod.attn_op.attn
    xb = gi.round_kind(x32, "bf16")
    merged, off, rev, w = orc.token_merge_2d_ragged(xb, 5, 3, 3, Hg, Wg, mask)
    merged = gi.round_kind(merged, "bf16")
    P = merged.shape[0]
    with torch.no_grad():
        qkv = a.qkv(torch.from_numpy(merged).cuda().bfloat16()).reshape(P, 3, heads, dim // heads)
    cos_t, sin_t = orc.rope_tables(dim // heads // 2, 256, 100.0, "bf16")
    pos = orc.packed_positions(mask, 5, Hg, Wg, 3, 3)
    prepared = orc.qkv_prepare(to_np(qkv), to_np(a.q_norm.weight), to_np(a.q_norm.bias), to_np(a.k_norm.weight),
                               to_np(a.k_norm.bias), a.q_norm.eps, pos, cos_t, sin_t, "bf16")
    cu = off.astype(np.int32)
    if is_global:
        cu = cu[::S]
    att, _ = orc.attention_bias(prepared[:, 0], prepared[:, 1], prepared[:, 2], orc.perkey_bias_from_weight(w, "bf16"), cu,
                                a.scale)
    with torch.no_grad():
        proj = a.proj(torch.from_numpy(att.reshape(P, dim)).cuda().bfloat16())
    want = orc.token_split(to_np(proj), rev).reshape(x_in.shape)
    err = np.abs(to_np(y) - want).max()
    assert err <= 2e-2, err


def test_direct_attention_residual_branch():
    """x + ls1(attn(norm1(x))) through the fused kernels (LayerNorm inside the merge, LayerScale + residual inside the
    unmerge) against the oracle chain around the same two GEMMs."""
    from come_b200 import _lib
    from come_b200.direct import DirectAttention
    from come_b200.token_merger import MergePlan
    torch.manual_seed(6)
    dim, heads, S, Hg, Wg = 128, 2, 2, 6, 6
    rng = np.random.default_rng(31)
    mask = rng.random((S, 4)) < 0.5
    plan = MergePlan(torch.from_numpy(mask).cuda(), _lib.Layout.two_d(5, Hg, Wg, 3, 3))
    N = 5 + Hg * Wg
    mod = DirectAttention(_Attention(dim, heads).cuda(), is_global=False).eval()
    norm1 = torch.nn.LayerNorm(dim, eps=1e-6).cuda().bfloat16()
    with torch.no_grad():
        norm1.weight.copy_(torch.from_numpy(1 + 0.2 * rng.standard_normal(dim, dtype=np.float32)).cuda())
        norm1.bias.copy_(torch.from_numpy(0.1 * rng.standard_normal(dim, dtype=np.float32)).cuda())
    gamma = torch.from_numpy(gi.round_kind(0.5 * rng.random(dim, dtype=np.float32), "bf16")).cuda().bfloat16()
    xb = gi.round_kind(rng.standard_normal((S, N, dim), dtype=np.float32), "bf16")
    x = to_dev(xb, "bf16")
    with torch.no_grad():
        y = mod.forward_residual(x, plan, S, norm1, gamma)
    assert y.shape == x.shape and y.dtype == torch.bfloat16
    a = mod.attn_op.attn
    normed = orc.layer_norm_rows(xb, to_np(norm1.weight), to_np(norm1.bias), 1e-6, "bf16")
    merged, off, rev, w = orc.token_merge_2d_ragged(normed, 5, 3, 3, Hg, Wg, mask)
    merged = gi.round_kind(merged, "bf16")
    P = merged.shape[0]
    with torch.no_grad():
        qkv = a.qkv(torch.from_numpy(merged).cuda().bfloat16()).reshape(P, 3, heads, dim // heads)
    cos_t, sin_t = orc.rope_tables(dim // heads // 2, 256, 100.0, "bf16")
    prepared = orc.qkv_prepare(to_np(qkv), to_np(a.q_norm.weight), to_np(a.q_norm.bias), to_np(a.k_norm.weight),
                               to_np(a.k_norm.bias), a.q_norm.eps, orc.packed_positions(mask, 5, Hg, Wg, 3, 3), cos_t, sin_t, "bf16")
    att, _ = orc.attention_bias(prepared[:, 0], prepared[:, 1], prepared[:, 2], orc.perkey_bias_from_weight(w, "bf16"),
                                off.astype(np.int32), a.scale)
    with torch.no_grad():
        proj = a.proj(torch.from_numpy(att.reshape(P, dim)).cuda().bfloat16())
    want = orc.token_split_residual(to_np(proj), rev, xb.reshape(-1, dim), to_np(gamma), "bf16").reshape(S, N, dim)
    assert np.abs(to_np(y) - want).max() <= 2e-2
