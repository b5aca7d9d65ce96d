"""Failure paths and memory-safety substitutes, in forms that neither fault nor hang a GPU.

* the bounded wait of the attention kernel, exercised by the library's self-test (a barrier nothing arrives at, a
  limit of a fraction of a millisecond): the wait gives up, the status word is raised and reported, attention launches
  issued while it is raised return at once without touching their outputs, and clearing the word restores service;
* every merge mask of up to 8 groups, for group sizes 1, 2, 3 and 9, bit-exact against the oracle;
* outputs of merge, unmerge and attention placed between canary rows that must survive the launch.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import golden_inputs as gi
from gpu_util import to_dev, to_np
from oracle import clib, come_oracle as orc

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_is_reported():
    from come_b200 import _lib, flash_attn_fwd_cuda as fa
    from come_b200._torch_util import ptr, stream_ptr
    lib = _lib.lib()
    assert _lib.device_status(clear=True) == 0
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    ticks = 100_000
    _lib.check(lib.come_selftest_bounded_wait(ticks, ptr(waited), stream_ptr(waited.device)))
    torch.cuda.synchronize()  # the kernel returned by itself
    w = int(waited.item())
    assert ticks < w < 50 * ticks, w  # it waited out the limit (not -1 = "the barrier completed") and not much longer
    # the word is raised and reported through the C ABI
    v = C.c_uint32(0)
    rc = lib.come_device_status(C.byref(v), 0)
    assert rc == _lib.COME_ERR_DEVICE and v.value == 1 << 15
    assert "self-test" in _lib.last_error()
    with pytest.raises(RuntimeError, match="status word"):
        _lib.raise_on_device_error(clear=False)
    # an attention launch issued while the word is raised returns at once and leaves its outputs alone
    fa.set_backend(fa.BACKEND_TCGEN05)
    try:
        P, H, D = 700, 2, 64
        rng = np.random.default_rng(0)
        qkv = to_dev(rng.standard_normal((P, 3, H, D), dtype=np.float32), "bf16")
        cu = torch.tensor([0, P], dtype=torch.int32, device="cuda")
        out = torch.full((P, H, D), 7.0, dtype=torch.bfloat16, device="cuda")
        res, lse = fa.varlen_fwd_rows(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, P, None, D ** -0.5, 0, out_=out)
        torch.cuda.synchronize()
        assert res.data_ptr() == out.data_ptr() and bool((out == 7.0).all())
        # cleared: the same launch computes
        assert _lib.device_status(clear=True) == 1 << 15
        assert _lib.device_status(clear=False) == 0
        res, lse = fa.varlen_fwd_rows(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, P, None, D ** -0.5, 0, out_=out)
        want, _ = clib.attention_bias(to_np(qkv), None, np.array([0, P], np.int32), D ** -0.5)
        assert np.abs(to_np(res) - want).max() <= 2e-2
    finally:
        fa.set_backend(fa.BACKEND_AUTO)
        _lib.device_status(clear=True)
    with pytest.raises(RuntimeError, match="ticks"):
        _lib.check(lib.come_selftest_bounded_wait(1 << 40, None, None))


@pytest.mark.parametrize("G", [1, 2, 3, 9])
@pytest.mark.parametrize("M", range(1, 9))
def test_every_mask_of_up_to_8_groups(G, M):
    """All 2^M masks of M groups in one call (one frame per mask): offsets, rev_id, counts and features bit-exact."""
    from come_b200 import token_merger as tm
    start, Cc = 2, 8
    B = 1 << M
    mask = ((np.arange(B)[:, None] >> np.arange(M)[None, :]) & 1).astype(bool)
    rng = np.random.default_rng(100 * G + M)
    tokens = rng.standard_normal((B, start + M * G, Cc), dtype=np.float32)
    jag, rev = tm.func_token_merge(to_dev(tokens), start, G, torch.from_numpy(mask).cuda())
    out, off, rev_o, w = orc.token_merge(tokens, start, G, mask)
    np.testing.assert_array_equal(to_np(jag.offset), off)
    np.testing.assert_array_equal(to_np(rev), rev_o)
    np.testing.assert_array_equal(to_np(jag.weight), w)
    np.testing.assert_array_equal(to_np(jag.tokens[0]), out)
    back = tm.func_token_split(jag, rev, (1, B, start + M * G, Cc))
    np.testing.assert_array_equal(to_np(back).reshape(-1, Cc), orc.token_split(out, rev_o))


CANARY = 1234.5
PAD = 3  # canary rows in front of and behind every output


def _padded(rows, width, dtype):
    buf = torch.full((rows + 2 * PAD, width), CANARY, dtype=dtype, device="cuda")
    return buf, buf[PAD:PAD + rows]


def _pads_intact(buf, rows):
    return bool((buf[:PAD] == CANARY).all()) and bool((buf[PAD + rows:] == CANARY).all())


@pytest.mark.parametrize("kind,Cc", [("f32", 1024), ("bf16", 1024), ("f32", 20), ("f16", 7)])
def test_merge_and_unmerge_write_only_their_rows(kind, Cc):
    """Outputs embedded between canary rows (ragged 37x37 layout, half merged): the rows are right, the canaries survive."""
    from come_b200 import _lib
    from come_b200._torch_util import dtype_code, ptr, stream_ptr
    from come_b200.token_merger import MergePlan
    frames, start, H, W = 3, 5, 37, 37
    rng = np.random.default_rng(9)
    mask = rng.random((frames, 144)) < 0.5
    tokens = gi.round_kind(rng.standard_normal((frames, start + H * W, Cc), dtype=np.float32), kind)
    layout = _lib.Layout.two_d(start, H, W, 3, 3)
    plan = MergePlan(torch.from_numpy(mask).cuda(), layout)
    x = to_dev(tokens, kind)
    P, total = plan.total, frames * (start + H * W)
    lib, st = _lib.lib(), stream_ptr(x.device)
    buf, out = _padded(P, Cc, x.dtype)
    _lib.check(lib.come_merge(ptr(x), dtype_code(x.dtype), frames, Cc, C.byref(layout), ptr(plan._mask_u8),
                              ptr(plan.group_prefix), ptr(plan.offsets_i32), ptr(out), st))
    torch.cuda.synchronize()
    assert torch.equal(out, plan.merge(x)) and _pads_intact(buf, P)
    want, _, rev, _ = clib.token_merge_2d(tokens, start, 3, 3, H, W, mask, kind)
    np.testing.assert_array_equal(to_np(out), want)
    buf2, restored = _padded(total, Cc, x.dtype)
    _lib.check(lib.come_unmerge(ptr(out.contiguous()), ptr(plan.rev_id), total, Cc, dtype_code(x.dtype), ptr(restored), st))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(to_np(restored), want[rev])
    assert _pads_intact(buf2, total)


@pytest.mark.parametrize("lengths", [[1, 63, 129, 385], [798, 807]])
def test_attention_writes_only_its_rows(lengths):
    """Attention output and log-sum-exp embedded between canaries, lengths that leave ragged query and key tiles."""
    from come_b200 import flash_attn_fwd_cuda as fa
    fa.set_backend(fa.BACKEND_TCGEN05)
    try:
        H, D, P = 2, 64, sum(lengths)
        rng = np.random.default_rng(len(lengths))
        qkv = gi.round_kind(rng.standard_normal((P, 3, H, D), dtype=np.float32), "bf16")
        bias = gi.round_kind(np.log(np.where(rng.random(P) < 0.2, 9.0, 1.0)).astype(np.float32), "bf16")
        cu_np = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
        t, b = to_dev(qkv, "bf16"), to_dev(bias, "bf16")
        buf, out2d = _padded(P, H * D, torch.bfloat16)
        out = out2d.view(P, H, D)
        res, lse = fa.varlen_fwd_rows(t[:, 0], t[:, 1], t[:, 2], torch.from_numpy(cu_np).cuda(), max(lengths), b, D ** -0.5, 0, out_=out)
        torch.cuda.synchronize()
        want, want_lse = clib.attention_bias(qkv, bias, cu_np, D ** -0.5)
        assert np.abs(to_np(out) - want).max() <= 2e-2 and _pads_intact(buf, P)
        np.testing.assert_allclose(to_np(lse), want_lse, atol=2e-3, rtol=1e-3)
    finally:
        fa.set_backend(fa.BACKEND_AUTO)
    from come_b200 import _lib
    assert _lib.device_status(clear=True) == 0
