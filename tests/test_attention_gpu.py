"""Biased variable-length attention parity on the GPU, through the C ABI.

Mirrors test/auto_test/test_flex_attention_bias.py:206-331 of the reference (segment-length sets, head shapes,
fp16 + bf16, zero-bias == plain kernel, bias has an effect) with the reference's tolerance (1e-2 abs/rel), plus
the 2e-2 absolute bar against the fp32 oracle on the post-merge lengths of the benchmark configurations.
Every case runs on both device kernels where both apply: the tcgen05 tensor-core kernel (head_dim 64) and the
CUDA-core kernel (any head_dim).
"""
import os

import numpy as np
import pytest
import torch

import golden_inputs as gi
import reference_cases as rc
from gpu_util import TORCH_DTYPE, to_dev, to_np
from oracle import clib

pytestmark = pytest.mark.gpu

ALL_CASES = list(rc.ATTENTION_CASES) + list(gi.EXTRA_ATTENTION_CASES)


@pytest.fixture
def backend():
    from come_b200 import flash_attn_fwd_cuda as fa

    def setter(b):
        fa.set_backend(b)

    yield setter
    fa.set_backend(fa.BACKEND_AUTO)


def _check_status():
    from come_b200 import _lib
    assert _lib.device_status(clear=True) == 0, "a tensor-core kernel wait ran out (device status word raised)"


def _backends_for(D):
    return ["cuda-core", "tcgen05"] if D == 64 else ["cuda-core"]


@pytest.mark.parametrize("idx", range(len(ALL_CASES)))
@pytest.mark.parametrize("which", ["cuda-core", "tcgen05"])
def test_bias_matches_reference_oracle(golden_dir, backend, idx, which):
    from come_b200 import flash_attn as api, flash_attn_fwd_cuda as fa
    seq_lens, H, D, kind = ALL_CASES[idx]
    if which not in _backends_for(D):
        pytest.skip("tensor-core kernel serves head_dim 64 only")
    backend(fa.BACKEND_TCGEN05 if which == "tcgen05" else fa.BACKEND_CUDA_CORE)
    z = np.load(os.path.join(golden_dir, "attention.npz"))
    qkv, bias, cu = gi.attention_inputs(idx, ALL_CASES[idx])
    want = z[f"a{idx}_out"]
    out = api.flash_attn_varlen_qkvpacked_func_w_perkey_bias(
        to_dev(qkv, kind), torch.from_numpy(cu).cuda(), max(seq_lens), perkey_bias=to_dev(bias, kind),
        softmax_scale=1.0 / (D ** 0.5))
    assert isinstance(out, torch.Tensor) and tuple(out.shape) == (sum(seq_lens), H, D)
    assert out.dtype == TORCH_DTYPE[kind]
    np.testing.assert_allclose(to_np(out), want, atol=rc.ATTENTION_ATOL, rtol=rc.ATTENTION_RTOL)
    _check_status()


@pytest.mark.parametrize("which", ["cuda-core", "tcgen05"])
@pytest.mark.parametrize("kind", ["f16", "bf16"])
def test_zero_bias_matches_plain_and_lse(backend, which, kind):
    from come_b200 import flash_attn as api, flash_attn_fwd_cuda as fa
    backend(fa.BACKEND_TCGEN05 if which == "tcgen05" else fa.BACKEND_CUDA_CORE)
    seq_lens, H, D = [64, 64, 200], 4, 64
    P = sum(seq_lens)
    rng = np.random.default_rng(21)
    qkv = gi.round_kind(rng.standard_normal((P, 3, H, D), dtype=np.float32), kind)
    cu = torch.tensor([0, 64, 128, 328], dtype=torch.int32, device="cuda")
    scale = 1.0 / (D ** 0.5)
    q_dev = to_dev(qkv, kind)
    plain, lse, _ = api.flash_attn_varlen_qkvpacked_func(q_dev, cu, 200, softmax_scale=scale, return_attn_probs=True)
    biased = api.flash_attn_varlen_qkvpacked_func_w_perkey_bias(q_dev, cu, 200, perkey_bias=torch.zeros(P, device="cuda", dtype=q_dev.dtype), softmax_scale=scale)
    torch.testing.assert_close(plain, biased, atol=1e-4, rtol=1e-4)
    want, want_lse = clib.attention_bias(qkv, None, cu.cpu().numpy(), scale)
    np.testing.assert_allclose(to_np(plain), want, atol=1e-2, rtol=1e-2)
    assert tuple(lse.shape) == (H, P) and lse.dtype == torch.float32
    np.testing.assert_allclose(to_np(lse), want_lse, atol=2e-3, rtol=1e-3)
    _check_status()


@pytest.mark.parametrize("which", ["cuda-core", "tcgen05"])
def test_bias_has_effect(backend, which):
    from come_b200 import flash_attn as api, flash_attn_fwd_cuda as fa
    backend(fa.BACKEND_TCGEN05 if which == "tcgen05" else fa.BACKEND_CUDA_CORE)
    P, H, D = 128, 2, 64
    g = torch.Generator(device="cpu").manual_seed(42)
    qkv = torch.randn(P, 3, H, D, generator=g).half().cuda()
    cu = torch.tensor([0, 128], device="cuda", dtype=torch.int32)
    b0 = torch.zeros(P, device="cuda", dtype=torch.float16)
    b1 = torch.randn(P, generator=g).half().cuda()
    o0 = api.flash_attn_varlen_qkvpacked_func_w_perkey_bias(qkv, cu, 128, perkey_bias=b0, softmax_scale=D ** -0.5)
    o1 = api.flash_attn_varlen_qkvpacked_func_w_perkey_bias(qkv, cu, 128, perkey_bias=b1, softmax_scale=D ** -0.5)
    assert not torch.allclose(o0, o1, atol=1e-4)
    _check_status()


def _merge_like_inputs(rng, lengths, H, D, kind):
    """Segments laid out like merged frames: 78 never-merged tokens, then windows; merged windows count 9."""
    P = int(sum(lengths))
    qkv = gi.round_kind(rng.standard_normal((P, 3, H, D), dtype=np.float32), kind)
    count = np.ones(P, np.float32)
    pos = 0
    for L in lengths:
        k = (1374 - L) // 8
        merged = np.zeros(144, bool)
        merged[rng.permutation(144)[:k]] = True
        row = pos + 78
        for m in range(144):
            if merged[m]:
                count[row] = 9.0
                row += 1
            else:
                row += 9
        assert row == pos + L
        pos += L
    cu = np.zeros(len(lengths) + 1, np.int32)
    cu[1:] = np.cumsum(lengths)
    return qkv, count, cu


@pytest.mark.parametrize("which", ["cuda-core", "tcgen05"])
def test_post_merge_lengths_bf16_vs_fp32_oracle(backend, which):
    """Ragged post-merge frame lengths 1374 - 8k (kernel-sweep configuration, reduced to 6 segments x 4 heads so
    that the CPU oracle finishes in seconds); bias = log(count) with counts in {1, 9}; bar 2e-2 absolute."""
    from come_b200 import flash_attn as api, flash_attn_fwd_cuda as fa
    backend(fa.BACKEND_TCGEN05 if which == "tcgen05" else fa.BACKEND_CUDA_CORE)
    rng = np.random.default_rng(0)
    lengths = [1374 - 8 * int(k) for k in rng.integers(0, 73, size=6)]
    H, D = 4, 64
    qkv, count, cu = _merge_like_inputs(rng, lengths, H, D, "bf16")
    bias32 = np.log(count)
    bias = to_dev(bias32, "bf16")
    out = api.flash_attn_varlen_qkvpacked_func_w_perkey_bias(to_dev(qkv, "bf16"), torch.from_numpy(cu).cuda(), max(lengths),
                                                             perkey_bias=bias, softmax_scale=D ** -0.5)
    want, _ = clib.attention_bias(qkv, bias32, cu, D ** -0.5)  # fp32 log(count), as the oracle is specified
    assert np.abs(to_np(out) - want).max() <= 2e-2
    _check_status()


def test_global_segment_and_strided_views(backend):
    """One long segment (all frames of a scene concatenated) and q/k/v given as strided views of one buffer."""
    from come_b200 import flash_attn_fwd_cuda as fa
    backend(fa.BACKEND_TCGEN05)
    rng = np.random.default_rng(3)
    P, H, D = 3 * 798 + 17, 2, 64
    qkv = gi.round_kind(rng.standard_normal((P, 3, H, D), dtype=np.float32), "bf16")
    count = np.where(rng.random(P) < 0.1, 9.0, 1.0).astype(np.float32)
    bias = gi.round_kind(np.log(count), "bf16")
    cu = np.array([0, P], np.int32)
    t = to_dev(qkv, "bf16")
    res = fa.varlen_fwd_w_perkey_bias(t[:, 0], t[:, 1], t[:, 2], None, torch.from_numpy(cu).cuda(), torch.from_numpy(cu).cuda(),
                                      None, None, None, None, to_dev(bias, "bf16"), P, P, 0.0, D ** -0.5, False, False, -1, -1,
                                      0.0, False, None)
    out, lse, p, rng_state = res
    want, want_lse = clib.attention_bias(qkv, bias, cu, D ** -0.5)
    assert np.abs(to_np(out) - want).max() <= 2e-2
    np.testing.assert_allclose(to_np(lse), want_lse, atol=2e-3, rtol=1e-3)
    assert p.numel() == 0 and tuple(rng_state.shape) == (2,) and rng_state.dtype == torch.int64
    _check_status()


@pytest.mark.parametrize("kind", ["bf16", "f16"])
@pytest.mark.parametrize("gain", [6.0, 40.0])
def test_large_magnitude_scores_rescale_path(backend, kind, gain):
    """Scores that grow along the keys: the reference max taken from the first key tile becomes too small, the kernel
    has to redo a tile with its true row max and rescale the output accumulator (float16 probabilities overflow first;
    gain 40 overflows float32 exponentials as well)."""
    from come_b200 import flash_attn as api, flash_attn_fwd_cuda as fa
    backend(fa.BACKEND_TCGEN05)
    rng = np.random.default_rng(4)
    P, H, D = 700, 2, 64
    qkv = rng.standard_normal((P, 3, H, D), dtype=np.float32)
    qkv[:, 1] *= np.linspace(0.2, gain, P, dtype=np.float32)[:, None, None]  # later keys score much higher / lower
    qkv = gi.round_kind(qkv, kind)
    cu = np.array([0, 300, 700], np.int32)
    out = api.flash_attn_varlen_qkvpacked_func(to_dev(qkv, kind), torch.from_numpy(cu).cuda(), 400, softmax_scale=D ** -0.5)
    want, _ = clib.attention_bias(qkv, None, cu, D ** -0.5)
    got = to_np(out)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 2e-2
    _check_status()


def test_rejects_what_it_does_not_implement():
    from come_b200 import flash_attn as api
    qkv = torch.zeros((16, 3, 2, 64), dtype=torch.float16, device="cuda")
    cu = torch.tensor([0, 16], dtype=torch.int32, device="cuda")
    with pytest.raises(NotImplementedError):
        api.flash_attn_varlen_qkvpacked_func(qkv, cu, 16, dropout_p=0.1)
    with pytest.raises(NotImplementedError):
        api.flash_attn_varlen_qkvpacked_func(qkv, cu, 16, causal=True)
    with pytest.raises(NotImplementedError):
        api.flash_attn_varlen_qkvpacked_func(qkv, cu, 16, window_size=(4, 4))
    with pytest.raises(NotImplementedError):
        api.flash_attn_varlen_qkvpacked_func(qkv, cu, 16, softcap=1.0)
    with pytest.raises(RuntimeError, match="fp16 and bf16"):
        api.flash_attn_varlen_qkvpacked_func(qkv.float(), cu, 16)
    with pytest.raises(RuntimeError, match="perkey_bias dtype"):
        api.flash_attn_varlen_qkvpacked_func_w_perkey_bias(qkv, cu, 16, perkey_bias=torch.zeros(16, device="cuda"))
    with pytest.raises(RuntimeError, match="int32"):
        api.flash_attn_varlen_qkvpacked_func(qkv, cu.long(), 16)
    x = torch.zeros((16, 3, 2, 64), dtype=torch.float16, device="cuda", requires_grad=True)
    with pytest.raises(RuntimeError, match="backward is not supported"):
        api.flash_attn_varlen_qkvpacked_func(x, cu, 16).sum().backward()


def test_infer_max_seqlen():
    from come_b200.flash_attn import infer_flash_attn_varlen_max_seqlen
    cu = torch.tensor([0, 5, 12, 14], dtype=torch.int32, device="cuda")
    assert infer_flash_attn_varlen_max_seqlen(cu) == 7


@pytest.mark.parametrize("which", ["cuda-core", "tcgen05"])
@pytest.mark.parametrize("seq_lens,cuts", [([3000], [0, 1111, 1999, 3000]), ([700, 300, 900], [0, 650, 1000, 1900])])
def test_query_row_slices_match_full_attention(backend, which, seq_lens, cuts):
    """Global attention sharded by query rows: attending every slice of the rows to all keys / values must give the
    same rows as one full launch (the per-GPU piece of the multi-GPU path, exercised here on one GPU)."""
    from come_b200 import flash_attn_fwd_cuda as fa
    backend(fa.BACKEND_TCGEN05 if which == "tcgen05" else fa.BACKEND_CUDA_CORE)
    H, D = 2, 64
    P = sum(seq_lens)
    rng = np.random.default_rng(31)
    qkv = to_dev(gi.round_kind(rng.standard_normal((P, 3, H, D), dtype=np.float32), "bf16"), "bf16")
    bias = to_dev(gi.round_kind(np.log(np.where(rng.random(P) < 0.2, 9.0, 1.0)).astype(np.float32), "bf16"), "bf16")
    cu = torch.tensor(np.concatenate([[0], np.cumsum(seq_lens)]), dtype=torch.int32, device="cuda")
    full, full_lse = fa.varlen_fwd_rows(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu, max(seq_lens), bias, D ** -0.5, 0)
    ref = fa.varlen_fwd_w_perkey_bias(qkv[:, 0], qkv[:, 1], qkv[:, 2], None, cu, cu, None, None, None, None, bias, max(seq_lens),
                                      max(seq_lens), 0.0, D ** -0.5, False, False, -1, -1, 0.0, False, None)
    assert torch.equal(full, ref[0]) and torch.equal(full_lse, ref[1])
    for a, b in zip(cuts[:-1], cuts[1:]):
        q_slice = qkv[a:b, 0].contiguous()  # a rank only holds its own query rows
        out, lse = fa.varlen_fwd_rows(q_slice, qkv[:, 1], qkv[:, 2], cu, max(seq_lens), bias, D ** -0.5, a)
        assert tuple(out.shape) == (b - a, H, D) and tuple(lse.shape) == (H, b - a)
        torch.testing.assert_close(out, full[a:b], atol=0, rtol=0)
        torch.testing.assert_close(lse, full_lse[:, a:b], atol=0, rtol=0)
    _check_status()


def test_tile_boundary_lengths(backend):
    """Segment lengths on and around the kernel's tile sizes (64 keys per step, 128-row query tiles, 384-row work items):
    every combination of one, two or three active query tiles and of a full or ragged last key tile, and more work items
    than SMs so that CTAs of the persistent kernel carry their barrier phases across several items."""
    from come_b200 import flash_attn as api, flash_attn_fwd_cuda as fa
    backend(fa.BACKEND_TCGEN05)
    rng = np.random.default_rng(12)
    lengths = [1, 63, 64, 65, 127, 128, 129, 383, 384, 385, 512, 513, 769, 2, 640, 256]
    H, D, P = 12, 64, sum([1, 63, 64, 65, 127, 128, 129, 383, 384, 385, 512, 513, 769, 2, 640, 256])
    qkv = gi.round_kind(rng.standard_normal((P, 3, H, D), dtype=np.float32), "bf16")
    weight = np.where(rng.random(P) < 0.3, np.float32(9), np.float32(1))
    bias = gi.round_kind(np.log(weight), "bf16")
    cu = np.zeros(len(lengths) + 1, np.int32)
    cu[1:] = np.cumsum(lengths)
    out = api.flash_attn_varlen_qkvpacked_func_w_perkey_bias(to_dev(qkv, "bf16"), torch.from_numpy(cu).cuda(), max(lengths),
                                                             perkey_bias=to_dev(bias, "bf16"), softmax_scale=D ** -0.5)
    want, _ = clib.attention_bias(qkv, bias, cu, D ** -0.5)
    assert np.abs(to_np(out) - want).max() <= 2e-2
    _check_status()


def test_device_side_longest_segment(backend):
    """A loose host-side max_seqlen plus the true longest segment in device memory (what a captured graph passes) gives
    the same result, bit for bit, as the exact host-side bound; a device value larger than the host bound is clamped."""
    from come_b200 import flash_attn_fwd_cuda as fa
    backend(fa.BACKEND_TCGEN05)
    rng = np.random.default_rng(13)
    lengths = [700, 420, 901, 130]
    H, D, P = 4, 64, 2151
    qkv = to_dev(gi.round_kind(rng.standard_normal((P, 3, H, D), dtype=np.float32), "bf16"), "bf16")
    bias = to_dev(np.zeros(P, np.float32), "bf16")
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lengths)]), dtype=torch.int32, device="cuda")
    q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
    exact, lse0 = fa.varlen_fwd_rows(q, k, v, cu, max(lengths), bias, D ** -0.5, 0)
    for dev_value in (max(lengths), 10 ** 6):
        md = torch.tensor([dev_value], dtype=torch.int32, device="cuda")
        loose, lse1 = fa.varlen_fwd_rows(q, k, v, cu, P, bias, D ** -0.5, 0, max_seqlen_dev=md)
        assert torch.equal(exact, loose) and torch.equal(lse0, lse1)
    _check_status()


@pytest.mark.parametrize("nseg", [15, 16, 1500, 2048, 2100])
def test_many_short_segments(backend, nseg):
    """Thousands of short segments: around the size of the kernel's shared-memory table of per-segment query-block counts
    (2048 entries; more segments fall back to a work list with empty slots).  Checked against the fp32 CPU oracle and
    against the CUDA-core kernel."""
    from come_b200 import flash_attn as api, flash_attn_fwd_cuda as fa
    rng = np.random.default_rng(nseg)
    lengths = rng.integers(1, 40, size=nseg)
    lengths[7] = 700  # one long segment among them
    P, H, D = int(lengths.sum()), 2, 64
    qkv = to_dev(gi.round_kind(rng.standard_normal((P, 3, H, D), dtype=np.float32), "bf16"), "bf16")
    bias = to_dev(gi.round_kind(np.log(np.where(rng.random(P) < 0.3, 9.0, 1.0)).astype(np.float32), "bf16"), "bf16")
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lengths)]), dtype=torch.int32, device="cuda")
    outs = []
    for which in (fa.BACKEND_TCGEN05, fa.BACKEND_CUDA_CORE):
        backend(which)
        outs.append(api.flash_attn_varlen_qkvpacked_func_w_perkey_bias(qkv, cu, int(lengths.max()), perkey_bias=bias,
                                                                       softmax_scale=D ** -0.5).float())
    assert (outs[0] - outs[1]).abs().max().item() <= 2e-2
    want, _ = clib.attention_bias(to_np(qkv), to_np(bias), cu.cpu().numpy(), D ** -0.5)
    for got in outs:
        assert np.abs(got.cpu().numpy() - want).max() <= 2e-2
    _check_status()


def test_kernel_sweep_configuration_full_shape(backend):
    """The kernel-sweep configuration at its real shape: 64 packed segments of 1374 - 8k tokens (k ~ U{0..72}), 16 heads,
    head_dim 64, counts {1, 9} laid out in merge order, bias = log(count).  64 segments run the instantiation of the
    tensor-core kernel that enumerates its work items from a per-segment table (16 to 2048 segments); the result is
    compared with the fp32 CPU oracle on every row and head, bar 2e-2 absolute."""
    from come_b200 import flash_attn as api, flash_attn_fwd_cuda as fa
    backend(fa.BACKEND_TCGEN05)
    rng = np.random.default_rng(0)
    lengths = [1374 - 8 * int(k) for k in rng.integers(0, 73, size=64)]
    H, D = 16, 64
    qkv, count, cu = _merge_like_inputs(rng, lengths, H, D, "bf16")
    bias32 = np.log(count)
    out, lse, _ = api.flash_attn_varlen_qkvpacked_func_w_perkey_bias(
        to_dev(qkv, "bf16"), torch.from_numpy(cu).cuda(), max(lengths), perkey_bias=to_dev(bias32, "bf16"),
        softmax_scale=D ** -0.5, return_attn_probs=True)
    want, want_lse = clib.attention_bias(qkv, bias32, cu, D ** -0.5)
    assert np.abs(to_np(out) - want).max() <= 2e-2
    np.testing.assert_allclose(to_np(lse), want_lse, atol=1e-2, rtol=1e-3)  # the device bias is log(9) rounded to bfloat16
    _check_status()


def test_global_segment_of_100_frames_sampled_rows(backend):
    """One global segment of 79,800 packed tokens (100 half-merged frames): the full launch and a launch on a slice of the
    query rows that does not start at row 0, compared with the fp32 CPU oracle on sampled query rows -- the first query
    tile, rows around a 384-row work-item boundary, rows around the start of the slice and the ragged last tile (896 rows
    x 2 heads against all 79,800 keys)."""
    from come_b200 import flash_attn_fwd_cuda as fa
    backend(fa.BACKEND_TCGEN05)
    rng = np.random.default_rng(100)
    P, H, D = 79800, 2, 64
    qkv = gi.round_kind(rng.standard_normal((P, 3, H, D), dtype=np.float32), "bf16")
    count = np.where(rng.random(P) < 0.11, np.float32(9), np.float32(1))
    bias32 = np.log(count)
    cu_np = np.array([0, P], np.int32)
    cu = torch.from_numpy(cu_np).cuda()
    t, b = to_dev(qkv, "bf16"), to_dev(bias32, "bf16")
    full, full_lse = fa.varlen_fwd_rows(t[:, 0], t[:, 1], t[:, 2], cu, P, b, D ** -0.5, 0)
    lo, hi = 30000, 40100  # a rank's share of the rows: neither end on a tile boundary of the full launch
    part, part_lse = fa.varlen_fwd_rows(t[lo:hi, 0].contiguous(), t[:, 1], t[:, 2], cu, P, b, D ** -0.5, lo)
    full_np, part_np, full_lse_np, part_lse_np = to_np(full), to_np(part), to_np(full_lse), to_np(part_lse)
    last_tile = (P // 128) * 128
    samples = [(0, 128), (384 * 100 - 64, 384 * 100 + 64), (lo, lo + 128), (lo + 384 * 3 - 64, lo + 384 * 3 + 64),
               (hi - 128, hi), (last_tile - 128, P)]
    checked = 0
    for a, e in samples:
        want, want_lse = clib.attention_bias(qkv, bias32, cu_np, D ** -0.5, a, e)
        assert np.abs(full_np[a:e] - want[a:e]).max() <= 2e-2, (a, e)
        np.testing.assert_allclose(full_lse_np[:, a:e], want_lse[:, a:e], atol=1e-2, rtol=1e-3)
        if a >= lo and e <= hi:
            assert np.abs(part_np[a - lo:e - lo] - want[a:e]).max() <= 2e-2, (a, e)
            np.testing.assert_allclose(part_lse_np[:, a - lo:e - lo], want_lse[:, a:e], atol=1e-2, rtol=1e-3)
        checked += e - a
    assert checked >= 512
    _check_status()


def test_very_long_segment(backend):
    """One segment of 24,700 tokens (193 query-tile rows, 386 key steps per work item), checked against the CUDA-core kernel
    (the CPU oracle would take minutes)."""
    from come_b200 import flash_attn as api, flash_attn_fwd_cuda as fa
    rng = np.random.default_rng(99)
    P, H, D = 24700, 1, 64
    qkv = to_dev(gi.round_kind(rng.standard_normal((P, 3, H, D), dtype=np.float32), "bf16"), "bf16")
    bias = to_dev(gi.round_kind(np.log(np.where(rng.random(P) < 0.3, 9.0, 1.0)).astype(np.float32), "bf16"), "bf16")
    cu = torch.tensor([0, P], dtype=torch.int32, device="cuda")
    outs = []
    for which in (fa.BACKEND_TCGEN05, fa.BACKEND_CUDA_CORE):
        backend(which)
        outs.append(api.flash_attn_varlen_qkvpacked_func_w_perkey_bias(qkv, cu, P, perkey_bias=bias, softmax_scale=D ** -0.5).float())
    assert (outs[0] - outs[1]).abs().max().item() <= 2e-2
    _check_status()


@pytest.mark.parametrize("which", ["cuda-core", "tcgen05"])
@pytest.mark.parametrize("rows,kv_rows", [(300, 1000), (1000, 300), (129, 64), (5, 1)])
def test_cross_attention_and_combine_match_full_attention(backend, which, rows, kv_rows):
    """Keys split into the query rows' own block and a block that does not contain them: attention to the own block
    (plain self-attention), attention to the other block (``cross_fwd``, more or fewer keys than query rows) and the merge
    of the two from their log-sum-exps must reproduce attention over all keys -- against the fp32 oracle, bar 2e-2 -- and
    the merge kernel must agree with the oracle's merge of the same two partial results."""
    from come_b200 import flash_attn_fwd_cuda as fa
    from oracle import come_oracle as orc
    backend(fa.BACKEND_TCGEN05 if which == "tcgen05" else fa.BACKEND_CUDA_CORE)
    H, D = 3, 64
    rng = np.random.default_rng(rows * 7 + kv_rows)
    P = rows + kv_rows
    qkv = gi.round_kind(rng.standard_normal((P, 3, H, D), dtype=np.float32), "bf16")
    bias = gi.round_kind(np.log(np.where(rng.random(P) < 0.2, 9.0, 1.0)).astype(np.float32), "bf16")
    t, b = to_dev(qkv, "bf16"), to_dev(bias, "bf16")
    scale = D ** -0.5
    q_own = t[:rows, 0].contiguous()
    cu_own = torch.tensor([0, rows], dtype=torch.int32, device="cuda")
    o_own, l_own = fa.varlen_fwd_rows(q_own, t[:rows, 1], t[:rows, 2], cu_own, rows, b[:rows].contiguous(), scale, 0)
    o_far, l_far = fa.cross_fwd(q_own, t[rows:, 1], t[rows:, 2], b[rows:].contiguous(), scale)
    assert tuple(o_far.shape) == (rows, H, D) and tuple(l_far.shape) == (H, rows)
    # the other block alone, against the oracle: queries = the first rows, keys = the second block
    want_far = _oracle_cross(qkv[:rows, 0], qkv[rows:, 1], qkv[rows:, 2], bias[rows:], scale)
    assert np.abs(to_np(o_far) - want_far[0]).max() <= 2e-2
    np.testing.assert_allclose(to_np(l_far), want_far[1], atol=2e-3, rtol=1e-3)
    out, lse = fa.combine(o_own, l_own, o_far, l_far)
    want, want_lse = clib.attention_bias(qkv, bias, np.array([0, P], np.int32), scale, 0, rows)
    assert np.abs(to_np(out) - want[:rows]).max() <= 2e-2
    np.testing.assert_allclose(to_np(lse), want_lse[:, :rows], atol=2e-3, rtol=1e-3)
    ref_out, ref_lse = orc.attention_combine(to_np(o_own), to_np(l_own), to_np(o_far), to_np(l_far))
    np.testing.assert_allclose(to_np(out), ref_out, atol=0, rtol=2 ** -7)  # one rounding to bfloat16
    np.testing.assert_allclose(to_np(lse), ref_lse, atol=1e-5, rtol=1e-6)
    # in place: the merged result may overwrite the first partial result
    fa.combine(o_own, l_own, o_far, l_far, out_=o_own, lse_out=l_own)
    assert torch.equal(o_own, out) and torch.equal(l_own, lse)
    _check_status()


def _oracle_cross(q, k, v, bias, scale):
    """fp32 attention of q [rows, H, D] to k / v [kv, H, D] with a per-key bias (numpy, small cases)."""
    s = np.einsum("ihd,jhd->hij", q.astype(np.float64), k.astype(np.float64)) * scale + bias.astype(np.float64)[None, None, :]
    m = s.max(axis=-1, keepdims=True)
    p = np.exp(s - m)
    l = p.sum(axis=-1, keepdims=True)
    out = np.einsum("hij,jhd->ihd", p / l, v.astype(np.float64))
    return out.astype(np.float32), (m + np.log(l))[:, :, 0].astype(np.float32)


@pytest.mark.parametrize("rows,kv_rows,parts", [(300, 1000, 2), (500, 1037, 7), (129, 4096, 64), (40, 130, 3)])
def test_cross_attention_with_key_shares(backend, rows, kv_rows, parts):
    """``come_attn_cross_fwd_parts`` + ``come_attn_combine_parts``: the keys of every work item split into shares (ragged
    last share, more shares than some launches have items), every share against the oracle on its own key range, the merged
    result against the oracle over all keys (bar 2e-2) and against the one-launch kernel."""
    from come_b200 import _lib, flash_attn_fwd_cuda as fa
    from come_b200._torch_util import dtype_code, ptr, stream_ptr
    backend(fa.BACKEND_TCGEN05)
    H, D = 3, 64
    rng = np.random.default_rng(rows + 13 * kv_rows + parts)
    q = gi.round_kind(rng.standard_normal((rows, H, D), dtype=np.float32), "bf16")
    kv = gi.round_kind(rng.standard_normal((kv_rows, 2, H, D), dtype=np.float32), "bf16")
    bias = gi.round_kind(np.log(np.where(rng.random(kv_rows) < 0.2, 9.0, 1.0)).astype(np.float32), "bf16")
    tq, tkv, tb = to_dev(q, "bf16"), to_dev(kv, "bf16"), to_dev(bias, "bf16")
    scale = D ** -0.5
    tiles = -(-kv_rows // 64)
    per = -(-tiles // parts)
    parts = -(-tiles // per)  # the caller's duty: no empty share
    out_parts = torch.full((parts, rows, H, D), 7.0, dtype=torch.bfloat16, device="cuda")
    lse_parts = torch.full((parts, H, rows), 7.0, dtype=torch.float32, device="cuda")
    lib, st = _lib.lib(), stream_ptr(tq.device)
    k, v = tkv[:, 0], tkv[:, 1]
    _lib.check(lib.come_attn_cross_fwd_parts(ptr(tq), ptr(k), ptr(v), dtype_code(tq.dtype), rows, kv_rows, H, D, tq.stride(0),
                                             k.stride(0), v.stride(0), ptr(tb), scale, parts, ptr(out_parts), ptr(lse_parts),
                                             fa.BACKEND_TCGEN05, st))
    for p in range(parts):
        lo, hi = p * per * 64, min(kv_rows, (p + 1) * per * 64)
        want = _oracle_cross(q, kv[lo:hi, 0], kv[lo:hi, 1], bias[lo:hi], scale)
        assert np.abs(to_np(out_parts[p]) - want[0]).max() <= 2e-2, p
        np.testing.assert_allclose(to_np(lse_parts[p]), want[1], atol=2e-3, rtol=1e-3)
    out = torch.empty((rows, H, D), dtype=torch.bfloat16, device="cuda")
    lse = torch.empty((H, rows), dtype=torch.float32, device="cuda")
    _lib.check(lib.come_attn_combine_parts(ptr(out_parts), ptr(lse_parts), parts, dtype_code(tq.dtype), rows, H, D, ptr(out),
                                           ptr(lse), st))
    want = _oracle_cross(q, kv[:, 0], kv[:, 1], bias, scale)
    assert np.abs(to_np(out) - want[0]).max() <= 2e-2
    np.testing.assert_allclose(to_np(lse), want[1], atol=2e-3, rtol=1e-3)
    from oracle import come_oracle as orc
    ref_out, ref_lse = orc.attention_combine_parts(to_np(out_parts), to_np(lse_parts))  # the merge kernel alone
    np.testing.assert_allclose(to_np(out), ref_out, atol=2e-6, rtol=2 ** -7)  # one rounding to bfloat16
    np.testing.assert_allclose(to_np(lse), ref_lse, atol=1e-5, rtol=1e-6)
    one, one_lse = fa.cross_fwd(tq, k, v, tb, scale)
    assert (out.float() - one.float()).abs().max().item() <= 2e-2
    torch.testing.assert_close(lse, one_lse, atol=2e-3, rtol=1e-3)
    # refusals: an empty share, no log-sum-exp output
    rc = lib.come_attn_cross_fwd_parts(ptr(tq), ptr(k), ptr(v), dtype_code(tq.dtype), rows, 64, H, D, tq.stride(0), k.stride(0),
                                       v.stride(0), ptr(tb), scale, 2, ptr(out_parts), ptr(lse_parts), fa.BACKEND_TCGEN05, st)
    assert rc == _lib.COME_ERR_ARG and "share" in _lib.last_error()
    _check_status()


def test_balanced_cross_attention_splits_the_last_round():
    """10,534 query rows x 16 heads are 448 work items: three rounds on 148 CTAs and four items.  ``cross_fwd_balanced``
    runs the last query block with its keys in shares (nine for 70,138 keys); the result must agree with the one-launch kernel (rounding of
    the shares' outputs only) and the plan must be the expected one."""
    from come_b200 import flash_attn_fwd_cuda as fa
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    rows, kv_rows, H, D = 10534, 4096, 16, 64
    main_rows, parts = fa.plan_tail_split(rows, H, kv_rows, sms)
    if sms == 148:
        assert (main_rows, parts) == (10368, 8)  # 64 key tiles in shares of 8 tiles (nine shares would leave one empty)
        assert fa.plan_tail_split(rows, H, 70138, sms) == (10368, 9) and fa.plan_tail_split(9656, H, 70138, sms) == (9656, 1)
    g = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn((rows, H, D), device="cuda", generator=g).bfloat16()
    kv = torch.randn((kv_rows, 2, H, D), device="cuda", generator=g).bfloat16()
    bias = torch.where(torch.rand(kv_rows, device="cuda", generator=g) < 0.2, 9.0, 1.0).log().bfloat16()
    one, one_lse = fa.cross_fwd(q, kv[:, 0], kv[:, 1], bias, D ** -0.5)
    out, lse = fa.cross_fwd_balanced(q, kv[:, 0], kv[:, 1], bias, D ** -0.5)
    assert tuple(out.shape) == (rows, H, D) and tuple(lse.shape) == (H, rows)
    assert torch.equal(out[:main_rows], one[:main_rows]) and torch.equal(lse[:, :main_rows], one_lse[:, :main_rows])
    assert (out.float() - one.float()).abs().max().item() <= 1e-2
    torch.testing.assert_close(lse, one_lse, atol=2e-3, rtol=1e-3)
    _check_status()
