"""Window selection parity on the GPU: masks must equal, bit for bit, what the reference's build_ctx tensor
code produced for the same confidences (tests/golden/select.npz) and what the oracle computes."""
import os

import numpy as np
import pytest
import torch

import golden_inputs as gi
from gpu_util import to_dev, to_np
from oracle import clib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", sorted(gi.SELECT_CASES))
def test_select_fixture(golden_dir, name):
    from come_b200.token_merger import select_windows
    z = np.load(os.path.join(golden_dir, "select.npz"))
    spec = gi.SELECT_CASES[name]
    conf = gi.select_inputs(name)
    shape = tuple(z[name + "_shape"])
    want = np.unpackbits(z[name + "_mask"])[: shape[0] * shape[1]].reshape(shape).astype(bool)
    scope = "batch" if spec["cls"] == "2d" else "frame"
    mask = select_windows(to_dev(conf, spec["kind"]), spec["B"], spec["S"], spec["H"], spec["W"], spec["gh"], spec["gw"],
                          spec["thr"], spec["mode"], scope)
    assert mask.dtype == torch.bool and tuple(mask.shape) == shape
    np.testing.assert_array_equal(to_np(mask), want)


@pytest.mark.parametrize("kind", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("scope", ["batch", "frame"])
@pytest.mark.parametrize("thr", [0.0, 0.2, 0.5, 0.77, 1.0])
def test_select_random_vs_oracle(kind, scope, thr):
    from come_b200.token_merger import select_windows
    B, S, H, W, gh, gw = 3, 5, 37, 37, 3, 3
    rng = np.random.default_rng(int(thr * 100) + len(kind))
    conf = gi.round_kind(rng.random((B, S * H * W), dtype=np.float32), kind)
    want = clib.select_windows(conf, B, S, H, W, gh, gw, thr, "pairwise-rank", scope, kind)
    got = select_windows(to_dev(conf, kind), B, S, H, W, gh, gw, thr, "pairwise-rank", scope)
    np.testing.assert_array_equal(to_np(got), want)
    # thresholds that are not numbers of the 16-bit types: the comparison rounds them to the confidence dtype
    for mode, level in (("abs_mse", thr), ("abs_mse", thr * 0.9 + 0.0413), ("mse", thr * 2.0 - 1.0), ("mse", 0.0413)):
        want = clib.select_windows(conf, B, S, H, W, gh, gw, level, mode, scope, kind)
        got = select_windows(to_dev(conf, kind), B, S, H, W, gh, gw, level, mode, scope)
        np.testing.assert_array_equal(to_np(got), want)


def test_select_largest_group():
    """32768 windows in one quantile group (the documented maximum) and one above it."""
    from come_b200.token_merger import select_windows
    S, H, W = 128, 48, 48  # 128 * 256 windows
    rng = np.random.default_rng(5)
    conf = gi.round_kind(rng.random((1, S * H * W), dtype=np.float32), "bf16")
    want = clib.select_windows(conf, 1, S, H, W, 3, 3, 0.5, "pairwise-rank", "batch", "bf16")
    got = select_windows(to_dev(conf, "bf16"), 1, S, H, W, 3, 3, 0.5, "pairwise-rank", "batch")
    np.testing.assert_array_equal(to_np(got), want)
    with pytest.raises(RuntimeError, match="windows per quantile group"):
        select_windows(torch.zeros((1, 129 * H * W), device="cuda"), 1, 129, H, W, 3, 3, 0.5, "pairwise-rank", "batch")


def test_select_rejects_bad_arguments():
    from come_b200.token_merger import select_windows
    conf = torch.zeros((1, 36), device="cuda")
    with pytest.raises(ValueError, match="threshold in"):
        select_windows(conf, 1, 1, 6, 6, 3, 3, 1.5)
    with pytest.raises(ValueError, match="unknown confidence mode"):
        select_windows(conf, 1, 1, 6, 6, 3, 3, 0.5, mode="l1")


def test_select_zscore_single_confidence_merges_nothing():
    """One confidence per batch element: the unbiased standard deviation is NaN and no window is selected, as in the
    reference's tensor expression."""
    from come_b200.token_merger import select_windows
    mask = select_windows(torch.full((3, 1), 0.25, device="cuda"), 3, 1, 1, 1, 1, 1, 10.0, mode="mse")
    assert tuple(mask.shape) == (3, 1) and not mask.any().item()
