"""The allocation-free plan entry point (come_merge_plan_static) against the regular one (come_merge_plan).

Collected last on purpose: a run that stops at the first failure has then already been through every other test.
The check calls the C ABI directly, twice in a row with different masks, because the second call reuses the scratch
array the first one left behind.  It has to pass in a fresh process and after the rest of the suite.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _plan(lib, fn_name, mask_u8, layout, n_tok, with_workspace):
    frames, M = mask_u8.shape
    dev = mask_u8.device
    gp = torch.full((frames, M), -7, dtype=torch.int32, device=dev)
    off = torch.full((frames + 1,), -7, dtype=torch.int32, device=dev)
    rev = torch.full((frames * n_tok,), -7, dtype=torch.int64, device=dev)
    w = torch.full((frames * n_tok,), -7.0, dtype=torch.float32, device=dev)
    seg = torch.full((1,), -7, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    args = [mask_u8.data_ptr(), frames, C.byref(layout), gp.data_ptr(), off.data_ptr(), rev.data_ptr(), w.data_ptr(),
            seg.data_ptr()]
    if with_workspace:
        nbytes = lib.come_merge_plan_workspace_bytes(frames)
        ws = torch.empty((nbytes,), dtype=torch.uint8, device=dev)
        args += [ws.data_ptr(), nbytes]
    rc = getattr(lib, fn_name)(*args, st)
    torch.cuda.synchronize()
    return rc, (gp, off, rev, w, seg)


def test_static_plan_matches_regular_plan_twice():
    from come_b200 import _lib
    lib = _lib.lib()
    layout = _lib.Layout.two_d(5, 37, 37, 3, 3)
    rng = np.random.default_rng(99)
    for frames, ratio in ((100, 0.5), (37, 0.2)):  # second call: fewer frames, stale scratch beyond them
        mask = torch.from_numpy(rng.random((frames, 144)) < ratio).cuda().view(torch.uint8)
        rc_a, a = _plan(lib, "come_merge_plan", mask, layout, 1374, True)
        rc_b, b = _plan(lib, "come_merge_plan_static", mask, layout, 1374, False)
        assert rc_a == 0 and rc_b == 0, _lib.last_error()
        total = int(a[1][-1].item())
        assert total == frames * 1374 - 8 * int(mask.sum().item())
        for x, y, name in zip(a, b, ("group_prefix", "offsets", "rev_id", "weight", "seg_max")):
            if name == "weight":
                x, y = x[:total], y[:total]
            assert torch.equal(x, y), f"{name} differs between come_merge_plan_static and come_merge_plan"


def test_static_plan_refuses_more_frames_than_its_scratch_holds():
    from come_b200 import _lib
    lib = _lib.lib()
    layout = _lib.Layout.one_d(0, 2, 1)
    frames = 4097
    mask = torch.zeros((frames, 1), dtype=torch.uint8, device="cuda")
    rc, _ = _plan(lib, "come_merge_plan_static", mask, layout, 2, False)
    assert rc == _lib.COME_ERR_ARG
    assert "at most 4096 frames" in _lib.last_error()
    rc, out = _plan(lib, "come_merge_plan_static", mask[:4096], layout, 2, False)  # the documented maximum works
    assert rc == 0 and int(out[1][-1].item()) == 4096 * 2
