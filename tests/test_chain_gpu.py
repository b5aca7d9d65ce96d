"""The captured, read-back-free scene runner (StaticScene) against the eager operator chain (CoMeOpChain), and the
eager chain's first layer against the CPU oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scene_replay_matches_eager_chain_for_changing_masks():
    from come_b200 import _lib
    from come_b200.chain import CoMeOpChain
    from come_b200.static_scene import StaticScene
    frames, C, H, D = 3, 256, 4, 64
    kinds = ["frame", "global", "frame"]
    scene = StaticScene(frames, channels=C, num_heads=H, head_dim=D, layer_kinds=kinds).capture()
    chain = CoMeOpChain(frames, num_heads=H, head_dim=D, layer_kinds=kinds, scope="frame")
    g = torch.Generator(device="cpu").manual_seed(7)
    for trial in range(3):  # a new confidence map each time: new mask, new packed length, same captured graph
        x = torch.randn((frames, 1374, C), generator=g).bfloat16()
        conf = torch.rand((1, frames * 1369), generator=g).bfloat16()
        if trial == 2:
            conf = torch.ones_like(conf)  # all window means tie: nothing is below the quantile, nothing merges
        qkv = torch.randn((frames * 1374, 3, H, D), generator=g).bfloat16()
        got = scene.run(x.pin_memory(), conf.pin_memory(), qkv.pin_memory()).clone()
        P = scene.packed_rows()
        want = chain.forward_scene(x.cuda(), conf.cuda(), lambda total: qkv[:total].cuda())
        plan = chain.build_plan(conf.cuda())
        assert plan.total == P
        if trial == 2:
            assert P == frames * 1374
        torch.testing.assert_close(got, want, atol=0, rtol=0)
    assert _lib.device_status(clear=True) == 0


def test_eager_chain_layer_matches_oracle():
    from come_b200.chain import CoMeOpChain
    from oracle import clib
    frames, C, H, D = 2, 128, 2, 64
    rng = np.random.default_rng(3)
    tokens = rng.standard_normal((frames, 1374, C), dtype=np.float32)
    conf = rng.random((1, frames * 1369), dtype=np.float32)
    chain = CoMeOpChain(frames, num_heads=H, head_dim=D, layer_kinds=["global"])
    plan = chain.build_plan(torch.from_numpy(conf).cuda())
    mask = clib.select_windows(conf, 1, frames, 37, 37, 3, 3, 0.5, "pairwise-rank", "frame")
    np.testing.assert_array_equal(plan.mask.cpu().numpy(), mask)
    _, off, rev, w = clib.token_merge_2d(tokens, 5, 3, 3, 37, 37, mask)
    P = plan.total
    qkv32 = rng.standard_normal((P, 3, H, D), dtype=np.float32)
    qkv = torch.from_numpy(qkv32).cuda().bfloat16()
    y = chain.layer(plan, torch.from_numpy(tokens).cuda().bfloat16(), qkv, "global")
    bias = plan.perkey_bias(torch.bfloat16).float().cpu().numpy()
    want, _ = clib.attention_bias(qkv.float().cpu().numpy(), bias, np.array([0, P], np.int32), D ** -0.5)
    want_tokens = want.reshape(P, C)[rev].reshape(frames, 1374, C)
    assert np.abs(y.float().cpu().numpy() - want_tokens).max() <= 2e-2


def test_static_scene_pipeline_matches_plain_run():
    """Staging the next scene's host inputs and draining the previous result on a side stream must not change results."""
    from come_b200.static_scene import StaticScene
    frames, C, H, D = 2, 128, 2, 64
    kinds = ["frame", "global"]
    scene = StaticScene(frames, channels=C, num_heads=H, head_dim=D, layer_kinds=kinds).capture()
    g = torch.Generator(device="cpu").manual_seed(11)
    scenes = [(torch.randn((frames, 1374, C), generator=g).bfloat16().pin_memory(),
               torch.rand((1, frames * 1369), generator=g).bfloat16().pin_memory(),
               torch.randn((frames * 1374, 3, H, D), generator=g).bfloat16().pin_memory()) for _ in range(5)]
    want = [scene.run(*sc).clone().cpu() for sc in scenes]
    outs = [torch.empty((frames, 1374, C), dtype=torch.bfloat16).pin_memory() for _ in scenes]
    scene.stage(*scenes[0])
    for k in range(len(scenes)):
        if k + 1 < len(scenes):
            scene.stage(*scenes[k + 1])
        scene.run_staged(outs[k])
    scene.drain()
    torch.cuda.synchronize()
    for got, ref in zip(outs, want):
        torch.testing.assert_close(got, ref, atol=0, rtol=0)
