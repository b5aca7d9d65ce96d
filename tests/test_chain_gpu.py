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


def test_batch_of_ragged_scenes_matches_oracle_plan_and_per_scene_runs():
    """Several independent scenes of 4 frames in one static batch, merge ratio drawn per frame from U(0.25, 0.75)
    (the batch-throughput configuration, reduced): the mask must equal the oracle's per-frame quantile selection, and
    every scene's output must equal what a one-scene runner computes for it alone."""
    from come_b200.static_scene import StaticScene
    from oracle import come_oracle as orc
    scenes, fps, C, H, D = 3, 4, 128, 2, 64
    frames = scenes * fps
    kinds = ["frame", "global"]
    batch = StaticScene(frames, channels=C, num_heads=H, head_dim=D, layer_kinds=kinds, frames_per_scene=fps,
                        per_frame_ratios=True).capture()
    single = StaticScene(fps, channels=C, num_heads=H, head_dim=D, layer_kinds=kinds, per_frame_ratios=True).capture()
    g = torch.Generator(device="cpu").manual_seed(23)
    x = torch.randn((frames, 1374, C), generator=g).bfloat16()
    conf = torch.rand((scenes, fps * 1369), generator=g).bfloat16()
    ratios = (torch.rand(frames, generator=g) * 0.5 + 0.25).float()
    # every scene gets its own packed qkv rows: scene s of the batch starts at the batch's packed offset of its first frame
    qkv_full = torch.randn((frames * 1374, 3, H, D), generator=g).bfloat16()
    batch.ratios.copy_(ratios)
    got = batch.run(x, conf, qkv_full).clone()
    want_mask = orc.select_windows(conf.float().numpy(), scenes, fps, 37, 37, 3, 3, ratios.numpy(), "pairwise-rank", "frame", "bf16")
    np.testing.assert_array_equal(batch.mask.cpu().numpy().astype(bool), want_mask)
    lengths = 1374 - 8 * want_mask.sum(axis=1)
    assert lengths.min() < lengths.max()  # ragged
    offsets = batch.offsets.cpu().numpy()
    np.testing.assert_array_equal(np.diff(offsets), lengths)
    for s_ in range(scenes):
        f0 = s_ * fps
        single.ratios.copy_(ratios[f0:f0 + fps])
        r0, r1 = int(offsets[f0]), int(offsets[f0 + fps])
        out = single.run(x[f0:f0 + fps], conf[s_:s_ + 1], qkv_full[r0:r1])
        torch.testing.assert_close(got[f0:f0 + fps], out, atol=0, rtol=0)
