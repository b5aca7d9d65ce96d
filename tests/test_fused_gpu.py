"""GPU parity of the merged forward pass of the aggregator (blocks over packed tokens, retained layers unmerged)
against the float32 oracle chain, plus the properties that hold at any size."""
import numpy as np
import pytest
import torch

import oracle.come_oracle as orc
from tests.golden import golden_inputs as gi
from tests.gpu_util import to_np

pytestmark = pytest.mark.gpu


def _small_model(rng, depth, C, heads, ls_init, dtype):
    """An AggregatorCore whose parameters are the seeded ones of the golden helpers (rounded to bfloat16, so that the
    oracle and the device hold the same numbers), plus the per-block parameter dictionaries for the oracle."""
    from come_b200.vggt_arch import AggregatorCore
    core = AggregatorCore(embed_dim=C, depth=depth, num_heads=heads, mlp_ratio=2.0, init_values=ls_init,
                          retain_layers=None, patch_start_idx=5)
    params = {"frame": [], "global": []}
    for kind, blocks in (("frame", core.frame_blocks), ("global", core.global_blocks)):
        for blk in blocks:
            p = gi.block_params(rng, C, heads, 2.0, True, ls_init, kind="bf16")
            blk.load_state_dict({k: torch.from_numpy(v) for k, v in p.items()})
            params[kind].append(dict(p, norm_eps=blk.norm1.eps, qk_norm_eps=blk.attn.q_norm.eps))
    return core.cuda().to(dtype).eval(), params


def _relative_error(a: np.ndarray, b: np.ndarray) -> float:
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) / np.linalg.norm(b.astype(np.float64)))


# bfloat16 activations through `depth` pairs of blocks against float32 arithmetic: every block rounds its branches to
# 8 bits of mantissa (relative 2^-9 per element); errors of independent roundings add in quadrature.
FUSED_REL_TOL = 2e-2
FUSED_ABS_TOL = 0.15  # worst single element, activations of magnitude ~1-4


@pytest.mark.parametrize("B,S,side,ratio", [(1, 3, 7, 0.5), (2, 2, 6, 0.5), (1, 2, 7, 0.0), (1, 4, 7, 1.0)])
def test_fused_forward_against_oracle(B, S, side, ratio):
    from come_b200 import _lib
    from come_b200.fused import FusedAggregator
    from come_b200.token_merger import MergePlan
    rng = np.random.default_rng(100 + 10 * B + S)
    C, heads, depth, start = 128, 2, 2, 5
    N = start + side * side
    M = (side // 3) ** 2
    core, params = _small_model(rng, depth, C, heads, 0.5, torch.bfloat16)
    model = FusedAggregator(core)
    tokens = gi.round_kind(rng.standard_normal((B, S, N, C), dtype=np.float32), "bf16")
    mask = rng.random((B * S, M)) < ratio
    plan = MergePlan(torch.from_numpy(mask).cuda(), _lib.Layout.two_d(start, side, side, 3, 3))
    with torch.no_grad():
        out, patch_start = model(torch.from_numpy(tokens).cuda().bfloat16(), plan)
    assert patch_start == start and sorted(out) == list(range(depth))
    ref = orc.fused_aggregator(tokens, mask, start, side, side, 3, 3, params["frame"], params["global"], heads)
    for layer in range(depth):
        got = to_np(out[layer])
        assert got.shape == (B, S, N, 2 * C) and out[layer].dtype == torch.bfloat16
        assert _relative_error(got, ref[layer]) < FUSED_REL_TOL, (layer, _relative_error(got, ref[layer]))
        assert np.abs(got - ref[layer]).max() < FUSED_ABS_TOL, (layer, np.abs(got - ref[layer]).max())


def test_fused_forward_float32_stream():
    """A float32 model keeps its residual stream, norms and MLP in float32 and only the attention branch in bfloat16,
    as the reference's block does (the casts around the attention module)."""
    from come_b200 import _lib
    from come_b200.fused import FusedAggregator
    from come_b200.token_merger import MergePlan
    rng = np.random.default_rng(5)
    C, heads, depth, start, side, B, S = 128, 2, 1, 5, 6, 1, 2
    N, M = start + side * side, 4
    core, params = _small_model(rng, depth, C, heads, 0.5, torch.float32)
    model = FusedAggregator(core)
    tokens = rng.standard_normal((B, S, N, C), dtype=np.float32)
    mask = rng.random((B * S, M)) < 0.5
    plan = MergePlan(torch.from_numpy(mask).cuda(), _lib.Layout.two_d(start, side, side, 3, 3))
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        with torch.no_grad():
            out, _ = model(torch.from_numpy(tokens).cuda(), plan)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    ref = orc.fused_aggregator(tokens, mask, start, side, side, 3, 3, params["frame"], params["global"], heads)
    assert out[0].dtype == torch.float32
    assert _relative_error(to_np(out[0]), ref[0]) < 6e-3  # one bfloat16 attention branch per block, two blocks


def test_nothing_merged_equals_unmerged_model():
    """With an all-False mask the accelerated model runs the unmerged model's arithmetic on a permuted token order
    (log 1 = 0 bias); attention is equivariant under the permutation, so the outputs agree to bfloat16 rounding of
    differently ordered sums."""
    from come_b200 import _lib
    from come_b200.fused import FusedAggregator
    from come_b200.token_merger import MergePlan
    rng = np.random.default_rng(9)
    C, heads, depth, start, side, B, S = 128, 2, 2, 5, 7, 1, 3
    N, M = start + side * side, 4
    core, _ = _small_model(rng, depth, C, heads, 0.5, torch.bfloat16)
    model = FusedAggregator(core)
    tokens = torch.from_numpy(rng.standard_normal((B, S, N, C), dtype=np.float32)).cuda().bfloat16()
    plan = MergePlan(torch.zeros(B * S, M, dtype=torch.bool, device="cuda"), _lib.Layout.two_d(start, side, side, 3, 3))
    with torch.no_grad():
        merged_out, _ = model(tokens, plan)
        dense_out, _ = model.forward_unmerged(tokens)
    for layer in range(depth):
        assert _relative_error(to_np(merged_out[layer]), to_np(dense_out[layer])) < 1e-2


@pytest.mark.parametrize("B,S", [(1, 3), (2, 2)])
def test_captured_forward_replays_new_scenes(B, S):
    """The CUDA-graph replay gives the eager result bit for bit, also for a second scene with another mask of the same
    packed length (other segment lengths), and captures a second graph for another packed length."""
    from come_b200 import _lib
    from come_b200.fused import CapturedForward, FusedAggregator
    from come_b200.token_merger import MergePlan
    rng = np.random.default_rng(11)
    C, heads, depth, start, side = 128, 2, 2, 5, 7
    N, M = start + side * side, 4
    core, _ = _small_model(rng, depth, C, heads, 0.5, torch.bfloat16)
    model = FusedAggregator(core)
    captured = CapturedForward(model)
    layout = _lib.Layout.two_d(start, side, side, 3, 3)
    masks = []
    for merged_per_frame in ([2] * (B * S), [1] + [3] + [2] * (B * S - 2), [1] * (B * S)):
        m = np.zeros((B * S, M), bool)
        for f, k in enumerate(merged_per_frame):
            m[f, rng.permutation(M)[:k]] = True
        masks.append(m)
    for i, m in enumerate(masks):
        tokens = torch.from_numpy(rng.standard_normal((B, S, N, C), dtype=np.float32)).cuda().bfloat16()
        plan = MergePlan(torch.from_numpy(m).cuda(), layout)
        with torch.no_grad():
            eager, _ = model(tokens, MergePlan(torch.from_numpy(m).cuda(), layout))
            replay, _ = captured(tokens, plan)
        for layer in eager:
            assert torch.equal(eager[layer], replay[layer]), (i, layer)
    assert len(captured._graphs) == 2  # the first two masks pack to the same length


def test_timer_ranges():
    from come_b200.timer import Timer
    Timer.reset()
    Timer.activate()
    try:
        x = torch.ones(1 << 20, device="cuda")
        for _ in range(3):
            with Timer.range("fill"):
                x.mul_(2.0)
        with Timer.range("other"):
            x.add_(1.0)
        entries = {e.name: e for e in Timer.results()}
        assert entries["fill"].count == 3 and entries["other"].count == 1
        assert 0.0 < entries["fill"].P50 <= entries["fill"].P90 <= entries["fill"].P99
        report = Timer.report()
        assert "Median (ms)" in report and "fill" in report
    finally:
        Timer.activate(False)
        Timer.reset()
    with Timer.range("inactive"):
        pass
    assert Timer.results() == []


# ---- come_residual_layernorm: bit-exact against the oracle ------------------------------------------------------
RLN_CASES = [  # (rows, C, dtype, has_branch, has_scale, has_norm)
    (37, 1024, "bf16", True, True, True),
    (37, 1024, "f16", True, True, True),
    (19, 1024, "f32", True, True, True),   # 256 vectors per row: eight per lane
    (50, 2048, "bf16", True, True, True),
    (33, 384, "bf16", True, True, True),   # 48 vectors: the second vector of a lane exists for half the lanes
    (64, 128, "f16", True, False, True),
    (21, 64, "f32", True, True, False),    # residual update alone
    (40, 1024, "bf16", False, False, True),  # LayerNorm alone
    (1, 8, "bf16", True, True, True),
]


def _rln_inputs(i, case):
    rows, C, kind, has_branch, has_scale, has_norm = case
    rng = np.random.default_rng(4000 + i)
    r = lambda a: gi.round_kind(a.astype(np.float32), kind)  # noqa: E731
    x = r(rng.standard_normal((rows, C), dtype=np.float32) * 1.5 + 0.3)
    branch = r(rng.standard_normal((rows, C), dtype=np.float32) * 2.0) if has_branch else None
    scale = r(0.5 * rng.random(C, dtype=np.float32) + 0.01) if has_scale else None
    gamma = r(1.0 + 0.2 * rng.standard_normal(C, dtype=np.float32)) if has_norm else None
    beta = r(0.1 * rng.standard_normal(C, dtype=np.float32)) if has_norm else None
    return x, branch, scale, gamma, beta


@pytest.mark.parametrize("idx", range(len(RLN_CASES)))
def test_residual_layernorm_bit_exact(idx):
    from come_b200.block import residual_layernorm
    from tests.gpu_util import TORCH_DTYPE, to_dev
    case = RLN_CASES[idx]
    rows, C, kind, has_branch, has_scale, has_norm = case
    x, branch, scale, gamma, beta = _rln_inputs(idx, case)
    norm = None
    if has_norm:
        norm = torch.nn.LayerNorm(C, eps=1e-6).cuda().to(TORCH_DTYPE[kind])
        with torch.no_grad():
            norm.weight.copy_(to_dev(gamma, kind))
            norm.bias.copy_(to_dev(beta, kind))
    dev = lambda a: None if a is None else to_dev(a, kind)  # noqa: E731
    x_out, normed = residual_layernorm(dev(x), dev(branch), dev(scale), norm)
    ref_x, ref_n = orc.residual_layer_norm(x, branch, scale, gamma, beta, 1e-6, kind)
    assert np.array_equal(to_np(x_out), ref_x)
    if has_norm:
        assert np.array_equal(to_np(normed), ref_n)
        # and within one unit in the last place of PyTorch's own LayerNorm on the same rows
        with torch.no_grad():
            theirs = to_np(norm(to_dev(ref_x, kind)))
        ulp = {"bf16": 2.0 ** -7, "f16": 2.0 ** -10, "f32": 2.0 ** -20}[kind]
        assert np.all(np.abs(theirs - ref_n) <= ulp * np.maximum(np.abs(ref_n), 1.0))
    else:
        assert normed is None


def test_residual_layernorm_in_place_and_errors():
    from come_b200 import _lib
    from come_b200._torch_util import ptr, stream_ptr
    from come_b200.block import residual_layernorm
    from tests.gpu_util import to_dev
    case = (300, 1024, "bf16", True, True, True)
    x, branch, scale, gamma, beta = _rln_inputs(99, case)
    ref_x, ref_n = orc.residual_layer_norm(x, branch, scale, gamma, beta, 1e-5, "bf16")
    dx, db, ds, dg, dbeta = (to_dev(a, "bf16") for a in (x, branch, scale, gamma, beta))
    # x_out over x and normed over branch: a row is read completely before it is written
    _lib.check(_lib.lib().come_residual_layernorm(ptr(dx), ptr(db), ptr(ds), 300, 1024, _lib.COME_BF16, ptr(dg), ptr(dbeta),
                                                  1e-5, ptr(dx), ptr(db), stream_ptr(dx.device)))
    assert np.array_equal(to_np(dx), ref_x) and np.array_equal(to_np(db), ref_n)
    with pytest.raises(NotImplementedError):  # 8200 bytes per row
        residual_layernorm(torch.zeros(4, 4100, device="cuda", dtype=torch.bfloat16), None, None,
                           torch.nn.LayerNorm(4100).cuda().bfloat16())
    with pytest.raises(ValueError):
        residual_layernorm(dx, None, None, None)
    with pytest.raises(ValueError):
        residual_layernorm(dx, db[:10], None, None)
    assert _lib.device_status() == 0


def test_fused_elementwise_path_matches_module_path():
    """The aggregator with the fused LayerScale + residual + LayerNorm kernels against the module-by-module path:
    same arithmetic except the summation order inside the LayerNorm statistics."""
    from come_b200 import _lib
    from come_b200.fused import FusedAggregator
    from come_b200.token_merger import MergePlan
    rng = np.random.default_rng(13)
    C, heads, depth, start, side, B, S = 128, 2, 3, 5, 7, 1, 3
    N, M = start + side * side, 4
    core, params = _small_model(rng, depth, C, heads, 0.5, torch.bfloat16)
    fused, plain = FusedAggregator(core), FusedAggregator(core, fuse_elementwise=False)
    tokens = gi.round_kind(rng.standard_normal((B, S, N, C), dtype=np.float32), "bf16")
    mask = rng.random((B * S, M)) < 0.5
    plan = MergePlan(torch.from_numpy(mask).cuda(), _lib.Layout.two_d(start, side, side, 3, 3))
    t = torch.from_numpy(tokens).cuda().bfloat16()
    with torch.no_grad():
        a, _ = fused(t, plan)
        b, _ = plain(t, plan)
    ref = orc.fused_aggregator(tokens, mask, start, side, side, 3, 3, params["frame"], params["global"], heads)
    for layer in range(depth):
        # two bfloat16 evaluations whose LayerNorm outputs differ in the last place here and there: after six blocks they
        # are about as far from each other as each is from the float32 oracle
        assert _relative_error(to_np(a[layer]), to_np(b[layer])) < 1e-2
        assert _relative_error(to_np(a[layer]), ref[layer]) < FUSED_REL_TOL
        assert _relative_error(to_np(b[layer]), ref[layer]) < FUSED_REL_TOL


# ---- one scene sharded by frame over ranks ----------------------------------------------------------------------------
def _sharded_case(rng, frames, side=7, C=128, heads=2, depth=2, start=5):
    N, M = start + side * side, (side // 3) ** 2
    core, _ = _small_model(rng, depth, C, heads, 0.5, torch.bfloat16)
    tokens = torch.from_numpy(rng.standard_normal((1, frames, N, C), dtype=np.float32)).bfloat16()
    mask = torch.from_numpy(rng.random((frames, M)) < 0.5)
    return core, tokens, mask, (start, side, side, 3, 3)


@pytest.mark.parametrize("overlap", [False, True])
@pytest.mark.parametrize("world", [2, 3])
def test_sharded_aggregator_emulated_ranks(world, overlap):
    """Ranks emulated by host threads on one GPU: each runs ShardedFusedAggregator on its frames, and the K/V gather is a
    rendezvous between the threads (nothing on the device waits for anything).  Every rank's retained layers must equal
    its frames of the single-GPU result up to the rounding of differently tiled GEMMs.  ``overlap``: the exchange runs
    on a side stream while the rank attends to its own keys, the other ranks' keys are attended afterwards and the two
    results are merged."""
    import threading
    from come_b200 import _lib
    from come_b200.fused import FusedAggregator, ShardedFusedAggregator
    from come_b200.token_merger import MergePlan
    rng = np.random.default_rng(17)
    frames = 5
    core, tokens, mask, lay = _sharded_case(rng, frames)
    layout = _lib.Layout.two_d(*lay)
    tokens, mask = tokens.cuda(), mask.cuda()
    with torch.no_grad():
        whole, _ = FusedAggregator(core)(tokens, MergePlan(mask, layout))
    barrier = threading.Barrier(world)
    slots = [None] * world
    results, errors = [None] * world, []

    def gather(local, rows, rank):  # every rank deposits its rows, waits for the others, reads all
        torch.cuda.current_stream().synchronize()  # the ranks' streams are not ordered among themselves: hand over finished rows
        slots[rank] = local
        barrier.wait(timeout=120)
        out = torch.cat(slots, dim=0)
        barrier.wait(timeout=120)  # nobody overwrites a slot before everyone has read it
        return out

    def run(rank):
        try:
            torch.cuda.set_device(0)
            model = ShardedFusedAggregator(core, frames, world, rank, gather=gather, overlap=overlap)
            gp, lp = model.build_plans(mask, layout)
            with torch.no_grad():
                out, _ = model(tokens[:, model.f_lo:model.f_hi], gp, lp)
            results[rank] = (model.f_lo, model.f_hi, out)
        except Exception as e:  # noqa: BLE001
            errors.append((rank, repr(e)))
            barrier.abort()

    threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=300)
    assert not errors, errors
    torch.cuda.synchronize()
    covered = 0
    for lo, hi, out in results:
        covered += hi - lo
        for layer, ref in whole.items():
            assert out[layer].shape == ref[:, lo:hi].shape
            assert _relative_error(to_np(out[layer]), to_np(ref[:, lo:hi])) < 1e-2, (lo, hi, layer)
    assert covered == frames


def _sharded_worker(rank, world, port, q_out, overlap=False):
    import os
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from come_b200 import _lib
        from come_b200.fused import ShardedFusedAggregator
        rng = np.random.default_rng(17)
        core, tokens, mask, lay = _sharded_case(rng, 5)
        core = core.to(dev)
        model = ShardedFusedAggregator(core, 5, world, rank, overlap=overlap)
        gp, lp = model.build_plans(mask.to(dev), _lib.Layout.two_d(*lay))
        with torch.no_grad():
            out, _ = model(tokens[:, model.f_lo:model.f_hi].to(dev), gp, lp)
        q_out.put((rank, model.f_lo, model.f_hi, {k: v.float().cpu().numpy() for k, v in out.items()}))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("overlap", [False, True])
def test_sharded_aggregator_two_gpus(overlap):
    """Two processes, one GPU each, NCCL all-gather of the K/V rows (in line, or on a side stream behind attention to
    the local keys): against the single-GPU result."""
    import socket
    import torch.multiprocessing as mp
    from come_b200 import _lib
    from come_b200.fused import FusedAggregator
    from come_b200.token_merger import MergePlan
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    procs = [ctx.Process(target=_sharded_worker, args=(r, 2, port, q_out, overlap)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q_out.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    rng = np.random.default_rng(17)
    core, tokens, mask, lay = _sharded_case(rng, 5)
    with torch.no_grad():
        whole, _ = FusedAggregator(core)(tokens.cuda(), MergePlan(mask.cuda(), _lib.Layout.two_d(*lay)))
    for rank, lo, hi, out in results:
        for layer, ref in whole.items():
            assert _relative_error(out[layer], to_np(ref[:, lo:hi])) < 1e-2, (rank, layer)


# ---- the whole accelerated model: encoder-side merge + aggregator ----------------------------------------------------
def test_fused_model_against_oracle():
    """2 dense + 2 merged encoder blocks and 2 + 2 aggregator blocks on two frames of a 6 x 7 patch grid, against the
    float32 oracle chain (``oracle.fused_model``): the selection mask must be the oracle's (same bfloat16 confidences are
    not guaranteed after two bfloat16 blocks, so the device mask is handed to the oracle and must merge something), the
    retained layers agree within the bfloat16 tolerance; with a ratio of 0 the accelerated model equals the unmerged one."""
    from come_b200.fused import FusedModel
    from come_b200.vggt_arch import AggregatorCore, ConfidenceHead, PatchEncoderCore
    rng = np.random.default_rng(77)
    C, heads, patch, grid = 128, 2, 14, (6, 7)
    enc = PatchEncoderCore(embed_dim=C, depth=4, num_heads=heads, patch_size=patch, registers=4, grid=grid, mlp_ratio=2.0,
                           init_values=0.5)
    enc_params = []
    for blk in enc.blocks:
        p = gi.block_params(rng, C, heads, 2.0, False, 0.5, kind="bf16")
        blk.load_state_dict({k: torch.from_numpy(v) for k, v in p.items()})
        enc_params.append(dict(p, norm_eps=blk.norm1.eps))
    with torch.no_grad():  # parameters exactly representable in bfloat16, so that the oracle and the device hold the same numbers
        for p_ in list(enc.parameters()):
            p_.copy_(p_.bfloat16().float())
    core, params = _small_model(rng, 2, C, heads, 0.5, torch.bfloat16)
    head = ConfidenceHead(C, 32)
    with torch.no_grad():
        for p_ in head.parameters():
            p_.copy_(p_.bfloat16().float())
    f32 = lambda t: t.detach().float().cpu().numpy()  # noqa: E731
    enc_np = {"proj.weight": f32(enc.proj.weight), "proj.bias": f32(enc.proj.bias), "cls_token": f32(enc.cls_token),
              "register_tokens": f32(enc.register_tokens), "pos_embed": f32(enc.pos_embed), "norm.weight": f32(enc.norm.weight),
              "norm.bias": f32(enc.norm.bias), "patch": patch, "norm_eps": enc.norm.eps}
    head_np = {"fc1.weight": f32(head.fc1.weight), "fc1.bias": f32(head.fc1.bias), "fc2.weight": f32(head.fc2.weight),
               "fc2.bias": f32(head.fc2.bias)}
    tok_np = {"camera_token": f32(core.camera_token), "register_token": f32(core.register_token)}
    B, S = 1, 2
    images = gi.round_kind(rng.random((B, S, 3, grid[0] * patch, grid[1] * patch), dtype=np.float32), "bf16")
    model = FusedModel(enc.cuda().bfloat16(), core, head.cuda().bfloat16(), encoder_layer=1, threshold=0.5)
    with torch.no_grad():
        out, start = model(torch.from_numpy(images).cuda().bfloat16())
        mask = model.last_plan.mask.cpu().numpy()
        plain, _ = model.forward_unmerged(torch.from_numpy(images).cuda().bfloat16())
    assert start == 5 and 0 < mask.sum() < mask.size
    ref, _ = orc.fused_model(images, enc_np, enc_params, 1, head_np, tok_np, params["frame"], params["global"], heads, 3, 3, 0.5,
                             mask=mask)
    ref_mask = orc.fused_model(images, enc_np, enc_params, 1, head_np, tok_np, params["frame"], params["global"], heads, 3, 3, 0.5)[1]
    assert ref_mask.shape == mask.shape and ref_mask.sum() == mask.sum()  # the ranking merges the same number of windows
    N = 5 + grid[0] * grid[1]
    for layer in sorted(ref):
        got = to_np(out[layer])
        assert got.shape == (B, S, N, 2 * C)
        assert _relative_error(got, ref[layer]) < 2 * FUSED_REL_TOL, (layer, _relative_error(got, ref[layer]))
        assert to_np(plain[layer]).shape == got.shape
    never = FusedModel(enc, core, head, encoder_layer=1, threshold=0.0)
    with torch.no_grad():
        same, _ = never(torch.from_numpy(images).cuda().bfloat16())
    for layer in sorted(ref):
        assert _relative_error(to_np(same[layer]), to_np(plain[layer])) < 1e-2
