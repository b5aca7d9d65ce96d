"""Two-GPU check of the frame-sharded operator chain (skipped on a single-GPU box): every rank's output frames must
equal the frames a single GPU computes for the whole scene."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _scene(frames, C, H, D, device):
    g = torch.Generator(device="cpu").manual_seed(5)
    x = torch.randn((frames, 1374, C), generator=g).bfloat16().to(device)
    conf = torch.rand((1, frames * 1369), generator=g).bfloat16().to(device)
    q = torch.randn((frames * 1374, H, D), generator=g).bfloat16().to(device)
    kv = torch.randn((frames * 1374, 2, H, D), generator=g).bfloat16().to(device)
    return x, conf, q, kv


def _worker(rank, world, port, frames, q_out, overlap):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from come_b200.chain import ShardedOpChain
        C, H, D = 64 * 4, 4, 64
        x, conf, q, kv = _scene(frames, C, H, D, dev)
        chain = ShardedOpChain(frames, num_heads=H, head_dim=D, layer_kinds=["frame", "global"], overlap=overlap)
        gp, lp = chain.build_plans(conf)
        r0, r1 = chain.row_begin, chain.row_begin + lp.total
        outs = [chain.layer(gp, lp, x[chain.f_lo:chain.f_hi], q[r0:r1].contiguous(), kv[r0:r1].contiguous(), kind).cpu()
                for kind in ("frame", "global")]
        q_out.put((rank, chain.f_lo, chain.f_hi, outs))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("overlap", [False, True])
def test_sharded_chain_matches_single_gpu(overlap):
    """In line, the exchange changes nothing: bit-identical frames.  Overlapped (local keys first, the gathered keys
    afterwards, merged from the log-sum-exps) the global layer differs by the rounding of the two partial outputs."""
    import torch.multiprocessing as mp
    from come_b200.chain import ShardedOpChain
    frames, C, H, D = 5, 256, 4, 64
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, frames, q_out, overlap)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q_out.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    dev = torch.device("cuda", 0)
    x, conf, q, kv = _scene(frames, C, H, D, dev)
    single = ShardedOpChain(frames, num_heads=H, head_dim=D, layer_kinds=["frame", "global"])  # no process group: 1 rank
    gp, lp = single.build_plans(conf)
    P = lp.total
    want = [single.layer(gp, lp, x, q[:P].contiguous(), kv[:P].contiguous(), kind).cpu() for kind in ("frame", "global")]
    for rank, f_lo, f_hi, outs in results:
        for kind, got, ref in zip(("frame", "global"), outs, want):
            tol = 2e-2 if (overlap and kind == "global") else 0.0
            torch.testing.assert_close(got, ref[f_lo:f_hi], atol=tol, rtol=0)
