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


def _worker(rank, world, port, frames, q_out, mode):
    overlap, transport = mode != "inline", ("peer" if mode.startswith("overlap-peer") else "nccl")
    pulls_first = mode == "overlap-peer-pulls-first"
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from come_b200.chain import ShardedOpChain
        C, H, D = 64 * 4, 4, 64
        x, conf, q, kv = _scene(frames, C, H, D, dev)
        chain = ShardedOpChain(frames, num_heads=H, head_dim=D, layer_kinds=["frame", "global"], overlap=overlap,
                               transport=transport, pulls_first=pulls_first)
        gp, lp = chain.build_plans(conf)
        r0, r1 = chain.row_begin, chain.row_begin + lp.total
        kinds = ("frame", "global", "global", "global")  # the global layer three times: both window slots and a reuse
        outs = [chain.layer(gp, lp, x[chain.f_lo:chain.f_hi], q[r0:r1].contiguous(), kv[r0:r1].contiguous(), kind).cpu()
                for kind in kinds]
        # a second scene with other merge masks (other block heights) through the same chain object: the side stream, and
        # with the peer transport the windows, are kept
        gp, lp = chain.build_plans(1.0 - conf)
        r0, r1 = chain.row_begin, chain.row_begin + lp.total
        outs.append(chain.layer(gp, lp, x[chain.f_lo:chain.f_hi], q[r0:r1].contiguous(), kv[r0:r1].contiguous(), "global").cpu())
        from come_b200 import _lib
        status = _lib.device_status(clear=True)
        q_out.put((rank, chain.f_lo, chain.f_hi, outs, chain.exchange.transport, chain.exchange.peer_error, status))
        dist.barrier()
        chain.exchange.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode", ["inline", "overlap-nccl", "overlap-peer", "overlap-peer-pulls-first"])
def test_sharded_chain_matches_single_gpu(mode):
    """In line, the exchange changes nothing: bit-identical frames.  Overlapped (local keys first, the gathered keys
    afterwards, merged from the log-sum-exps) the global layer differs by the rounding of the two partial outputs."""
    import torch.multiprocessing as mp
    from come_b200.chain import ShardedOpChain
    frames, C, H, D = 5, 256, 4, 64
    world = 2
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, frames, q_out, mode)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q_out.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    dev = torch.device("cuda", 0)
    x, conf, q, kv = _scene(frames, C, H, D, dev)
    single = ShardedOpChain(frames, num_heads=H, head_dim=D, layer_kinds=["frame", "global"])  # no process group: 1 rank
    gp, lp = single.build_plans(conf)
    P = lp.total
    want = [single.layer(gp, lp, x, q[:P].contiguous(), kv[:P].contiguous(), kind).cpu() for kind in ("frame", "global")]
    gp, lp = single.build_plans(1.0 - conf)
    P = lp.total
    second = single.layer(gp, lp, x, q[:P].contiguous(), kv[:P].contiguous(), "global").cpu()
    want = [want[0], want[1], want[1], want[1], second]
    for rank, f_lo, f_hi, outs, transport, peer_error, status in results:
        assert status == 0, f"rank {rank}: device status word {status:#x}"
        if mode.startswith("overlap-peer"):
            assert transport == "peer", f"rank {rank} fell back to NCCL: {peer_error}"
        for kind, got, ref in zip(("frame", "global", "global", "global", "global"), outs, want):
            tol = 2e-2 if (mode != "inline" and kind == "global") else 0.0
            torch.testing.assert_close(got, ref[f_lo:f_hi], atol=tol, rtol=0)


def _gather_worker(rank, world, port, q_out):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from come_b200 import _lib
        from come_b200.dist import PeerGather, block_order
        rows = [1000 + 37 * r for r in range(world)]  # uneven blocks
        shape = (2, 4, 64)
        pg = PeerGather(rows, rank, 2 * 4 * 64 * 2, dev)
        assert pg.ok, pg.error
        side = torch.cuda.Stream(device=dev)
        worst = 0.0
        for k in range(5):  # both slots, several times; alternate the block order
            blocks = [torch.full((rows[r],) + shape, float(10 * k + r), dtype=torch.bfloat16) + torch.arange(rows[r]).view(-1, 1, 1, 1).bfloat16() * 0
                      for r in range(world)]
            local = blocks[rank].to(dev)
            out = torch.zeros((sum(rows),) + shape, dtype=torch.bfloat16, device=dev)
            remote_first = bool(k & 1)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                pg.gather(local, out, remote_first=remote_first)
            torch.cuda.current_stream(dev).wait_stream(side)
            want = torch.cat([blocks[r] for r in block_order(world, rank, remote_first)])
            worst = max(worst, float((out.cpu().float() - want.float()).abs().max()))
        status = _lib.device_status(clear=True)
        q_out.put((rank, worst, status))
        torch.cuda.synchronize()
        dist.barrier()
        pg.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_gather_uneven_blocks():
    """Five exchanges of uneven blocks through the peer-mapped windows (both slots, both block orders): every rank ends up
    with every rank's rows, and no wait ran out."""
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gather_worker, args=(r, world, port, q_out)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q_out.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, worst, status in results:
        assert worst == 0.0 and status == 0, (rank, worst, status)
