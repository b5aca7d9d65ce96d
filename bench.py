#!/usr/bin/env python3
"""Benchmark of the Co-Me hot path on B200: ms/scene of the merge -> biased attention -> unmerge chain at the
VGGT-1B shapes (100 frames of 518x518: 1374 tokens x 1024 channels per frame, 16 heads x 64, 24 frame + 24 global
attention layers, 3x3 windows at a 50 % merge ratio; the 8-frame scene as the extra key `scene8`), plus merge/unmerge
GB/s and biased-attention TFLOP/s.

    python bench.py --gpus N --steps K --warmup W            # this library: ONE 100-frame scene per step, frames sharded over the N GPUs
    python bench.py --impl reference ...                     # the CPU restatement of the reference path (rank 0), a bounded sample

Prints ONE JSON line (rank 0).  Inputs are synthetic (seeded).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FRAMES, GRID, WIN, START, CH, HEADS, HDIM = 8, 37, 3, 5, 1024, 16, 64
N_TOK = START + GRID * GRID  # 1374
N_WIN = (GRID // WIN) ** 2   # 144
LAYERS = ["frame", "global"] * 24
UNIT = "ms/scene"
FRAMES_BY_WORKLOAD = {"frames100": 100, "frames8": 8}


def metric_name(frames):
    return f"come_vggt_hot_path_ms_per_scene_{frames}f"


def workload_name(frames=FRAMES):
    return (f"VGGT-1B-shape Co-Me op chain, {frames} frames x 518x518 (1374 tok x 1024 ch), 48 attention layers "
            f"(24 frame + 24 global) each = merge + biased varlen attention (16 heads x 64) + unmerge, 3x3 windows at "
            f"50 % per frame; projections/MLP GEMMs excluded")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=float(p["hbm_gbs"]), tflops=float(p["bf16_tflops"]),
                    tflops_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


# ---- clocks sampler --------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ---- CPU restatement of the reference path (oracle) ---------------------------------------------------------
class CpuSceneSample:
    """A bounded sample of one scene of the operator chain on the host cores (all threads): selection, merge and unmerge
    with the C oracle, attention with the PyTorch-operator restatement of the reference's float32 biased softmax (the
    reference's fallback path is PyTorch; its matrix products run on PyTorch's BLAS).

    Every ``run()`` times, in float32 (the dtype of the reference's CPU path): the selection, a full merge and a full
    unmerge of all frames, the frame attention of ``frame_sample`` whole frames with all heads (all frames by default),
    and the global attention of ``attn_heads`` heads on ``attn_rows`` query rows against all keys.  The frame figure is
    scaled by ``frames / frame_sample`` and the global figure by ``heads / attn_heads * rows / attn_rows``; both are summed
    over the 24 + 24 layers.  The scene figure is therefore an extrapolation (``extrapolated`` in the report) and
    ``sample_s`` says how many seconds were timed (a few seconds per sample on 16 cores).  (The PyTorch expression
    materialises the score matrix; ``oracle/torch_path.py`` walks the query rows in blocks that keep it under 1.5 GB.)"""

    def __init__(self, frames, attn_rows=8192, frame_sample=100, attn_heads=4):
        from oracle import clib, torch_path
        self.clib, self.attn, self.frames, self.attn_rows = clib, torch_path, frames, attn_rows
        self.frame_sample = min(frames, frame_sample)
        # all the host threads this process may use: a multi-process launcher exports OMP_NUM_THREADS=1 for its workers,
        # which would time the CPU path on one core
        threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        clib.set_num_threads(threads)
        torch_path.set_num_threads(threads)
        rng = np.random.default_rng(0)
        self.tokens = rng.standard_normal((frames, N_TOK, CH), dtype=np.float32)
        self.conf = rng.random((1, frames * GRID * GRID), dtype=np.float32)
        mask = clib.select_windows(self.conf, 1, frames, GRID, GRID, WIN, WIN, 0.5, "pairwise-rank", "frame")
        _, off, _, w = clib.token_merge_2d(self.tokens[:1], START, WIN, WIN, GRID, GRID, mask[:1])
        self.P = int(frames * N_TOK - 8 * mask.sum())
        # attention inputs: all heads for the sampled frames, one head for the global slice
        self.qkv_frames = rng.standard_normal((self.frame_sample * N_TOK, 3, HEADS, HDIM), dtype=np.float32)
        self.attn_heads = min(HEADS, attn_heads)
        self.qkv_heads = rng.standard_normal((self.P, 3, self.attn_heads, HDIM), dtype=np.float32)

    def run(self):
        clib, frames = self.clib, self.frames
        t_all = time.perf_counter()
        t0 = time.perf_counter()
        mask = clib.select_windows(self.conf, 1, frames, GRID, GRID, WIN, WIN, 0.5, "pairwise-rank", "frame")
        t_sel = time.perf_counter() - t0
        t0 = time.perf_counter()
        out, off, rev, w = clib.token_merge_2d(self.tokens, START, WIN, WIN, GRID, GRID, mask)
        t_merge = time.perf_counter() - t0
        t0 = time.perf_counter()
        clib.token_split(out, rev)
        t_unmerge = time.perf_counter() - t0
        P = out.shape[0]
        bias = np.log(w)
        fs = self.frame_sample
        cu_f = off[: fs + 1].astype(np.int32)
        t0 = time.perf_counter()
        self.attn.attention_bias(self.qkv_frames[: cu_f[-1]], bias[: cu_f[-1]], cu_f, HDIM ** -0.5)
        t_frame = (time.perf_counter() - t0) * (frames / fs)
        rows = min(self.attn_rows, P)
        t0 = time.perf_counter()
        self.attn.attention_bias(self.qkv_heads[:P], bias, np.array([0, P], np.int32), HDIM ** -0.5, 0, rows)
        t_global = (time.perf_counter() - t0) * (HEADS / self.attn_heads) * (P / rows)
        sample_s = time.perf_counter() - t_all
        n_f = sum(1 for k in LAYERS if k == "frame")
        n_g = len(LAYERS) - n_f
        per_scene = t_sel + len(LAYERS) * (t_merge + t_unmerge) + n_f * t_frame + n_g * t_global
        detail = dict(select_ms=t_sel * 1e3, merge_ms=t_merge * 1e3, unmerge_ms=t_unmerge * 1e3,
                      attn_frame_layer_ms=t_frame * 1e3, attn_global_layer_ms=t_global * 1e3)
        return per_scene * 1e3, sample_s, detail

    def describe(self):
        return (f"per step: select + merge + unmerge of all {self.frames} frames (fp32, {self.frames}x{N_TOK}x{CH}), frame "
                f"attention of {self.frame_sample} whole frames x {HEADS} heads (scaled by {self.frames}/{self.frame_sample}), "
                f"global attention of {self.attn_heads} heads x {min(self.attn_rows, self.P)} of {self.P} query rows against all keys "
                f"(scaled to {HEADS} heads and all rows); x24 frame + x24 global layers")


def cpu_baseline_report(frames, steps, warmup=0):
    """``steps`` samples of the CPU path (median), as the ``cpu_baseline`` object of the JSON line."""
    sample = CpuSceneSample(frames)
    vals, secs, detail = [], [], {}
    for i in range(warmup + steps):
        v, s_, detail = sample.run()
        if i >= warmup:
            vals.append(v)
            secs.append(s_)
    return {"value": statistics.median(vals), "unit": UNIT, "cores": sample.attn.num_threads(), "kind": "port",
            "extrapolated": True, "sample_s": sum(secs), "samples": len(vals), "sample": sample.describe(), "detail": detail,
            "note": "restatement of the reference's PyTorch fallback (float32): merge / unmerge in C with OpenMP, attention with "
                    "PyTorch CPU operators; a reported baseline, extrapolated from the timed sample, not a measurement of the whole scene"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    frames = FRAMES_BY_WORKLOAD[args.workload]
    rep = cpu_baseline_report(frames, args.steps, args.warmup)
    val = rep["value"]
    line = {
        "impl": "reference", "metric": metric_name(frames), "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": val, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic (seeded)", "config": {"workload": workload_name(frames)},
        "extrapolated": True, "kind": "port", "sample_s": rep["sample_s"],
        "cpu_baseline": rep,
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---- GPU arm ---------------------------------------------------------------------------------------------------
COMM_SMS = 16  # SMs left to the all-gather kernel while attention to the local keys runs beside it


def init_ranks(cap_nccl_ctas=False):
    import torch
    import torch.distributed as dist
    if cap_nccl_ctas:
        # An all-gather that runs beside the persistent attention kernel completes only when ALL its CTAs have run: keep
        # their number within the SMs the attention launch leaves free (GlobalExchange.comm_sms), or the last ones wait for
        # the attention kernel to end and nothing overlaps.
        os.environ.setdefault("NCCL_MAX_CTAS", str(COMM_SMS))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    return torch, dist, world, rank, local, dev


def _lib_status_clear():
    from come_b200 import _lib
    return _lib.device_status(clear=True)


def sharded_check(torch, dist, world, rank, dev, transport="nccl", hidden=True, pulls_first=False):
    """Before anything is timed at N > 1: a small scene (one frame layer + one global layer) run sharded over the ranks
    and unsharded on every rank.  With the exchange in line the sharded frames must equal the unsharded ones bit for bit;
    with the exchange hidden behind attention to the local keys the global layer may differ by the rounding of the two
    partial outputs (bar 2e-2 absolute).  Raises on a mismatch of the in-line form on any rank; a hidden form that fails
    (an exception, a wait that ran out or a mismatch on any rank) is reported in ``hidden_failed`` and the caller falls
    back to the in-line exchange."""
    from come_b200.chain import ShardedOpChain
    frames, C, H, D = max(8, world), 256, 4, 64
    g = torch.Generator(device="cpu").manual_seed(5)
    x = torch.randn((frames, N_TOK, C), generator=g).bfloat16().to(dev)
    conf = torch.rand((1, frames * GRID * GRID), generator=g).bfloat16().to(dev)
    q = torch.randn((frames * N_TOK, H, D), generator=g).bfloat16().to(dev)
    kv = torch.randn((frames * N_TOK, 2, H, D), generator=g).bfloat16().to(dev)
    kinds = ["frame", "global"]
    whole = ShardedOpChain(frames, None, START, GRID, GRID, WIN, WIN, 0.5, H, D, kinds)
    whole.world, whole.rank, whole.f_lo, whole.f_hi = 1, 0, 0, frames  # every rank computes the whole scene for itself
    gp, lp = whole.build_plans(conf)
    P = lp.total
    want = [whole.layer(gp, lp, x, q[:P].contiguous(), kv[:P].contiguous(), k) for k in kinds]
    res = {"rows": P, "frames": frames}
    ok = True
    for overlap in ((False, True) if hidden else (False,)):  # the hidden exchange is checked where the timed run uses it
        chain = ShardedOpChain(frames, None, START, GRID, GRID, WIN, WIN, 0.5, H, D, kinds, overlap=overlap, transport=transport,
                               pulls_first=pulls_first and overlap)
        gp, lp = chain.build_plans(conf)
        r0, r1 = chain.row_begin, chain.row_begin + lp.total
        diffs, failed = [], 0.0
        try:
            for kind, ref in zip(kinds, want):
                got = chain.layer(gp, lp, x[chain.f_lo:chain.f_hi], q[r0:r1].contiguous(), kv[r0:r1].contiguous(), kind)
                diffs.append(float((got.float() - ref[chain.f_lo:chain.f_hi].float()).abs().max().item()) if got.numel() else 0.0)
            if _lib_status_clear() != 0:
                failed = 1.0
        except Exception as e:  # noqa: BLE001 - the ranks must still meet in the reduction below
            if not overlap:
                raise
            failed, diffs = 1.0, [0.0, 0.0]
            res["hidden_error"] = repr(e)
        t = torch.tensor(diffs + [failed], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        worst = t.tolist()
        if overlap:
            res["overlapped_max_abs_diff"] = {"frame": worst[0], "global": worst[1], "bar_global": 2e-2}
            res["overlapped_transport"] = chain.exchange.transport
            res["pulls_first"] = bool(pulls_first)
            res["hidden_failed"] = bool(worst[2] != 0.0 or worst[0] != 0.0 or worst[1] > 2e-2)
            torch.cuda.synchronize()
            dist.barrier()  # every rank has finished its pulls before anyone releases its window
            chain.exchange.close()
        else:
            res["in_line_bit_exact"] = worst[0] == 0.0 and worst[1] == 0.0
            ok = ok and res["in_line_bit_exact"] and worst[2] == 0.0
    res["ok"] = bool(ok)
    if not ok:
        raise RuntimeError(f"sharded scene differs from the unsharded one: {res}")
    return res


def run_frames(args):
    """The default arm: ONE scene of 100 frames (137,400 tokens before merging) sharded by frame over the ranks.  Frame
    layers are local; a global layer gathers the merged K/V rows of the other ranks (pulls out of peer-mapped windows, or an
    NCCL all-gather) on a side stream while the local query rows attend to the local keys, then attends them to the gathered
    rows and merges the two results (strong scaling: the scene is fixed, more GPUs shorten it).  At N = 1 there is no
    exchange and the global layer is one launch."""
    from come_b200.dist import hiding_exchange_pays
    frames = FRAMES_BY_WORKLOAD[args.workload]
    world_env = int(os.environ.get("WORLD_SIZE", "1"))
    # auto: with peer windows the exchange is hidden behind the attention to the local keys at every N (measured best on 2, 4
    # and 8 GPUs, even where that attention is shorter than the exchange); with NCCL it is hidden where the model of a global
    # layer says it pays (2 to 4 GPUs for the 100-frame scene) and in line otherwise.
    rows_est = frames * (START + GRID * GRID - (GRID // WIN) ** 2 // 2 * (WIN * WIN - 1))  # half of the windows merged: 798 per frame
    shape = (rows_est, world_env, 2 * HEADS * HDIM * 2, HEADS, HDIM)
    if world_env <= 1 or args.overlap == "off":
        overlap = False
    else:
        overlap = args.overlap == "on" or args.transport == "peer" or hiding_exchange_pays(*shape)
    pulls_first = overlap and args.transport == "peer" and args.pulls_first == "on"
    torch, dist, world, rank, local, dev = init_ranks(cap_nccl_ctas=overlap and args.transport == "nccl")
    from come_b200 import _lib
    from come_b200.chain import ShardedOpChain
    pk = peaks()
    check = sharded_check(torch, dist, world, rank, dev, args.transport, hidden=overlap, pulls_first=pulls_first) if world > 1 else None
    fallback = None
    if check is not None and check.get("hidden_failed"):
        # the hidden exchange did not reproduce the unsharded scene on this box: the timed run keeps the exchange in line
        fallback = check.get("hidden_error") or "the hidden exchange failed the sharded check"
        overlap = pulls_first = False
    chain = ShardedOpChain(frames, None, START, GRID, GRID, WIN, WIN, 0.5, HEADS, HDIM, LAYERS, overlap=overlap,
                           transport=args.transport, pulls_first=pulls_first)
    g = torch.Generator(device="cpu").manual_seed(4321)
    conf_host = torch.rand((1, frames * GRID * GRID), generator=g).bfloat16().pin_memory()  # replicated on every rank
    conf = conf_host.to(dev)
    gp, lp = chain.build_plans(conf)
    n_local = chain.f_hi - chain.f_lo
    P, P_local = gp.total, lp.total
    # this rank's inputs start in pinned host memory (the end-to-end region copies them in every step)
    gl = torch.Generator(device="cpu").manual_seed(100 + rank)
    x_host = torch.empty((n_local, N_TOK, CH), dtype=torch.bfloat16).pin_memory()
    q_host = torch.empty((P_local, HEADS, HDIM), dtype=torch.bfloat16).pin_memory()
    kv_host = torch.empty((P_local, 2, HEADS, HDIM), dtype=torch.bfloat16).pin_memory()
    for t_ in (x_host, q_host, kv_host):  # drawn in slices: a float32 draw of the whole tensor would double the host memory
        flat = t_.view(-1)
        for i in range(0, flat.numel(), 1 << 24):
            flat[i:i + (1 << 24)] = torch.randn(min(1 << 24, flat.numel() - i), generator=gl).bfloat16()
    out_host = torch.empty((n_local, N_TOK, CH), dtype=torch.bfloat16).pin_memory()
    x, q, kv = x_host.to(dev), q_host.to(dev), kv_host.to(dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step(x_, conf_, q_, kv_, timers=None):
        gp_, lp_ = chain.build_plans(conf_)
        out = None
        for kind in LAYERS:
            if timers is None:
                out = chain.layer(gp_, lp_, x_, q_, kv_, kind)
            else:
                out = chain.layer(gp_, lp_, x_, q_, kv_, kind, timers=timers)
        return out

    for _ in range(max(args.warmup, 3)):
        step(x, conf, q, kv)
    barrier()
    if _lib.device_status(clear=False) != 0:
        raise RuntimeError("attention kernel raised the device status word during warm-up")
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()  # the other ranks wait for rank 0's sampler here, not inside the first all-gather of the timed region
    # ---- timed region 0 (-> `value`, `roofline`, `split`): inputs resident in HBM; every kernel family of every layer is
    # bracketed by CUDA events on the launching stream, and the all-gather by events on its side stream, in these same
    # steps (a step is hundreds of milliseconds: the events cost nothing against it, and the split describes the very
    # steps `value` is taken from) ----------------------------------------------------------------------------------
    timers = []
    if chain.exchange is not None:
        chain.exchange.events = []
    s, e = ev(), ev()
    s.record()
    for _ in range(args.steps):
        step(x, conf, q, kv, timers)
    e.record()
    barrier()
    resident_ms = s.elapsed_time(e)
    exch = list(chain.exchange.events) if chain.exchange is not None and chain.exchange.events else []
    if chain.exchange is not None:
        chain.exchange.events = None
    # ---- timed region 1 (-> `e2e`): the same step through the same public calls with HOST buffers: this rank's inputs are
    # copied from pinned host memory and its restored tokens are copied back, inside the timed region, every step ------
    h2d = (x_host.numel() + q_host.numel() + kv_host.numel() + conf_host.numel()) * 2
    d2h = out_host.numel() * 2
    s, e = ev(), ev()
    barrier()
    s.record()
    for _ in range(args.steps):
        xd, cd = x_host.to(dev, non_blocking=True), conf_host.to(dev, non_blocking=True)
        qd, kvd = q_host.to(dev, non_blocking=True), kv_host.to(dev, non_blocking=True)
        out = step(xd, cd, qd, kvd)
        out_host.copy_(out.reshape(out_host.shape), non_blocking=True)
    e.record()
    barrier()
    e2e_ms = s.elapsed_time(e)
    clocks = sampler.stop() if rank == 0 else None
    if _lib.device_status(clear=False) != 0:
        raise RuntimeError("attention kernel raised the device status word during the timed region")
    n_inst = args.steps
    fam = {"merge": 0.0, "frame_attn": 0.0, "global_attn": 0.0, "unmerge": 0.0}
    for kind, e4 in timers:
        fam["merge"] += e4[0].elapsed_time(e4[1]) / n_inst
        fam["frame_attn" if kind == "frame" else "global_attn"] += e4[1].elapsed_time(e4[2]) / n_inst
        fam["unmerge"] += e4[2].elapsed_time(e4[3]) / n_inst
    split = {f"{k}_ms": v for k, v in fam.items()}
    if exch:
        gather_ms = [a.elapsed_time(b) for a, b, _, _ in exch]
        exposed = [max(0.0, c.elapsed_time(b)) for _, b, c, _ in exch]  # gather still running when the local attention ended
        local_ms = [a.elapsed_time(c) for a, _, c, _ in exch]
        split.update(allgather_ms_per_global_layer=statistics.mean(gather_ms), allgather_exposed_ms_per_global_layer=statistics.mean(exposed),
                     local_keys_attn_ms_per_global_layer=statistics.mean(local_ms))
    vals = torch.tensor([resident_ms, e2e_ms] + [split[k] for k in sorted(split)], dtype=torch.float64, device=dev)
    rows_t = torch.tensor([P_local, -P_local], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        dist.all_reduce(rows_t, op=dist.ReduceOp.MAX)
    resident_ms, e2e_ms = vals[0].item(), vals[1].item()
    split = {k: vals[2 + i].item() for i, k in enumerate(sorted(split))}  # max over ranks of every entry
    split["rows_per_rank"] = [int(-rows_t[1].item()), int(rows_t[0].item())]
    if exch:
        split["exchange_transport"] = chain.exchange.transport
        if chain.exchange.peer_error:
            split["exchange_fallback_reason"] = chain.exchange.peer_error

    if rank == 0:
        per_scene = resident_ms / args.steps
        seg = (gp.offset[1:] - gp.offset[:-1]).tolist()
        n_f = sum(1 for k in LAYERS if k == "frame")
        n_g = len(LAYERS) - n_f
        flops_frame, flops_global = sum(4.0 * L * L * HDIM * HEADS for L in seg), 4.0 * P * P * HDIM * HEADS
        attn_flops = n_f * flops_frame + n_g * flops_global                 # the whole scene, all ranks together
        attn_ms = split["frame_attn_ms"] + split["global_attn_ms"]          # slowest rank, per scene
        achieved = attn_flops / world / (attn_ms * 1e-3) / 1e12             # per GPU
        es = 2
        merge_bytes = n_local * N_TOK * CH * es + P_local * CH * es + n_local * N_WIN + (n_local + 1) * 4
        unmerge_bytes = P_local * CH * es + n_local * N_TOK * 8 + n_local * N_TOK * CH * es
        kv_bytes = P * 2 * HEADS * HDIM * 2
        items = -(-split["rows_per_rank"][1] // 384) * HEADS
        line = {
            "metric": metric_name(frames), "value": per_scene, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": per_scene, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded)",
            "config": {"workload": workload_name(frames), "merged_tokens": P, "frames_per_s": frames / per_scene * 1e3,
                       "exchange": ("none" if world == 1 else ("in line" + (f" (fallback: {fallback})" if fallback else "") if not chain.overlap else
                                    ("hidden behind attention to the local keys" if not pulls_first else
                                     "pulls started first, attention to the local keys fills in behind them"))),
                       "parallelism": ("one GPU: the whole scene, no exchange" if world == 1 else
                                       f"frames sharded over {world} GPUs; frame layers local; a global layer all-gathers "
                                       f"{kv_bytes / 1e6:.0f} MB of merged K/V "
                                       + ("with copy-engine transfers out of peer-mapped windows" if (chain.overlap and chain.exchange.transport == "peer")
                                          else "over NCCL")
                                       + (" on a side stream while the local query rows attend to the local keys, then attends "
                                          "them to the gathered rows and merges the two results from their log-sum-exps"
                                          if chain.overlap else " in line, then attends the local query rows to all keys")),
                       "l2": "inputs larger than L2 (the merged K/V of one layer alone is 327 MB)",
                       "launch": "kernel by kernel from Python (a step is hundreds of ms of device time)"},
            "roofline": {"kernel": f"attn_fwd_sm100_kernel ({n_f} frame + {n_g} global layers per scene)", "bound": "tensor",
                         "achieved": achieved, "peak": pk["tflops_sustained"], "unit": "TFLOP/s",
                         "frac": achieved / pk["tflops_sustained"],
                         "peak_source": pk["source"] + " cuBLAS bf16, sustained loop (steps of this workload keep the GPU at its power cap for seconds)",
                         "frac_of_burst_peak": achieved / pk["tflops"],
                         "per": "GPU (slowest rank)",
                         "traffic": 814.9e6 if (world == 1 and frames == 100) else None,
                         "traffic_note": ("bytes per global-layer launch (80,672 merged tokens): dram__bytes_read.sum 658.3 MB + "
                                          "dram__bytes_write.sum 156.6 MB from a one-pass ncu capture of that launch; algorithmic "
                                          "660.9 MB = packed q / k / v once + output (the K / V re-reads of the 3376 work items are "
                                          "served by L2)" if (world == 1 and frames == 100) else
                                          "captured for the one-GPU 100-frame launch only (profiles/)"),
                         "timing": "CUDA events around every attention call of the timed steps themselves (launches of 0.2 to 33 ms: host cost is hidden)",
                         "frame_tflops": n_f * flops_frame / world / (split["frame_attn_ms"] * 1e-3) / 1e12,
                         "global_tflops": n_g * flops_global / world / (split["global_attn_ms"] * 1e-3) / 1e12,
                         "work_items_per_cta_global": items / 148.0,
                         "share_of_scene": attn_ms / per_scene},
            "roofline_merge": {"bound": "hbm", "achieved": merge_bytes * len(LAYERS) / (split["merge_ms"] * 1e-3) / 1e9,
                               "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": merge_bytes * len(LAYERS) / (split["merge_ms"] * 1e-3) / 1e9 / pk["hbm_gbs"],
                               "per": "GPU", "bytes_per_launch": merge_bytes},
            "roofline_unmerge": {"bound": "hbm", "achieved": unmerge_bytes * len(LAYERS) / (split["unmerge_ms"] * 1e-3) / 1e9,
                                 "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": unmerge_bytes * len(LAYERS) / (split["unmerge_ms"] * 1e-3) / 1e9 / pk["hbm_gbs"],
                                 "per": "GPU", "bytes_per_launch": unmerge_bytes},
            "split": split,
            "e2e": {"value": e2e_ms / args.steps, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "note": "per rank: its frames, its q / k / v rows and the replicated confidences in, its restored tokens out"},
            "gpu_launches": (5 + n_f * 3 + n_g * ((7 if chain.exchange.transport == "peer" else 5) if (chain.overlap and world > 1) else 3)) * args.steps,
            "clocks": clocks,
        }
        if check is not None:
            line["sharded_check"] = check
        if world == 1 and not args.no_scene8:
            line["scene8"] = scene8_measure(torch, dev, pk, max(5, args.steps))
        if world == 1 and not args.no_micro:
            line["kernels"] = micro(torch, dev, pk)
            # the whole alternating-attention stack (48 blocks with their cuBLAS GEMMs) around the same kernels,
            # merged against unmerged: the reference's own end-to-end comparison (src/bench.py), 5 scenes per arm
            agg = aggregator_measure(8, 24, 5, report=False)
            agg.pop("only")
            line["aggregator_model"] = agg
            whole = model_measure(8, 5, report=False)
            whole.pop("only")
            line["model"] = whole
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline_report(frames, 3)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def scene8_measure(torch, dev, pk, steps):
    """The 8-frame scene of the same chain on one GPU (48 x (merge + attention + unmerge), one selection + plan), as ONE
    CUDA graph: ms/scene with inputs resident (L2 flushed between steps), end to end with host buffers, and device time
    per kernel family."""
    from come_b200 import _lib
    from come_b200.chain import CoMeOpChain
    from come_b200.flash_attn import flash_attn_varlen_qkvpacked_func_w_perkey_bias as attn_fn
    from come_b200.static_scene import StaticScene
    F8 = 8
    chain = CoMeOpChain(F8, START, GRID, GRID, WIN, WIN, 0.5, HEADS, HDIM, LAYERS, scope="frame")
    g = torch.Generator(device="cpu").manual_seed(1234)
    x_host = torch.randn((F8, N_TOK, CH), generator=g).bfloat16().pin_memory()
    conf_host = torch.rand((1, F8 * GRID * GRID), generator=g).bfloat16().pin_memory()
    qkv_host = torch.randn((F8 * N_TOK, 3, HEADS, HDIM), generator=g).bfloat16().pin_memory()
    out_host = torch.empty((F8, N_TOK, CH), dtype=torch.bfloat16).pin_memory()
    x, conf, qkv_buf = x_host.to(dev), conf_host.to(dev), qkv_host.to(dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)  # > 126 MB L2
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    scene = StaticScene(F8, CH, START, GRID, GRID, WIN, WIN, 0.5, HEADS, HDIM, LAYERS, "frame", torch.bfloat16, dev).capture()
    for _ in range(3):
        scene.run(x_host, conf_host, qkv_host)
    torch.cuda.synchronize()
    graph_ev = []
    for _ in range(steps):
        flush.fill_(1)  # L2 flush between timed iterations (outside the per-step events)
        s, e = ev(), ev()
        s.record()
        scene.run()
        e.record()
        graph_ev.append((s, e))
    torch.cuda.synchronize()
    graph_ms = sum(s.elapsed_time(e) for s, e in graph_ev) / steps
    # device time per kernel family: each family's launches of one scene captured into a graph of their own
    plan = chain.build_plan(conf)
    P = plan.total
    qkv_p, bias_p = qkv_buf[:P], plan.perkey_bias(torch.bfloat16)
    attn_p = attn_fn(qkv_p, plan.cu_seqlens(1), plan.max_seqlen, perkey_bias=bias_p, softmax_scale=chain.scale).reshape(P, CH)
    n_f = sum(1 for k in LAYERS if k != "global")
    n_g = len(LAYERS) - n_f
    families = {
        "frame": (n_f, lambda: attn_fn(qkv_p, plan.cu_seqlens(1), plan.max_seqlen, perkey_bias=bias_p, softmax_scale=chain.scale)),
        "global": (n_g, lambda: attn_fn(qkv_p, plan.cu_seqlens(F8), P, perkey_bias=bias_p, softmax_scale=chain.scale)),
        "merge": (len(LAYERS), lambda: plan.merge(x)),
        "unmerge": (len(LAYERS), lambda: plan.split(attn_p)),
    }
    family_ms = {}
    for name, (count, fn) in families.items():
        fn()
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for _ in range(count):
                fn()
        gr.replay()
        acc, reps = 0.0, max(3, steps // 4)
        for _ in range(reps):
            flush.fill_(1)
            s, e = ev(), ev()
            s.record()
            gr.replay()
            e.record()
            torch.cuda.synchronize()
            acc += s.elapsed_time(e)
        family_ms[name] = acc / reps
        del gr
    # end to end: every scene's inputs start in pinned host memory and its result ends there; the copies of scene k+1 /
    # k-1 run on a side stream while scene k computes (StaticScene.stage / run_staged), as a serving loop would
    h2d = (x_host.numel() + conf_host.numel() + qkv_host.numel()) * 2
    d2h = out_host.numel() * 2
    for _ in range(2):
        scene.stage(x_host, conf_host, qkv_host)
    for _ in range(2):
        scene.run_staged(out_host)
    scene.drain()
    torch.cuda.synchronize()
    s, e = ev(), ev()
    s.record()
    scene.stage(x_host, conf_host, qkv_host)
    for k in range(steps):
        if k + 1 < steps:
            scene.stage(x_host, conf_host, qkv_host)
        scene.run_staged(out_host)
    torch.cuda.current_stream().wait_stream(scene._copy_stream)
    e.record()
    torch.cuda.synchronize()
    e2e_ms = s.elapsed_time(e) / steps
    if _lib.device_status(clear=False) != 0:
        raise RuntimeError("attention kernel raised the device status word in the 8-frame scene")
    seg = (plan.offset[1:] - plan.offset[:-1]).tolist()
    flops_frame, flops_global = sum(4.0 * L * L * HDIM * HEADS for L in seg), 4.0 * P * P * HDIM * HEADS
    attn_ms = family_ms["frame"] + family_ms["global"]
    achieved = (n_f * flops_frame + n_g * flops_global) / (attn_ms * 1e-3) / 1e12
    merge_bytes = F8 * N_TOK * CH * 2 + P * CH * 2 + F8 * N_WIN + (F8 + 1) * 4
    unmerge_bytes = P * CH * 2 + F8 * N_TOK * 8 + F8 * N_TOK * CH * 2
    return {
        "metric": "come_vggt_hot_path_ms_per_scene_8f", "value": graph_ms, "unit": UNIT, "steps": steps,
        "workload": workload_name(F8), "merged_tokens": P, "launch": "one CUDA graph per scene (StaticScene): worst-case grids, no device-to-host read",
        "l2": "flushed between timed steps (256 MB write)",
        "e2e": {"value": e2e_ms, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "scene_ms_by_family": family_ms,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s", "frac": achieved / pk["tflops"],
                     "peak_source": pk["source"] + " burst cuBLAS bf16",
                     "frame_tflops": n_f * flops_frame / (family_ms["frame"] * 1e-3) / 1e12,
                     "global_tflops": n_g * flops_global / (family_ms["global"] * 1e-3) / 1e12,
                     "timing": "CUDA events around a graph of one scene's 24 frame / 24 global launches (device time)"},
        "merge_gbs": merge_bytes * len(LAYERS) / (family_ms["merge"] * 1e-3) / 1e9,
        "unmerge_gbs": unmerge_bytes * len(LAYERS) / (family_ms["unmerge"] * 1e-3) / 1e9,
        "gpu_launches": scene.launches_per_scene * steps,
    }


def run_batch(args):
    """256 independent scenes of 4 frames, merge ratio per frame ~U(0.25, 0.75) (ragged packed lengths), sharded by
    scene over the ranks with no inter-GPU traffic; each rank runs its scenes as ONE captured graph."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    from come_b200 import _lib
    from come_b200.dist import shard_range
    from come_b200.static_scene import StaticScene
    total_scenes, fps = 256, 4
    lo, hi = shard_range(total_scenes, world, rank)
    n_sc = hi - lo
    scene = StaticScene(n_sc * fps, CH, START, GRID, GRID, WIN, WIN, 0.5, HEADS, HDIM, LAYERS, "frame", torch.bfloat16, dev,
                        frames_per_scene=fps, per_frame_ratios=True)
    gl = torch.Generator(device=dev).manual_seed(77 + rank)
    scene.x.copy_(torch.randn(scene.x.shape, device=dev, generator=gl).bfloat16())
    scene.conf.copy_(torch.rand(scene.conf.shape, device=dev, generator=gl).bfloat16())
    for i in range(0, scene.qkv.shape[0], 1 << 18):  # fill in slices: the fp32 draw of the whole buffer would be 17 GB
        blk = scene.qkv[i:i + (1 << 18)]
        blk.copy_(torch.randn(blk.shape, device=dev, generator=gl).bfloat16())
    scene.ratios.copy_(torch.rand(n_sc * fps, device=dev, generator=gl) * 0.5 + 0.25)
    scene.capture()
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(min(args.warmup, 3)):
        scene.run()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    s, e = ev(), ev()
    s.record()
    for _ in range(args.steps):
        scene.run()
    e.record()
    barrier()
    ms = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if rank == 0 else None
    assert _lib.device_status(clear=False) == 0
    if rank == 0:
        per_step = ms.item() / args.steps
        off = scene.offsets.cpu().numpy().astype(np.int64)
        seg = np.diff(off)
        scene_len = np.diff(off[::fps])
        flops = 24 * (4.0 * HDIM * HEADS) * (float((seg ** 2).sum()) + float((scene_len ** 2).sum())) * (total_scenes / n_sc)
        line = {
            "metric": "come_vggt_hot_path_scenes_per_s_256x4f", "value": total_scenes / (per_step * 1e-3), "unit": "scenes/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded)",
            "config": {"workload": "256 independent scenes x 4 frames x 518x518 (VGGT-1B shapes, 48 attention layers each = merge + "
                                   "biased varlen attention + unmerge), merge ratio per frame ~U(0.25,0.75); projections/MLP GEMMs excluded",
                       "parallelism": f"{n_sc} scenes per GPU x {world}, no inter-GPU traffic; one CUDA graph per rank and step",
                       "packed_rows_rank0": int(off[-1]), "min_max_frame_len": [int(seg.min()), int(seg.max())],
                       "l2": "inputs larger than L2 (GBs per rank)"},
            "attention_tflops_aggregate": flops / (per_step * 1e-3) / 1e12,
            "gpu_launches": scene.launches_per_scene * args.steps, "clocks": clocks,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_model100(args):
    """The alternating-attention stack (48 blocks with their GEMMs) on ONE scene of 100 frames sharded by frame over the
    ranks (`ShardedFusedAggregator`): everything row-wise and the frame blocks are local, a global block all-gathers the
    prepared K/V rows of the packed tokens.  Strong scaling: the scene is fixed."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    from come_b200 import _lib
    from come_b200.fused import ShardedFusedAggregator
    from come_b200.token_merger import select_windows
    from come_b200.vggt_arch import AggregatorCore
    frames = 100
    pk = peaks()
    core = AggregatorCore(depth=24).to(dev).bfloat16()  # seeded: the same weights on every rank
    model = ShardedFusedAggregator(core, frames, world, rank)
    layout = _lib.Layout.two_d(START, GRID, GRID, WIN, WIN)
    g = torch.Generator(device="cpu").manual_seed(4321)
    conf = torch.rand((1, frames * GRID * GRID), generator=g).bfloat16().to(dev)  # replicated
    n_local = model.f_hi - model.f_lo
    gl = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn((1, n_local, N_TOK, CH), device=dev, generator=gl).bfloat16()
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    plans = []

    def step():
        mask = select_windows(conf, 1, frames, GRID, GRID, WIN, WIN, 0.5, "pairwise-rank", "frame")
        gp, lp = model.build_plans(mask, layout)
        plans[:] = [gp, lp]
        with torch.no_grad():
            out, _ = model(x, gp, lp)
        return out

    for _ in range(min(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    s, e = ev(), ev()
    s.record()
    for _ in range(args.steps):
        step()
    e.record()
    barrier()
    ms = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if rank == 0 else None
    assert _lib.device_status(clear=False) == 0
    if rank == 0:
        per_scene = ms.item() / args.steps
        gp = plans[0]
        P = gp.total
        seg = (gp.offset[1:] - gp.offset[:-1]).tolist()
        attn_flops = 24 * (sum(4.0 * L * L * HDIM * HEADS for L in seg) + 4.0 * P * P * HDIM * HEADS)
        gemm_flops = 48 * 2.0 * P * CH * CH * 12
        kv_bytes = P * 2 * HEADS * HDIM * 2
        print(json.dumps({
            "metric": "come_vggt_aggregator_ms_per_scene_100f", "value": per_scene, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_scene, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded)",
            "config": {"workload": "VGGT-1B-shaped alternating-attention stack (48 blocks incl. qkv / proj / MLP GEMMs, seeded "
                                   "random bf16 weights) on one scene of 100 frames x 518x518, 3x3 windows at 50 % per frame",
                       "merged_tokens": P, "frames_per_s": frames / per_scene * 1e3,
                       "parallelism": f"frames sharded over {world} GPU(s); global blocks all-gather {kv_bytes / 1e6:.0f} MB of "
                                      f"prepared K/V per block over NCCL",
                       "l2": "inputs larger than L2"},
            "tflop_per_scene": {"attention": attn_flops / 1e12, "gemm": gemm_flops / 1e12},
            "tflops_aggregate": (attn_flops + gemm_flops) / (per_scene * 1e-3) / 1e12,
            "frac_of_bf16_peak_per_gpu": (attn_flops + gemm_flops) / (per_scene * 1e-3) / 1e12 / world / pk["tflops"],
            "clocks": clocks,
        }))
    if world > 1:
        dist.destroy_process_group()


def micro(torch, dev, pk):
    """Kernel-level numbers on inputs larger than L2: 100-frame fp32 merge / unmerge (GB/s) and the 64-segment
    ragged biased-attention sweep (TFLOP/s)."""
    from come_b200 import _lib
    from come_b200.flash_attn import flash_attn_varlen_qkvpacked_func_w_perkey_bias as attn_fn
    from come_b200.token_merger import MergePlan
    res = {}
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731

    def timeit(fn, iters, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        s, e = ev(), ev()
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / iters

    frames = 100
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn((frames, N_TOK, CH), device=dev, generator=g)
    mask = torch.rand((frames, N_WIN), device=dev, generator=g) < 0.5
    plan = MergePlan(mask, _lib.Layout.two_d(START, GRID, GRID, WIN, WIN))
    P = plan.total
    merged = plan.merge(x)
    mb = frames * N_TOK * CH * 4 + P * CH * 4 + frames * N_WIN + (frames + 1) * 4
    ub = P * CH * 4 + frames * N_TOK * 8 + frames * N_TOK * CH * 4
    tm = timeit(lambda: plan.merge(x), 20)
    tu = timeit(lambda: plan.split(merged), 20)
    tp = timeit(lambda: MergePlan(mask, plan.layout), 10)
    res["merge_fp32_100f"] = {"GB/s": mb / tm / 1e6, "ms": tm, "bytes": mb, "frac_of_hbm_peak": mb / tm / 1e6 / pk["hbm_gbs"]}
    res["unmerge_fp32_100f"] = {"GB/s": ub / tu / 1e6, "ms": tu, "bytes": ub, "frac_of_hbm_peak": ub / tu / 1e6 / pk["hbm_gbs"]}
    res["plan_100f"] = {"ms": tp, "note": "select excluded; 2 kernels + one host read"}
    del x, merged

    rng = np.random.default_rng(0)
    lens = [1374 - 8 * int(k) for k in rng.integers(0, 73, size=64)]
    Pt = sum(lens)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=dev)
    qkv = torch.randn((Pt, 3, HEADS, HDIM), device=dev, generator=g).bfloat16()
    cnt = torch.where(torch.rand(Pt, device=dev, generator=g) < 0.1, 9.0, 1.0)
    bias = cnt.log().bfloat16()
    flops = sum(4.0 * L * L * HDIM * HEADS for L in lens)
    ta = timeit(lambda: attn_fn(qkv, cu, max(lens), perkey_bias=bias, softmax_scale=HDIM ** -0.5), 10)
    res["attn_bias_sweep_64seg"] = {"TFLOP/s": flops / ta / 1e9, "ms": ta, "gflop": flops / 1e9,
                                    "frac_of_bf16_peak": flops / ta / 1e9 / pk["tflops"]}
    if _lib.device_status(clear=False) != 0:
        raise RuntimeError("attention kernel raised the device status word in the kernel sweep")
    return res


def run_only(args):
    """One kernel family on one size, a few launches: the command the ncu captures under profiles/ were made with."""
    import torch
    from come_b200 import _lib
    from come_b200.flash_attn import flash_attn_varlen_qkvpacked_func_w_perkey_bias as attn_fn
    from come_b200.token_merger import MergePlan
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    out = {"only": args.only}
    if args.only in ("merge", "unmerge", "merge_ln", "unmerge_res"):
        dt = {"f32": torch.float32, "bf16": torch.bfloat16}[args.dtype]
        x = torch.randn((args.frames, N_TOK, CH), device=dev, generator=g).to(dt)
        mask = torch.rand((args.frames, N_WIN), device=dev, generator=g) < 0.5
        plan = MergePlan(mask, _lib.Layout.two_d(START, GRID, GRID, WIN, WIN))
        merged = plan.merge(x)
        es = x.element_size()
        if args.only == "merge":
            fn, nbytes = (lambda: plan.merge(x)), args.frames * N_TOK * CH * es + plan.total * CH * es + args.frames * N_WIN + (args.frames + 1) * 4
        elif args.only == "merge_ln":  # LayerNorm over the channels fused into the merge: same traffic + gamma / beta
            ln = torch.nn.LayerNorm(CH, eps=1e-6).to(dev).to(dt)
            fn, nbytes = (lambda: plan.merge_layernorm(x, ln)), args.frames * N_TOK * CH * es + plan.total * CH * es + args.frames * N_WIN + (args.frames + 1) * 4 + 2 * CH * es
        elif args.only == "unmerge_res":  # unmerge + LayerScale + residual add: one more dense read
            gamma = torch.rand(CH, device=dev, generator=g).to(dt)
            res = x.reshape(-1, CH)
            fn, nbytes = (lambda: plan.split_add(merged, res, gamma)), plan.total * CH * es + args.frames * N_TOK * 8 + 2 * args.frames * N_TOK * CH * es + CH * es
        else:
            fn, nbytes = (lambda: plan.split(merged)), plan.total * CH * es + args.frames * N_TOK * 8 + args.frames * N_TOK * CH * es
        out.update(frames=args.frames, dtype=args.dtype, bytes=nbytes)
    elif args.only == "direct":
        # The complete replacement of block.attn.forward in the reference's per-layer mode, 48 layers of one scene:
        # merge -> qkv GEMM -> q/k LayerNorm + RoPE + bias -> biased attention -> proj GEMM -> unmerge (GEMMs = cuBLAS).
        from come_b200.direct import DirectAttention

        class Attn(torch.nn.Module):
            def __init__(self):
                super().__init__()
                self.num_heads, self.head_dim, self.scale = HEADS, HDIM, HDIM ** -0.5
                self.qkv, self.proj = torch.nn.Linear(CH, 3 * CH), torch.nn.Linear(CH, CH)
                self.q_norm, self.k_norm = torch.nn.LayerNorm(HDIM), torch.nn.LayerNorm(HDIM)
                self.rope = type("Rope", (), {"base_frequency": 100.0})()

        torch.manual_seed(0)
        frames = args.frames if args.frames != 100 else 8
        mask = torch.rand((frames, N_WIN), device=dev, generator=g) < 0.5
        plan = MergePlan(mask, _lib.Layout.two_d(START, GRID, GRID, WIN, WIN))
        layers = [DirectAttention(Attn().to(dev), is_global=bool(i % 2)).eval() for i in range(48)]
        x = torch.randn((frames, N_TOK, CH), device=dev, generator=g).bfloat16()

        def scene():
            y = x
            with torch.no_grad():
                for layer in layers:
                    y = layer(y.reshape(1, frames * N_TOK, CH) if layer.is_global else y.reshape(frames, N_TOK, CH), plan, frames)
            return y

        scene()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            scene()
        fn = graph.replay
        gemm_flops = 48 * 2.0 * plan.total * CH * 4 * CH
        out.update(frames=frames, tokens=plan.total, layers=48, launch="CUDA graph of 48 layers",
                   flops=gemm_flops + sum(4.0 * L * L * HDIM * HEADS for L in ([plan.total] * 24 + [plan.total / frames] * 24 * frames)))
    elif args.only == "residual_ln":
        # LayerScale + residual add + LayerNorm on the packed rows of `frames` half-merged frames: x and the branch are
        # read once, the updated stream and its normalised copy written once
        from come_b200.block import residual_layernorm
        dt = {"f32": torch.float32, "bf16": torch.bfloat16}[args.dtype]
        rows = args.frames * (N_TOK - 8 * (N_WIN // 2))
        x = torch.randn((rows, CH), device=dev, generator=g).to(dt)
        br = torch.randn((rows, CH), device=dev, generator=g).to(dt)
        gamma = torch.rand(CH, device=dev, generator=g).to(dt)
        ln = torch.nn.LayerNorm(CH, eps=1e-6).to(dev).to(dt)
        fn = lambda: residual_layernorm(x, br, gamma, ln)  # noqa: E731
        out.update(frames=args.frames, tokens=rows, dtype=args.dtype, bytes=4 * rows * CH * x.element_size() + 3 * CH * x.element_size())
    elif args.only == "cross":
        # Attention of `--rows` query rows to `--tokens` keys that do not contain them (what a rank of the sharded scene runs
        # on the gathered rows of the other ranks): `--balanced 0` one launch, `--balanced 1` the launch cut by
        # plan_tail_split (the last query blocks with their keys in shares).
        from come_b200 import flash_attn_fwd_cuda as fa
        q = torch.randn((args.rows, HEADS, HDIM), device=dev, generator=g).bfloat16()
        kv = torch.randn((args.tokens, 2, HEADS, HDIM), device=dev, generator=g).bfloat16()
        bias = torch.where(torch.rand(args.tokens, device=dev, generator=g) < 0.1, 9.0, 1.0).log().bfloat16()
        call = fa.cross_fwd_balanced if args.balanced else fa.cross_fwd
        fn = lambda: call(q, kv[:, 0], kv[:, 1], bias, HDIM ** -0.5)  # noqa: E731
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        out.update(rows=args.rows, keys=args.tokens, flops=4.0 * args.rows * args.tokens * HDIM * HEADS,
                   work_items=-(-args.rows // 384) * HEADS, plan=list(fa.plan_tail_split(args.rows, HEADS, args.tokens, sms)) if args.balanced else None)
    elif args.only == "prepare":
        # q/k LayerNorm + 2-D rotary embedding + log(count) bias on the packed rows of `frames` half-merged frames
        from come_b200.qkv import RotaryPositionEmbedding2D, prepare_packed_self_attention_qkv
        mask = torch.rand((args.frames, N_WIN), device=dev, generator=g) < 0.5
        plan = MergePlan(mask, _lib.Layout.two_d(START, GRID, GRID, WIN, WIN))
        Pt = plan.total
        qkv = torch.randn((Pt, 3, HEADS, HDIM), device=dev, generator=g).bfloat16()
        ln_q = torch.nn.LayerNorm(HDIM).to(dev).bfloat16()
        ln_k = torch.nn.LayerNorm(HDIM).to(dev).bfloat16()
        rope, pos = RotaryPositionEmbedding2D(100.0), plan.positions()
        fn = lambda: prepare_packed_self_attention_qkv(qkv, ln_q, ln_k, rope, pos, torch.bfloat16, weight=plan.weight)  # noqa: E731
        # q and k read and written once, positions, counts in, bias out
        out.update(frames=args.frames, tokens=Pt, bytes=Pt * (4 * HEADS * HDIM * 2 + 16 + 4 + 2))
    else:
        if args.segments == 1:
            lens = [args.tokens]
        else:
            rng = np.random.default_rng(0)
            lens = [1374 - 8 * int(k) for k in rng.integers(0, 73, size=args.segments)]
        Pt = sum(lens)
        cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=dev)
        qkv = torch.randn((Pt, 3, HEADS, HDIM), device=dev, generator=g).bfloat16()
        bias = torch.where(torch.rand(Pt, device=dev, generator=g) < 0.1, 9.0, 1.0).log().bfloat16()
        fn = lambda: attn_fn(qkv, cu, max(lens), perkey_bias=bias, softmax_scale=HDIM ** -0.5)  # noqa: E731
        out.update(segments=len(lens), tokens=Pt, flops=sum(4.0 * L * L * HDIM * HEADS for L in lens))
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    if args.graph and args.only != "direct":
        # device time without the host's per-call cost: `iters` launches captured into one graph, replayed once
        eager, graph = fn, torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(args.iters):
                eager()
        graph.replay()
        torch.cuda.synchronize()
        s, e = ev(), ev()
        s.record()
        graph.replay()
        e.record()
        torch.cuda.synchronize()
        out["launch"] = f"{args.iters} launches in one CUDA graph"
        out["ms"] = s.elapsed_time(e) / args.iters
        key = "GB/s" if "bytes" in out else "TFLOP/s"
        out[key] = (out["bytes"] / out["ms"] / 1e6) if "bytes" in out else (out["flops"] / out["ms"] / 1e9)
        assert _lib.device_status(clear=False) == 0
        print(json.dumps(out))
        return
    s, e = ev(), ev()
    s.record()
    for _ in range(args.iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / args.iters
    out["ms"] = ms
    if "bytes" in out:
        out["GB/s"] = out["bytes"] / ms / 1e6
    else:
        out["TFLOP/s"] = out["flops"] / ms / 1e9
    assert _lib.device_status(clear=False) == 0
    print(json.dumps(out))


def aggregator_measure(S, depth, iters, arms_wanted="", report=True, B=1, ragged=False):
    """End-to-end driver in the form of the reference's benchmark (``src/bench.py:13-46``): the unmerged model and the
    accelerated model are run over the same synthetic scenes inside ``Timer.range`` and the timer's table is printed.
    The model is the alternating-attention stack of a VGGT-1B-shaped aggregator with seeded random weights in bf16
    (24 frame + 24 global blocks, width 1024, 16 heads, q/k norm, rotary embedding, LayerScale, MLP ratio 4); the patch
    encoder and the heads are outside.  A scene's work in the accelerated arm: confidence head (seeded 2-layer MLP) ->
    window selection -> merge plan -> merge -> 48 blocks on packed tokens -> unmerge of the retained layers.
    GEMMs are PyTorch's (cuBLAS); everything else on the packed tokens is this library's kernels.
    ``B`` independent scenes per call (frame blocks attend inside a frame, global blocks inside a scene); ``ragged``:
    every frame gets its own merge ratio ~U(0.25, 0.75), so the packed lengths differ from frame to frame."""
    import torch
    from come_b200 import _lib
    from come_b200.fused import CapturedForward, FusedAggregator
    from come_b200.timer import Timer
    from come_b200.token_merger import MergePlan, select_windows
    from come_b200.vggt_arch import AggregatorCore
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    core = AggregatorCore(depth=depth).to(dev).bfloat16()
    model = FusedAggregator(core)
    captured = CapturedForward(model)
    torch.manual_seed(0)
    head = torch.nn.Sequential(torch.nn.Linear(CH, 128), torch.nn.GELU(), torch.nn.Linear(128, 1)).to(dev).bfloat16().eval()
    layout = _lib.Layout.two_d(START, GRID, GRID, WIN, WIN)
    g = torch.Generator(device=dev).manual_seed(0)
    scenes = [torch.randn((B, S, N_TOK, CH), device=dev, generator=g).bfloat16() for _ in range(iters)]
    ratios = (0.25 + 0.5 * torch.rand(B * S, device=dev, generator=g)) if ragged else None

    def plan_of(tokens):
        conf = head(tokens[:, :, START:, :]).reshape(B, S * GRID * GRID)
        if ragged:
            mask = select_windows(conf, B, S, GRID, GRID, WIN, WIN, ratios, "pairwise-rank", "frame")
        else:
            mask = select_windows(conf, B, S, GRID, GRID, WIN, WIN, 0.5, "pairwise-rank", "batch")
        return MergePlan(mask, layout)

    arms = {
        "Reference Model": lambda t: model.forward_unmerged(t),
        "Accelerated Model": lambda t: model(t, plan_of(t)),
        "Accelerated Model (CUDA graph)": lambda t: captured(t, plan_of(t)),
    }
    if arms_wanted:
        wanted = {"reference": "Reference Model", "accelerated": "Accelerated Model", "graph": "Accelerated Model (CUDA graph)"}
        arms = {wanted[a]: arms[wanted[a]] for a in arms_wanted.split(",")}
    Timer.reset()
    with torch.no_grad():
        for name, fn in arms.items():
            Timer.activate(False)
            for t in scenes[:2]:  # warm-up (and graph capture) outside the table
                fn(t)
            torch.cuda.synchronize()
            Timer.activate()
            for t in scenes:
                with Timer.range(name):
                    fn(t)
            torch.cuda.synchronize()
        packed = [plan_of(t).total for t in scenes]
    Timer.activate(False)
    entries = {e.name: e for e in Timer.results()}
    if report:
        print(Timer.report(), file=sys.stderr)
    Timer.reset()
    assert _lib.device_status(clear=False) == 0
    P = float(np.mean(packed)) / B  # per scene
    blocks = 2 * depth
    gemm = lambda rows: blocks * 2.0 * rows * CH * CH * 12  # qkv 3, proj 1, fc1 4, fc2 4  # noqa: E731
    attn = lambda rows: depth * 4.0 * HDIM * HEADS * (rows * rows + S * (rows / S) ** 2)  # noqa: E731
    return {
        "only": "aggregator", "frames": S, "scenes_per_call": B, "merge_ratio": "per frame ~U(0.25, 0.75)" if ragged else 0.5,
        "blocks": blocks, "calls": len(scenes), "dtype": "bf16",
        "packed_tokens_mean": P, "dense_tokens": S * N_TOK, "graphs_captured": len(captured._graphs),
        "ms_per_scene": {k: round(v.P50 / B, 3) for k, v in entries.items()},
        "scenes_per_s": {k: round(B / v.P50 * 1e3, 1) for k, v in entries.items()},
        "speedup_vs_unmerged": ({k: round(entries["Reference Model"].P50 / v.P50, 3) for k, v in entries.items()}
                                if "Reference Model" in entries else None),
        "tflop_per_scene": {"unmerged": round((gemm(S * N_TOK) + attn(S * N_TOK)) / 1e12, 2),
                            "merged": round((gemm(P) + attn(P)) / 1e12, 2)},
        "timer": "CUDA events around each scene (src/utility/timer.py form), median over the scenes",
    }


def model_measure(S, iters, arms_wanted="", report=True):
    """The whole accelerated model in the form of the reference's benchmark (``src/bench.py:13-46``): images -> patch
    encoder (ViT-L/14-reg shape, 24 blocks; the merge context is built after block 14 and blocks 15..23 run on the merged
    tokens, ``src/accelerate/vggt/fused.py:40-94``) -> aggregator (24 + 24 blocks), seeded random bf16 weights, against
    the same weights with nothing merged.  The prediction heads are outside.  GEMMs and the patch convolution are
    PyTorch's; everything else on the tokens is this library's kernels."""
    import torch
    from come_b200 import _lib
    from come_b200.fused import FusedModel
    from come_b200.timer import Timer
    from come_b200.vggt_arch import AggregatorCore, ConfidenceHead, PatchEncoderCore
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    enc = PatchEncoderCore().to(dev).bfloat16()
    core = AggregatorCore(depth=24).to(dev).bfloat16()
    head = ConfidenceHead().to(dev).bfloat16()
    model = FusedModel(enc, core, head, encoder_layer=14, threshold=0.5).eval()
    g = torch.Generator(device=dev).manual_seed(0)
    scenes = [torch.rand((1, S, 3, 518, 518), device=dev, generator=g).bfloat16() for _ in range(iters)]
    arms = {"Reference Model": model.forward_unmerged, "Accelerated Model": model}
    if arms_wanted:
        wanted = {"reference": "Reference Model", "accelerated": "Accelerated Model"}
        arms = {wanted[a]: arms[wanted[a]] for a in arms_wanted.split(",") if a in wanted}
    Timer.reset()
    packed = []
    with torch.no_grad():
        for name, fn in arms.items():
            Timer.activate(False)
            for t in scenes[:2]:
                fn(t)
            torch.cuda.synchronize()
            Timer.activate()
            for i, t in enumerate(scenes):
                with torch.cuda.nvtx.range(f"{'Ref' if name.startswith('Ref') else 'Acc'}:sample_{i}"), \
                        torch.cuda.nvtx.range("inference"), Timer.range(name):
                    fn(t)
                if name == "Accelerated Model":
                    packed.append(model.last_plan.total)
            torch.cuda.synchronize()
    Timer.activate(False)
    entries = {e.name: e for e in Timer.results()}
    if report:
        print(Timer.report(), file=sys.stderr)
    Timer.reset()
    assert _lib.device_status(clear=False) == 0
    return {
        "only": "model", "frames": S, "dtype": "bf16", "calls": len(scenes), "encoder": "ViT-L/14-reg shape, 24 blocks, merge context after block 14",
        "aggregator": "24 frame + 24 global blocks", "heads": "not included", "packed_tokens_mean": float(np.mean(packed)) if packed else None,
        "dense_tokens": S * N_TOK,
        "ms_per_scene": {k: round(v.P50, 3) for k, v in entries.items()},
        "speedup_vs_unmerged": ({k: round(entries["Reference Model"].P50 / v.P50, 3) for k, v in entries.items()}
                                if "Reference Model" in entries else None),
        "timer": "CUDA events around each scene (src/utility/timer.py form), median over the scenes; launched from Python",
    }


def run_aggregator(args):
    S = 8 if args.frames == 100 else args.frames  # 100 is the flag's default, meant for the merge kernels
    print(json.dumps(aggregator_measure(S, args.depth, args.iters, args.arms, B=args.scenes, ragged=args.ragged)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", choices=["attn", "cross", "merge", "unmerge", "merge_ln", "unmerge_res", "prepare", "residual_ln", "direct", "aggregator", "model"],
                    help="run one kernel family on one size and exit; aggregator = the alternating-attention stack, merged against "
                         "unmerged; model = the same comparison from the images on (patch encoder with its merge after block 14 + aggregator)")
    ap.add_argument("--depth", type=int, default=24, help="--only aggregator: frame/global block pairs")
    ap.add_argument("--scenes", type=int, default=1, help="--only aggregator: independent scenes per call")
    ap.add_argument("--ragged", action="store_true", help="--only aggregator: per-frame merge ratios ~U(0.25, 0.75)")
    ap.add_argument("--arms", default="", help="--only aggregator: comma list of reference, accelerated, graph (default all)")
    ap.add_argument("--frames", type=int, default=100, help="--only merge/unmerge: frames")
    ap.add_argument("--dtype", default="f32", choices=["f32", "bf16"], help="--only merge/unmerge: element type")
    ap.add_argument("--tokens", type=int, default=6384, help="--only attn with --segments 1: segment length")
    ap.add_argument("--segments", type=int, default=1, help="--only attn: 1 = one segment, else ragged 1374-8k sweep")
    ap.add_argument("--rows", type=int, default=10534, help="--only cross: query rows (the keys are --tokens)")
    ap.add_argument("--balanced", type=int, default=1, help="--only cross: 1 = launch cut by plan_tail_split, 0 = one launch")
    ap.add_argument("--iters", type=int, default=3, help="--only: timed launches")
    ap.add_argument("--graph", action="store_true", help="--only: time the launches inside one CUDA graph (no host cost)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="come_b200", choices=["come_b200", "reference"])
    ap.add_argument("--workload", default="frames100", choices=["frames100", "frames8", "batch256x4", "model100"],
                    help="frames100 (default): ONE 100-frame scene whose frames are sharded over the GPUs, global attention over "
                         "all-gathered K/V; frames8: the same for an 8-frame scene (quick runs); batch256x4: 256 independent "
                         "4-frame scenes with per-frame merge ratios ~U(0.25,0.75), sharded by scene, reported as scenes/s; model100: the "
                         "100-frame scene through the whole alternating-attention stack (with its GEMMs), sharded by frame")
    ap.add_argument("--transport", default="peer", choices=["peer", "nccl"],
                    help="transport of the hidden K/V exchange at N > 1: copy engines over peer-mapped windows, or an NCCL all-gather")
    ap.add_argument("--pulls-first", default="off", choices=["on", "off"],
                    help="peer transport, hidden exchange: launch the attention to the local keys only once the pulls are runnable")
    ap.add_argument("--overlap", default="auto", choices=["auto", "on", "off"],
                    help="N > 1: hide the K/V all-gather of a global layer behind attention to the local keys (on), keep it in line "
                         "(off: the sharded result is then bit-identical to one GPU), or decide from a model of the layer (auto: "
                         "hidden on 2 to 4 GPUs, in line on 8 for the 100-frame scene)")
    ap.add_argument("--no-scene8", action="store_true", help="skip the 8-frame scene (extra key scene8)")
    ap.add_argument("--no-micro", action="store_true", help="skip the kernel-level sweep")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    args = ap.parse_args()
    if args.only == "model":
        print(json.dumps(model_measure(8 if args.frames == 100 else args.frames, args.iters, args.arms)))
    elif args.only == "aggregator":
        run_aggregator(args)
    elif args.only:
        run_only(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.workload == "batch256x4":
        args.warmup = max(args.warmup, 3)
        run_batch(args)
    elif args.workload == "model100":
        run_model100(args)
    else:
        run_frames(args)


if __name__ == "__main__":
    main()
