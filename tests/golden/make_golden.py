"""Generate the golden fixtures in this directory by running the REFERENCE implementation on CPU.

Usage (only where a checkout of the reference is available)::

    python tests/golden/make_golden.py --reference /path/to/CoMe

The reference's PyTorch fallback path (``CUDAExtension.disable()``) is imported unmodified; four modules that
are not installed here (``hydra``, ``omegaconf``, ``pypose`` and the compiled ``src.cuda_extension``) are
replaced by empty stubs.  Inputs are drawn from ``numpy.random.default_rng(seed)`` so that the tests can
regenerate them without the reference; outputs are stored in ``*.npz`` files (integer outputs in full, large
float outputs as per-row float64 sums plus a strided sample of complete rows).

The tests never import the reference; they only read the ``*.npz`` files written here.
"""
from __future__ import annotations

import argparse
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from reference_cases import RANDOM_CONFIGS_1D, RANDOM_CONFIGS_2D, ATTENTION_CASES  # noqa: E402
from golden_inputs import (  # noqa: E402
    merge1d_inputs, merge2d_inputs, select_inputs, SELECT_CASES, attention_inputs, EXTRA_ATTENTION_CASES,
    cfg1_inputs, summarize_rows, PREPARE_CASES, PREPARE_EPS, PREPARE_MAX_POSITION, prepare_inputs, POSITION_CASES,
    position_mask, LN_MERGE_CASES, LN_MERGE_EPS, ln_merge_inputs, ln_merge_tolerance, BLOCK_CASES, BLOCK_TOLERANCE,
    block_inputs, SUFFIX_CASES, suffix_inputs,
)


def import_reference(root: str):
    def stub(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    stub("hydra")
    sys.modules["hydra"].utils = stub("hydra.utils", instantiate=lambda *a, **k: None)
    stub("omegaconf", DictConfig=dict, OmegaConf=object)
    stub("pypose")
    sys.path.insert(0, root)
    import src  # noqa: F401  (the reference's real top-level package)

    ce = types.ModuleType("src.cuda_extension")
    ce.__path__ = []
    ce.co_me_cuext = types.ModuleType("co_me_cuext")
    ce.flash_attn_varlen_qkvpacked_func = None
    ce.flash_attn_varlen_qkvpacked_func_w_perkey_bias = None
    ce.infer_flash_attn_varlen_max_seqlen = None
    sys.modules["src.cuda_extension"] = ce
    fa = types.ModuleType("src.cuda_extension.flash_attn")
    fa.infer_flash_attn_varlen_max_seqlen = None
    sys.modules["src.cuda_extension.flash_attn"] = fa

    from src.accelerate.token_merger import co_me, co_me_2d
    from src.utility.feature import CUDAExtension
    import test.auto_test.test_flex_attention_bias as attn_test

    return co_me, co_me_2d, CUDAExtension, attn_test


def import_file(root: str, rel: str, name: str):
    """A single reference source file as a module (its package __init__ pulls in unrelated model code)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location(name, os.path.join(root, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference project")
    args = ap.parse_args()
    import torch

    co_me, co_me_2d, CUDAExtension, attn_test = import_reference(args.reference)
    import oracle.come_oracle as orc

    def t(x):
        return torch.from_numpy(np.ascontiguousarray(x))

    def close(ours, ref, kind="f32"):
        """Features: the reference's vectorised CPU reduction may differ from the left-to-right sum by one
        rounding (observed <= 1.2e-7 relative); indices and counts are compared exactly elsewhere."""
        tol = 1e-6 if kind == "f32" else 8e-3
        return np.allclose(ours, ref, rtol=tol, atol=tol)

    # ---- 1-D merge / split -----------------------------------------------------------------------------
    store = {}
    for i, cfg in enumerate(RANDOM_CONFIGS_1D):
        for kind in ("f32", "bf16"):
            tokens, mask = merge1d_inputs(i, cfg, kind)
            B, M, G, S, C = cfg
            tt = t(tokens).bfloat16() if kind == "bf16" else t(tokens)
            with CUDAExtension.disable():
                jag, rev = co_me.func_token_merge(tt, S, G, t(mask))
                restored = co_me.func_token_split(jag, rev, (1, B, S + M * G, C))
            out = jag.tokens[0].float().numpy()
            # the oracle must agree bit for bit with the reference before anything is written
            o_out, o_off, o_rev, o_w = orc.token_merge(tokens, S, G, mask)
            if kind == "bf16":
                o_out = orc._round_like(o_out, "bf16")
            assert close(o_out, out, kind), ("merge tokens", cfg, kind)
            assert np.array_equal(o_off, jag.offset.numpy()) and np.array_equal(o_rev, rev.numpy())
            assert np.array_equal(o_w, jag.weight.numpy())
            assert close(orc.token_split(o_out, o_rev), restored.float().numpy().reshape(-1, C), kind)
            key = f"c{i}_{kind}"
            store[key + "_offset"] = jag.offset.numpy()
            store[key + "_rev"] = rev.numpy().astype(np.int32)
            store[key + "_weight"] = jag.weight.numpy().astype(np.uint8)
            store.update({f"{key}_out_{k}": v for k, v in summarize_rows(out).items()})
            store.update({f"{key}_res_{k}": v for k, v in summarize_rows(restored.float().numpy().reshape(-1, C)).items()})
    np.savez_compressed(os.path.join(HERE, "merge_1d.npz"), **store)

    # ---- 2-D merge ---------------------------------------------------------------------------------------
    store = {}
    for i, cfg in enumerate(RANDOM_CONFIGS_2D):
        tokens, mask = merge2d_inputs(i, cfg)
        B, H, W, gh, gw, S, C = cfg
        with CUDAExtension.disable():
            jn, rn = co_me_2d.naive_func_token_merge_2d(t(tokens), S, gh, gw, H, W, t(mask))
            jc, rc = co_me_2d.func_token_merge_2d(t(tokens), S, gh, gw, H, W, t(mask))
        assert torch.allclose(jn.tokens, jc.tokens, rtol=1e-6, atol=1e-6) and torch.equal(rn, rc) and torch.equal(jn.offset, jc.offset)
        o_out, o_off, o_rev, o_w = orc.token_merge_2d(tokens, S, gh, gw, H, W, mask)
        assert close(o_out, jn.tokens[0].numpy()) and np.array_equal(o_rev, rn.numpy())
        assert np.array_equal(o_off, jn.offset.numpy()) and np.array_equal(o_w, jn.weight.numpy())
        key = f"c{i}"
        store[key + "_offset"] = jn.offset.numpy()
        store[key + "_rev"] = rn.numpy().astype(np.int32)
        store[key + "_weight"] = jn.weight.numpy().astype(np.uint8)
        store.update({f"{key}_out_{k}": v for k, v in summarize_rows(jn.tokens[0].numpy()).items()})
    np.savez_compressed(os.path.join(HERE, "merge_2d.npz"), **store)

    # ---- window selection: the reference's own build_ctx tensor code behind a stand-in predictor -------
    store = {}
    for name, spec in SELECT_CASES.items():
        conf = select_inputs(name)  # float32 array holding values exactly representable in spec["kind"]
        B, S, H, W = spec["B"], spec["S"], spec["H"], spec["W"]
        dt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[spec["kind"]]
        conf_t = t(conf).to(dt).reshape(B, S * H * W, 1)
        if spec["cls"] == "2d":
            merger = object.__new__(co_me_2d.CoMe_2D_TokenMerger)
            merger.group_h, merger.group_w = spec["gh"], spec["gw"]
            merger.conf_mode = co_me_2d.CoMe_2D_TokenMerger.ConfidenceMode(spec["mode"])
        else:
            merger = object.__new__(co_me.CoMe_TokenMerger)
            merger.group_size = spec["gh"] * spec["gw"]
            merger.conf_mode = co_me.CoMe_TokenMerger.ConfidenceMode(spec["mode"])
        merger.start_idx = 5
        merger.threshold = spec["thr"]
        merger.predictor = lambda feature, BPHWC, _c=conf_t: _c
        feature = torch.zeros(B, S, 4, H, W)
        mask, _shape = merger.build_ctx(feature)
        mask = mask.numpy()
        scope = "batch" if spec["cls"] == "2d" else "frame"
        o_mask = orc.select_windows(conf, B, S, H, W, spec["gh"], spec["gw"], spec["thr"], spec["mode"], scope,
                                    spec["kind"])
        assert np.array_equal(o_mask, mask), ("select", name, int((o_mask != mask).sum()))
        store[name + "_mask"] = np.packbits(mask.reshape(-1))
        store[name + "_shape"] = np.asarray(mask.shape)
    np.savez_compressed(os.path.join(HERE, "select.npz"), **store)

    # ---- biased attention: the reference test-suite's fp32 oracle ----------------------------------------
    store = {}
    for i, case in enumerate(list(ATTENTION_CASES) + list(EXTRA_ATTENTION_CASES)):
        seq_lens, Hh, D, kind = case
        qkv, bias, cu = attention_inputs(i, case)
        scale = 1.0 / (D ** 0.5)
        out = np.zeros((qkv.shape[0], Hh, D), np.float32)
        q, k, v = (t(qkv[:, j]) for j in range(3))
        for s in range(len(seq_lens)):
            a, b = int(cu[s]), int(cu[s + 1])
            for h in range(Hh):
                out[a:b, h] = attn_test._reference_attention_with_bias(
                    q[a:b, h], k[a:b, h], v[a:b, h], t(bias)[a:b], scale).numpy()
        o_out, _ = orc.attention_bias(qkv[:, 0], qkv[:, 1], qkv[:, 2], bias, cu, scale)
        assert np.allclose(o_out, out, atol=2e-6, rtol=1e-5), ("attention", case, np.abs(o_out - out).max())
        store[f"a{i}_out"] = out.astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "attention.npz"), **store)

    # ---- pre-attention preparation: the reference's prepare_packed_self_attention_qkv + rotary module ------
    ref_qkv = import_file(args.reference, "src/accelerate/common/qkv.py", "ref_common_qkv")
    ref_rope = import_file(args.reference, "src/thirdparty/vggt/layers/rope.py", "ref_vggt_rope")
    store = {}
    for i, case in enumerate(PREPARE_CASES):
        P, Hh, D, kind, use_norm, use_rope = case
        dt = {"bf16": torch.bfloat16, "f16": torch.float16}[kind]
        qkv, params, pos = prepare_inputs(i, case)
        norms = []
        for j in range(2):
            if use_norm:
                n = torch.nn.LayerNorm(D, eps=PREPARE_EPS).to(dt)
                with torch.no_grad():
                    n.weight.copy_(t(params[2 * j]))
                    n.bias.copy_(t(params[2 * j + 1]))
            else:
                n = torch.nn.Identity()
            norms.append(n)
        rope = ref_rope.RotaryPositionEmbedding2D(frequency=100.0) if use_rope else None
        with torch.no_grad():
            ref = ref_qkv.prepare_packed_self_attention_qkv(t(qkv).to(dt), norms[0], norms[1], rope,
                                                            t(pos)[None] if use_rope else None, dt)
        ref = ref.float().numpy()
        cos_t, sin_t = orc.rope_tables(D // 2, PREPARE_MAX_POSITION, 100.0, kind)
        if use_rope:  # the tables themselves must agree bit for bit
            rc, rs = rope._compute_frequency_components(D // 2, PREPARE_MAX_POSITION, torch.device("cpu"), dt)
            assert np.array_equal(rc.float().numpy(), cos_t) and np.array_equal(rs.float().numpy(), sin_t), case
        ours = orc.qkv_prepare(qkv, *(params if use_norm else [None] * 4), PREPARE_EPS, pos if use_rope else None,
                               cos_t, sin_t, kind)
        # LayerNorm statistics are summed in another order by the reference's CPU kernel: a normalised value
        # that lands next to a rounding boundary may differ by one unit in the last place of the run dtype, and
        # the rotation mixes two such values: bound = 2 ulp at the head vector's largest magnitude
        ulp = 2.0 * np.abs(ref).max(axis=-1, keepdims=True) * (2.0 ** -7 if kind == "bf16" else 2.0 ** -10)
        assert np.all(np.abs(ours - ref) <= ulp), ("prepare", case, np.abs(ours - ref).max())
        assert np.mean(ours != ref) < (1e-3 if use_norm else 1e-12), ("prepare", case, np.mean(ours != ref))
        assert np.array_equal(ours[:, 2], ref[:, 2])
        store[f"p{i}_qk"] = ref[:, :2].astype(np.float16 if kind == "f16" else np.float32).view(
            np.uint16 if kind == "f16" else np.uint32)
        if kind == "bf16":
            store[f"p{i}_qk"] = (store[f"p{i}_qk"] >> 16).astype(np.uint16)  # bfloat16 bit patterns
    # packed positions: the position tensor merged in bfloat16 by the reference's 2-D merger, truncated
    for i, case in enumerate(POSITION_CASES):
        frames, H, W, gh, gw, start = case
        mask = position_mask(i, case)
        ys, xs = np.meshgrid(np.arange(H), np.arange(W), indexing="ij")
        p = np.zeros((start + H * W, 2), np.float32)
        p[start:, 0] = ys.reshape(-1) + 1
        p[start:, 1] = xs.reshape(-1) + 1
        pos = t(np.broadcast_to(p, (frames,) + p.shape).copy()).to(torch.bfloat16)
        with CUDAExtension.disable():
            jag, _rev = co_me_2d.func_token_merge_2d(pos, start, gh, gw, H, W, t(mask))
        ref_pos = jag.tokens[0].long().numpy()
        assert np.array_equal(orc.packed_positions(mask, start, H, W, gh, gw), ref_pos), ("positions", case)
        store[f"pos{i}"] = ref_pos.astype(np.int16)
    np.savez_compressed(os.path.join(HERE, "prepare.npz"), **store)

    # ---- LayerNorm + merge: nn.LayerNorm on CPU, then the reference's 2-D merge of its output ---------------------
    store = {}
    for i, case in enumerate(LN_MERGE_CASES):
        frames, H, W, gh, gw, start, C, kind = case
        dt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[kind]
        x, gamma, beta, mask = ln_merge_inputs(i, case)
        ln = torch.nn.LayerNorm(C, eps=LN_MERGE_EPS).to(dt)
        with torch.no_grad():
            ln.weight.copy_(t(gamma))
            ln.bias.copy_(t(beta))
            y = ln(t(x).to(dt))
        with CUDAExtension.disable():
            jag, _rev = co_me_2d.func_token_merge_2d(y, start, gh, gw, H, W, t(mask))
        ref = jag.tokens[0].float().numpy()
        ours, _o, _r, _w = orc.token_merge_2d(orc.layer_norm_rows(x, gamma, beta, LN_MERGE_EPS, kind), start, gh, gw, H, W, mask)
        ours = orc._round_like(ours, kind)
        tol = ln_merge_tolerance(kind)
        assert np.allclose(ours, ref, rtol=tol, atol=tol), ("ln+merge", case, np.abs(ours - ref).max())
        store.update({f"l{i}_out_{k}": v for k, v in summarize_rows(ref, 7).items()})
    np.savez_compressed(os.path.join(HERE, "ln_merge.npz"), **store)

    # ---- transformer block on unmerged tokens: the reference model's own Block in float32 -------------------------
    from src.thirdparty.vggt.layers.block import Block as RefBlock
    store = {}
    for i, case in enumerate(BLOCK_CASES):
        frames, side, start, C, heads, mlp_ratio, qk_norm, use_rope, ls_init = case
        x, params, pos = block_inputs(i, case)
        rope = ref_rope.RotaryPositionEmbedding2D(frequency=100.0) if use_rope else None
        blk = RefBlock(dim=C, num_heads=heads, mlp_ratio=mlp_ratio, init_values=ls_init, qk_norm=qk_norm, rope=rope).eval()
        state = blk.state_dict()
        assert set(state) == set(params), (sorted(state), sorted(params))
        blk.load_state_dict({k: t(v) for k, v in params.items()})
        with torch.no_grad():
            ref = blk(t(x), pos=t(pos) if use_rope else None).numpy()
        N = x.shape[1]
        cos_t = sin_t = None
        if use_rope:
            cos_t, sin_t = orc.rope_tables(C // heads // 2, side + 1, 100.0, "f32")
        cu = np.arange(frames + 1, dtype=np.int64) * N
        ours = orc.jagged_block(x.reshape(-1, C), np.ones(frames * N, np.float32), cu, pos.reshape(-1, 2),
                                dict(params, norm_eps=blk.norm1.eps, qk_norm_eps=1e-5), heads, cos_t, sin_t)
        assert np.allclose(ours, ref.reshape(-1, C), rtol=BLOCK_TOLERANCE, atol=BLOCK_TOLERANCE), (
            "block", case, np.abs(ours - ref.reshape(-1, C)).max())
        store.update({f"b{i}_out_{k}": v for k, v in summarize_rows(ref.reshape(-1, C), 5).items()})
    np.savez_compressed(os.path.join(HERE, "block.npz"), **store)

    # ---- suffix tokens: the reference's own JaggedTokens.add_suffix / split_suffix -----------------------------------
    from src.interface.token_merger import ITokenMerger
    store = {}
    for i, case in enumerate(SUFFIX_CASES):
        tokens, weight, offset, suffix = suffix_inputs(i, case)
        jag = ITokenMerger.JaggedTokens(tokens=t(tokens)[None], weight=t(weight), offset=t(offset))
        ext = jag.add_suffix(t(suffix))
        o_tok, o_w, o_off = orc.jagged_add_suffix(tokens, weight, offset, suffix)
        assert np.array_equal(o_tok, ext.tokens[0].numpy()) and np.array_equal(o_w, ext.weight.numpy()), ("suffix", case)
        assert np.array_equal(o_off, ext.offset.numpy()), ("suffix", case)
        back, suf = ext.split_suffix(case[1])
        b_tok, b_w, b_off, b_suf = orc.jagged_split_suffix(o_tok, o_w, o_off, case[1])
        assert np.array_equal(b_tok, back.tokens[0].numpy()) and np.array_equal(b_w, back.weight.numpy()), ("split", case)
        assert np.array_equal(b_off, back.offset.numpy()) and np.array_equal(b_suf, suf.numpy()), ("split", case)
        assert np.array_equal(b_tok, tokens) and np.array_equal(b_suf, suffix)
        store[f"s{i}_tokens"], store[f"s{i}_weight"], store[f"s{i}_offset"] = (
            ext.tokens[0].numpy(), ext.weight.numpy().astype(np.uint8), ext.offset.numpy().astype(np.int32))
    np.savez_compressed(os.path.join(HERE, "suffix.npz"), **store)

    # ---- standalone op chain of the headline configuration (8 x 1374 tokens, 37x37 grid, 3x3 windows) ----
    tokens, conf = cfg1_inputs()
    B, N, C = tokens.shape
    mask = orc.select_windows(conf, 8, 1, 37, 37, 3, 3, 0.5, "pairwise-rank", "frame", "f32")
    # reference selection arithmetic on the same window means (torch.quantile + strict <)
    means = t(orc.window_means(conf, 37, 37, 3, 3))
    ref_mask = (means < torch.quantile(means.float(), 0.5, dim=-1, keepdim=True)).numpy()
    assert np.array_equal(mask, ref_mask)
    perm, prefix, M = orc.ragged_layout_2d(5, 37, 37, 3, 3)
    with CUDAExtension.disable():
        jag, rev_perm = co_me.func_token_merge(t(tokens[:, perm, :]), prefix, 9, t(mask))
    inv = np.empty(N, np.int64)
    inv[perm] = np.arange(N)
    rev = rev_perm.numpy().reshape(B, N)[:, inv].reshape(-1)
    o_out, o_off, o_rev, o_w = orc.token_merge_2d_ragged(tokens, 5, 3, 3, 37, 37, mask)
    assert close(o_out, jag.tokens[0].numpy()) and np.array_equal(o_rev, rev)
    assert np.array_equal(o_off, jag.offset.numpy()) and np.array_equal(o_w, jag.weight.numpy())
    with CUDAExtension.disable():
        restored = co_me.func_token_split(jag, t(rev), (1, B, N, C)).numpy().reshape(-1, C)
    store = dict(mask=np.packbits(mask.reshape(-1)), offset=jag.offset.numpy(), rev=rev.astype(np.int32),
                 weight=jag.weight.numpy().astype(np.uint8))
    store.update({f"out_{k}": v for k, v in summarize_rows(jag.tokens[0].numpy(), 97).items()})
    store.update({f"res_{k}": v for k, v in summarize_rows(restored, 211).items()})
    np.savez_compressed(os.path.join(HERE, "cfg1_chain.npz"), **store)
    print("fixtures written to", HERE)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f"  {f}: {os.path.getsize(os.path.join(HERE, f)) / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
