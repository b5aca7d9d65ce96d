"""CPU-only checks of the boundary: the C-ABI library loads and exports every symbol declared in
include/come_b200.h; host-only entry points work without a GPU; validators raise before anything launches."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "come_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(come_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from come_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        from come_b200.build import build
        build()
    lib = ctypes.CDLL(_lib.LIB_PATH)
    declared = _declared_symbols()
    assert len(declared) >= 10
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/come_b200.h but not exported"
    assert set(_lib.EXPORTS) <= set(declared)


def test_version_and_layout_info_need_no_gpu():
    from come_b200 import _lib
    lib = _lib.lib()
    assert lib.come_version() == 100
    n_groups, n_tok, prefix = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
    lay = _lib.Layout.two_d(5, 37, 37, 3, 3)
    assert lib.come_layout_info(ctypes.byref(lay), ctypes.byref(n_groups), ctypes.byref(n_tok), ctypes.byref(prefix)) == 0
    assert (n_groups.value, n_tok.value, prefix.value) == (144, 1374, 78)
    lay = _lib.Layout.one_d(2, 4, 10)
    assert lib.come_layout_info(ctypes.byref(lay), ctypes.byref(n_groups), ctypes.byref(n_tok), ctypes.byref(prefix)) == 0
    assert (n_groups.value, n_tok.value, prefix.value) == (10, 42, 2)
    bad = _lib.Layout.one_d(-1, 4, 10)
    assert lib.come_layout_info(ctypes.byref(bad), None, None, None) == _lib.COME_ERR_ARG
    assert "start_index" in _lib.last_error()


def test_argument_errors_are_reported_without_a_gpu():
    from come_b200 import _lib
    lib = _lib.lib()
    rc = lib.come_attn_varlen_fwd(None, None, None, _lib.COME_F32, 16, 2, 64, 384, 384, 384, None, None, 1, 16, 0.125, None,
                                  128, None, 0, None)
    assert rc == _lib.COME_ERR_ARG and "fp16 and bf16" in _lib.last_error()
    rc = lib.come_select_windows(None, _lib.COME_F32, 1, 1, 6, 6, 3, 3, 1.5, 0, 0, None, None)
    assert rc == _lib.COME_ERR_ARG and "threshold" in _lib.last_error()


def test_peer_entry_points_validate_before_touching_the_device():
    """The peer-window entry points check their arguments first (no GPU needed to be told so)."""
    from come_b200 import _lib
    lib = _lib.lib()
    assert lib.come_peer_alloc(0, None, None) == _lib.COME_ERR_ARG and "bytes" in _lib.last_error()
    assert lib.come_peer_open(None, None) == _lib.COME_ERR_ARG
    assert lib.come_peer_copy(None, None, -1, None) == _lib.COME_ERR_ARG
    assert lib.come_peer_copy(None, None, 0, None) == _lib.COME_OK  # nothing to copy
    assert lib.come_peer_signal(None, 2, 0, 1, None) == _lib.COME_ERR_ARG
    flags = (ctypes.c_int32 * 4)()
    assert lib.come_peer_wait(flags, 4, 7, 1, 10 ** 9, None) == _lib.COME_ERR_ARG and "rank" in _lib.last_error()
    assert lib.come_peer_wait(flags, 4, 0, 1, 0, None) == _lib.COME_ERR_ARG and "limit_ns" in _lib.last_error()
    assert lib.come_peer_close(None) == _lib.COME_OK and lib.come_peer_free(None) == _lib.COME_OK


def test_python_validators_raise_value_error_on_cpu_tensors():
    import torch
    from come_b200 import token_merger as tm
    with pytest.raises(ValueError, match="Expected N = start_index"):
        tm.func_token_merge(torch.randn(2, 7, 4), 0, 2, torch.ones(2, 3, dtype=torch.bool))
    with pytest.raises(ValueError, match="torch.bool"):
        tm.func_token_merge(torch.randn(1, 6, 4), 0, 2, torch.ones(1, 3))
    with pytest.raises(ValueError, match="H.*divisible"):
        tm.func_token_merge_2d(torch.randn(1, 15, 4), 0, 2, 3, 3, 5, torch.ones(1, 3, dtype=torch.bool))
    # nothing silently computes on the CPU: a valid CPU call is refused by the extension shim
    with pytest.raises(RuntimeError, match="on CUDA"):
        tm.func_token_merge(torch.randn(1, 6, 4), 0, 2, torch.ones(1, 3, dtype=torch.bool))


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from come_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libcome_b200.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _lib.lib()


def test_jagged_suffix_roundtrip_cpu():
    """add_suffix / split_suffix of the packed container (reference: src/interface/token_merger.py:23-100,
    goldens of test/auto_test/test_jagged_suffix.py) -- pure tensor code, runs on CPU."""
    import torch
    from come_b200.token_merger import JaggedTokens
    tokens = torch.arange(10, dtype=torch.float32).reshape(1, 5, 2)
    jag = JaggedTokens(tokens=tokens, weight=torch.tensor([1., 2., 1., 1., 3.]), offset=torch.tensor([0, 2, 5]))
    suffix = torch.tensor([[[100., 101.]], [[200., 201.]]])
    ext = jag.add_suffix(suffix)
    assert ext.offset.tolist() == [0, 3, 7]
    assert ext.tokens[0, :, 0].tolist() == [0., 2., 100., 4., 6., 8., 200.]
    assert ext.weight.tolist() == [1., 2., 1., 1., 1., 3., 1.]
    back, suf = ext.split_suffix(1)
    assert torch.equal(back.tokens, jag.tokens) and torch.equal(back.weight, jag.weight)
    assert torch.equal(back.offset, jag.offset) and torch.equal(suf, suffix)


def test_tail_split_plan_is_a_pure_function_of_the_shape():
    """``plan_tail_split``: 10,534 rows x 16 heads = 448 work items -> the 27 query blocks of three full rounds on 148 CTAs
    in one launch, the last block with its keys in nine shares; launches whose last round is at least half full, launches
    shorter than one round and exact multiples are left alone; no share is ever empty."""
    from come_b200.flash_attn_fwd_cuda import plan_tail_split
    assert plan_tail_split(10534, 16, 70138, 148) == (10368, 9)
    assert plan_tail_split(10534, 16, 4096, 148) == (10368, 8)     # 64 key tiles: shares of 8 tiles
    assert plan_tail_split(9656, 16, 71016, 148) == (9656, 1)      # 416 items: the third round is 81 % full
    assert plan_tail_split(807, 16, 807, 148) == (807, 1)          # 48 items: less than one round
    assert plan_tail_split(384 * 37, 4, 5000, 148) == (384 * 37, 1)  # 148 items: one exact round
    assert plan_tail_split(80672, 16, 80672, 146) == (80256, 4)
    for rows in range(1, 30000, 997):
        for kv in (64, 65, 1000, 70138):
            main_rows, parts = plan_tail_split(rows, 16, kv, 148)
            tiles = -(-kv // 64)
            assert 0 < main_rows <= rows and main_rows % 384 == 0 or main_rows == rows
            assert parts == 1 or (2 <= parts <= 64 and (parts - 1) * -(-tiles // parts) < tiles)
