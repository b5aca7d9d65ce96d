"""ctypes binding of ``libcome_b200.so`` (declared in ``include/come_b200.h``).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcome_b200.so")

COME_F32, COME_F16, COME_BF16 = 0, 1, 2
COME_OK, COME_ERR_ARG, COME_ERR_CUDA, COME_ERR_UNSUPPORTED, COME_ERR_DEVICE = 0, -1, -2, -3, -4
COME_SELECT_RANK, COME_SELECT_ABS, COME_SELECT_ZSCORE = 0, 1, 2
COME_SCOPE_BATCH, COME_SCOPE_FRAME = 0, 1

EXPORTS = (
    "come_version", "come_last_error", "come_layout_info", "come_select_windows", "come_select_windows_ratios",
    "come_merge_plan_workspace_bytes", "come_merge_plan", "come_merge_plan_static", "come_merge", "come_merge_layernorm", "come_unmerge",
    "come_unmerge_strided", "come_unmerge_residual", "come_residual_layernorm", "come_suffix_add", "come_suffix_split",
    "come_attn_varlen_fwd", "come_attn_varlen_fwd_rows", "come_attn_cross_fwd", "come_attn_cross_fwd_parts", "come_attn_combine", "come_attn_combine_parts", "come_attn_set_cta_limit", "come_qkv_prepare", "come_packed_positions",
    "come_device_status", "come_selftest_bounded_wait",
    "come_peer_alloc", "come_peer_open", "come_peer_close", "come_peer_free", "come_peer_copy", "come_peer_signal", "come_peer_wait",
)
COME_PEER_HANDLE_BYTES = 64


class Layout(C.Structure):
    """``come_layout_t``."""
    _fields_ = [("start_index", C.c_int32), ("grid_h", C.c_int32), ("grid_w", C.c_int32),
                ("group_h", C.c_int32), ("group_w", C.c_int32), ("n_groups", C.c_int32)]

    @classmethod
    def one_d(cls, start_index: int, group_size: int, n_groups: int) -> "Layout":
        return cls(start_index, 0, 0, 1, group_size, n_groups)

    @classmethod
    def two_d(cls, start_index: int, H: int, W: int, gh: int, gw: int) -> "Layout":
        return cls(start_index, H, W, gh, gw, 0)


_lib = None


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built (``python -m come_b200.build``)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m come_b200.build` (needs nvcc); "
            "come_b200 has no CPU or PyTorch fallback")
    l = C.CDLL(LIB_PATH)
    vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_int64, C.c_float
    l.come_version.restype = C.c_int
    l.come_last_error.restype = C.c_char_p
    l.come_layout_info.argtypes = [C.POINTER(Layout), C.POINTER(i64), C.POINTER(i64), C.POINTER(i64)]
    l.come_select_windows.argtypes = [vp, i32, i64, i64, i32, i32, i32, i32, f32, i32, i32, vp, vp]
    l.come_select_windows_ratios.argtypes = [vp, i32, i64, i64, i32, i32, i32, i32, vp, i32, vp, vp]
    l.come_merge_plan_workspace_bytes.argtypes = [i64]
    l.come_merge_plan_workspace_bytes.restype = C.c_size_t
    l.come_merge_plan.argtypes = [vp, i64, C.POINTER(Layout), vp, vp, vp, vp, vp, vp, C.c_size_t, vp]
    l.come_merge_plan_static.argtypes = [vp, i64, C.POINTER(Layout), vp, vp, vp, vp, vp, vp]
    l.come_merge.argtypes = [vp, i32, i64, i64, C.POINTER(Layout), vp, vp, vp, vp, vp]
    l.come_merge_layernorm.argtypes = [vp, i32, i64, i64, C.POINTER(Layout), vp, vp, f32, vp, vp, vp, vp, vp]
    l.come_unmerge.argtypes = [vp, vp, i64, i64, i32, vp, vp]
    l.come_unmerge_strided.argtypes = [vp, vp, i64, i64, i32, vp, i64, vp]
    l.come_unmerge_residual.argtypes = [vp, vp, i64, i64, i32, vp, vp, vp, vp]
    l.come_residual_layernorm.argtypes = [vp, vp, vp, i64, i64, i32, vp, vp, f32, vp, vp, vp]
    l.come_suffix_add.argtypes = [vp, vp, vp, i64, i64, i64, i32, vp, i64, vp, vp, vp, vp]
    l.come_suffix_split.argtypes = [vp, vp, vp, i64, i64, i64, i32, i64, vp, vp, vp, vp, vp]
    l.come_attn_varlen_fwd.argtypes = [vp, vp, vp, i32, i64, i32, i32, i64, i64, i64, vp, vp, i32, i32, f32, vp, i64,
                                       vp, i32, vp]
    l.come_attn_varlen_fwd_rows.argtypes = [vp, vp, vp, i32, i64, i64, i64, i32, i32, i64, i64, i64, vp, vp, i32, i32, vp, f32,
                                            vp, i64, vp, i32, vp]
    l.come_attn_cross_fwd.argtypes = [vp, vp, vp, i32, i64, i64, i32, i32, i64, i64, i64, vp, f32, vp, i64, vp, i32, vp]
    l.come_attn_combine.argtypes = [vp, vp, vp, vp, i32, i64, i32, i32, vp, vp, vp]
    l.come_attn_cross_fwd_parts.argtypes = [vp, vp, vp, i32, i64, i64, i32, i32, i64, i64, i64, vp, f32, i32, vp, vp, i32, vp]
    l.come_attn_combine_parts.argtypes = [vp, vp, i32, i32, i64, i32, i32, vp, vp, vp]
    l.come_attn_set_cta_limit.argtypes = [i32]
    l.come_qkv_prepare.argtypes = [vp, i32, i64, i32, i32, vp, vp, vp, vp, f32, vp, vp, vp, i64, vp, vp, vp]
    l.come_packed_positions.argtypes = [vp, vp, i64, C.POINTER(Layout), vp, vp]
    l.come_device_status.argtypes = [C.POINTER(C.c_uint32), i32]
    l.come_selftest_bounded_wait.argtypes = [i64, vp, vp]
    l.come_peer_alloc.argtypes = [i64, C.POINTER(vp), vp]
    l.come_peer_open.argtypes = [vp, C.POINTER(vp)]
    l.come_peer_close.argtypes = [vp]
    l.come_peer_free.argtypes = [vp]
    l.come_peer_copy.argtypes = [vp, vp, i64, vp]
    l.come_peer_signal.argtypes = [vp, i32, i32, i32, vp]
    l.come_peer_wait.argtypes = [vp, i32, i32, i32, i64, vp]
    for name in EXPORTS:
        fn = getattr(l, name)
        if name not in ("come_last_error", "come_merge_plan_workspace_bytes"):
            fn.restype = C.c_int
    _lib = l
    return l


def last_error() -> str:
    return lib().come_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    """Turn a COME_* status into the exception class the reference raises for the same condition:
    argument errors -> ValueError is raised by the Python validators before dispatch, so what reaches the
    library and fails its checks is a RuntimeError (the reference's TORCH_CHECK)."""
    if rc == COME_OK:
        return
    msg = last_error()
    if rc == COME_ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(f"come_b200 error {rc}: {msg}")


def device_status(clear: bool = True) -> int:
    """The device status word (0 = no kernel reported a problem); synchronises the device."""
    v = C.c_uint32(0)
    rc = lib().come_device_status(C.byref(v), 1 if clear else 0)
    if rc not in (COME_OK, COME_ERR_DEVICE):
        check(rc)
    return int(v.value)


def raise_on_device_error(clear: bool = True) -> None:
    """RuntimeError with the library's description of the status word when a kernel reported a problem."""
    v = C.c_uint32(0)
    check(lib().come_device_status(C.byref(v), 1 if clear else 0))
