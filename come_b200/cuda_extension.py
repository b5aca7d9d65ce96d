"""Stands in for the reference's ``src.cuda_extension`` package (``src/cuda_extension/__init__.py:1-23``):
the three attention helpers plus the ``co_me_cuext`` module object that
``src/utility/feature.py:135-168`` looks accelerated entry points up on.

Install it into an unmodified reference checkout with :func:`install`.
"""
from __future__ import annotations

import sys
import types

from . import co_me_cuext, flash_attn, flash_attn_fwd_cuda
from .flash_attn import (
    flash_attn_varlen_qkvpacked_func,
    flash_attn_varlen_qkvpacked_func_w_perkey_bias,
    infer_flash_attn_varlen_max_seqlen,
)

__all__ = [
    "co_me_cuext",
    "flash_attn_varlen_qkvpacked_func",
    "flash_attn_varlen_qkvpacked_func_w_perkey_bias",
    "infer_flash_attn_varlen_max_seqlen",
    "install",
]

__version__ = "0.1.0"


def install(package: str = "src.cuda_extension") -> None:
    """Register this module (and its sub-modules) under the reference's import names, so that
    ``from src.cuda_extension import co_me_cuext, flash_attn_varlen_qkvpacked_func`` and
    ``from src.cuda_extension.flash_attn import infer_flash_attn_varlen_max_seqlen`` resolve to the sm_100a
    kernels.  Call it before anything imports ``src.accelerate``."""
    me = sys.modules[__name__]
    sys.modules[package] = me
    sys.modules[package + ".flash_attn"] = flash_attn
    sys.modules[package + ".flash_attn.flash_attn_fwd_cuda"] = flash_attn_fwd_cuda
    co_me_pkg = types.ModuleType(package + ".co_me")
    co_me_pkg.co_me_cuext = co_me_cuext
    sys.modules[package + ".co_me"] = co_me_pkg
    if not hasattr(me, "__path__"):
        me.__path__ = []  # lets `import src.cuda_extension.flash_attn` succeed
