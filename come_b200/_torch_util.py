"""Small helpers shared by the host-side modules: dtype codes, stream and pointer access."""
from __future__ import annotations

import torch

from . import _lib

_DTYPE = {torch.float32: _lib.COME_F32, torch.float16: _lib.COME_F16, torch.bfloat16: _lib.COME_BF16}


def dtype_code(dtype: torch.dtype, what: str = "tensor") -> int:
    try:
        return _DTYPE[dtype]
    except KeyError:
        raise RuntimeError(f"{what}: unsupported dtype {dtype}; expected float32, float16 or bfloat16") from None


def require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be on CUDA")


def ptr(t):
    return None if t is None else t.data_ptr()


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream
