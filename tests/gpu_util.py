"""Helpers of the GPU parity tests: numpy <-> CUDA tensors in a given storage dtype."""
import numpy as np
import torch

TORCH_DTYPE = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def to_dev(a: np.ndarray, kind: str = "f32") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda().to(TORCH_DTYPE[kind])


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy() if t.is_floating_point() else t.detach().cpu().numpy()
