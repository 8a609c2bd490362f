"""Helpers for the GPU parity tests: numpy <-> device word tensors."""
import numpy as np
import torch


def to_dev(a: np.ndarray) -> torch.Tensor:
    """uint32/int32 numpy words -> int32 CUDA tensor holding the same bit patterns."""
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int32)).cuda()


def to_host(t: torch.Tensor, dtype=np.uint32) -> np.ndarray:
    return t.cpu().numpy().view(dtype)
