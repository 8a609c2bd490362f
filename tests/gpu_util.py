"""Helpers for the GPU parity tests: numpy <-> device word tensors."""
import numpy as np
import torch


def to_dev(a: np.ndarray) -> torch.Tensor:
    """uint32/int32 numpy words -> int32 CUDA tensor holding the same bit patterns."""
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int32)).cuda()


def to_host(t: torch.Tensor, dtype=np.uint32) -> np.ndarray:
    return t.cpu().numpy().view(dtype)


def spread_bytes(levels: np.ndarray) -> np.ndarray:
    """Byte order of the int8 operands: inside each group of 32 k, element e sits at byte
    4*((31-e)&7) + ((31-e)>>3) (the order apnn_expand_planes writes and both GEMM operands share)."""
    K = levels.shape[-1]
    e = np.arange(32)
    pos = 4 * ((31 - e) & 7) + ((31 - e) >> 3)
    out = np.zeros(levels.shape, dtype=np.uint8)
    grouped = levels.reshape(levels.shape[:-1] + (K // 32, 32))
    og = out.reshape(grouped.shape)
    og[..., pos] = grouped
    return out
