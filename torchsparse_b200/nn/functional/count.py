import torch

from ... import backend

__all__ = ["spcount"]


def spcount(coords: torch.Tensor, num) -> torch.Tensor:
    """Histogram of voxel indices: points per voxel (torchsparse/nn/functional/count.py:8-16)."""
    return backend.count_cuda(coords.contiguous(), int(num))
