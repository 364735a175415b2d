import torch

from ... import backend

__all__ = ["spvoxelize"]


def spvoxelize(feats: torch.Tensor, coords: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    """Average the features of the points that fall into each voxel; ``coords`` holds the voxel
    index of every point (torchsparse/nn/functional/voxelize.py:11-59; forward only)."""
    return backend.voxelize_forward_cuda(feats.contiguous(), coords.contiguous().int(), counts)
