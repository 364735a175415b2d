import torch
from torch.autograd import Function

from ... import backend

__all__ = ["spvoxelize"]


class _Voxelize(Function):
    """Average pooling of point features into voxels and its gradient
    (torchsparse/nn/functional/voxelize.py:11-59)."""

    @staticmethod
    def forward(ctx, feats: torch.Tensor, coords: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
        ctx.save_for_backward(coords, counts)
        ctx.n = feats.shape[0]
        return backend.voxelize_forward_cuda(feats, coords, counts)

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        coords, counts = ctx.saved_tensors
        grad = backend.voxelize_backward_cuda(grad_output, coords, counts, ctx.n)
        return grad.to(grad_output.dtype), None, None


def spvoxelize(feats: torch.Tensor, coords: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    """Average the features of the points that fall into each voxel; ``coords`` holds the voxel
    index of every point (torchsparse/nn/functional/voxelize.py:11-59)."""
    feats, coords = feats.contiguous(), coords.contiguous().int()
    if torch.is_grad_enabled() and feats.requires_grad:
        return _Voxelize.apply(feats, coords, counts)
    return backend.voxelize_forward_cuda(feats, coords, counts)
