from typing import Tuple

import torch
from torch.autograd import Function

__all__ = ["to_dense"]


class ToDenseFunction(Function):
    """Scatter of sparse rows into a dense tensor and its gather backward
    (torchsparse/utils/to_dense.py:13-64)."""

    @staticmethod
    def forward(ctx, feats: torch.Tensor, coords: torch.Tensor, spatial_range: Tuple[int, ...]) -> torch.Tensor:
        from .. import backend

        if feats.device.type != "cuda":
            raise NotImplementedError
        feats = feats.contiguous()
        coords = coords.contiguous().int()
        outputs = torch.zeros(tuple(spatial_range) + (feats.size(1),), dtype=feats.dtype, device=feats.device)
        backend.to_dense_forward_cuda(feats, coords, spatial_range, outputs)
        ctx.for_backwards = (coords, tuple(spatial_range))
        return outputs

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        from .. import backend

        coords, spatial_range = ctx.for_backwards
        grad_output = grad_output.contiguous()
        grad_feats = torch.empty((coords.size(0), grad_output.size(-1)), dtype=grad_output.dtype,
                                 device=grad_output.device)
        backend.to_dense_backward_cuda(grad_output, coords, spatial_range, grad_feats)
        return grad_feats, None, None


def to_dense(feats: torch.Tensor, coords: torch.Tensor, spatial_range: Tuple[int, ...]) -> torch.Tensor:
    """Dense [B, X, Y, Z, C] tensor holding the rows of ``feats`` at their coordinates (zeros elsewhere)."""
    return ToDenseFunction.apply(feats, coords, tuple(spatial_range))
