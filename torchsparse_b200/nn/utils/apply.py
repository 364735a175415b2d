from typing import Callable

import torch

from ...tensor import SparseTensor

__all__ = ["fapply"]


def fapply(input: SparseTensor, fn: Callable[..., torch.Tensor], *args, **kwargs) -> SparseTensor:
    """Apply a dense function to the feature matrix, keeping coordinates and caches
    (torchsparse/nn/utils/apply.py:10-21)."""
    output = SparseTensor(coords=input.coords, feats=fn(input.feats, *args, **kwargs), stride=input.stride,
                          spatial_range=input.spatial_range)
    output._caches = input._caches
    return output
