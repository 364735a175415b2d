"""Lifting a dense function to SparseTensor features (torchsparse/nn/utils/apply.py:10-21)."""
from typing import Callable

import torch

from ...tensor import SparseTensor

__all__ = ["fapply"]


def fapply(input: SparseTensor, fn: Callable[..., torch.Tensor], *args, **kwargs) -> SparseTensor:
    """``fn(input.feats, *args, **kwargs)`` wrapped back into a SparseTensor that shares the input's
    coordinates, stride, spatial range and kernel-map cache (the geometry does not change)."""
    mapped = fn(input.feats, *args, **kwargs)
    return SparseTensor._from_parts(mapped, input.coords, input.stride, input.spatial_range, input._caches)
