from typing import List

import torch

from .tensor import SparseTensor

__all__ = ["cat"]


def cat(inputs: List[SparseTensor]) -> SparseTensor:
    """Channel-wise concatenation of tensors living on the same coordinates
    (torchsparse/operators.py:12-16); used by the U-Net skip connections."""
    feats = torch.cat([inp.feats for inp in inputs], dim=1)
    output = SparseTensor(coords=inputs[0].coords, feats=feats, stride=inputs[0].stride,
                          spatial_range=inputs[0].spatial_range)
    output._caches = inputs[0]._caches
    return output
