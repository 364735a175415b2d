from typing import List

import torch

from .tensor import CatSparseTensor, SparseTensor

__all__ = ["cat"]

# When True (set by the inference engine around its forward), `cat` of two tensors returns a
# CatSparseTensor: the concatenated matrix is only written if a layer asks for `.feats`; the fused
# convolutions read the two matrices directly.
lazy = False


def cat(inputs: List[SparseTensor]) -> SparseTensor:
    """Channel-wise concatenation of tensors living on the same coordinates
    (torchsparse/operators.py:12-16); used by the U-Net skip connections."""
    first = inputs[0]
    if lazy and len(inputs) == 2 and not torch.is_grad_enabled():
        out = CatSparseTensor([inp.feats for inp in inputs], first.coords, first.stride, first.spatial_range,
                              first._caches)
        dyn = getattr(first, "dyn", None)      # a tensor of the static engine: sizes live in device memory
        if dyn is not None:
            out.dyn = dyn
        return out
    feats = torch.cat([inp.feats for inp in inputs], dim=1)
    output = SparseTensor(coords=first.coords, feats=feats, stride=first.stride, spatial_range=first.spatial_range)
    output._caches = first._caches
    return output
