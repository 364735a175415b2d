from typing import List

import torch

from .tensor import CatSparseTensor, SparseTensor

__all__ = ["cat", "generative_add"]

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


def generative_add(a: SparseTensor, b: SparseTensor) -> SparseTensor:
    """Sum of two tensors over the union of their coordinates (torchsparse/operators.py:53-64): rows with equal
    coordinates are added, the rest are kept; the output rows are in lexicographic coordinate order
    (``torch.unique(dim=0)``), stride, spatial range and caches are those of the operand with more rows."""
    first, second = (a, b) if a.feats.shape[0] >= b.feats.shape[0] else (b, a)
    union_coords = torch.cat([first.coords, second.coords], dim=0)
    union_feats = torch.cat([first.feats, second.feats], dim=0)
    unique_coords, inverse = torch.unique(union_coords, dim=0, return_inverse=True)
    out_feats = torch.zeros((unique_coords.shape[0], union_feats.shape[1]), dtype=union_feats.dtype,
                            device=union_feats.device)
    out_feats.index_add_(0, inverse, union_feats)
    out = SparseTensor(out_feats, unique_coords, first.stride, spatial_range=first.spatial_range)
    out._caches = first._caches
    return out
