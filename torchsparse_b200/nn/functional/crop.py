"""``spcrop``: keep the voxels inside a coordinate box (torchsparse/nn/functional/crop.py:10-35)."""
from typing import Optional, Tuple

import torch

from ...tensor import SparseTensor

__all__ = ["spcrop"]


def spcrop(input: SparseTensor, coords_min: Optional[Tuple[int, ...]] = None,
           coords_max: Optional[Tuple[int, ...]] = None) -> SparseTensor:
    """Voxels whose first three coordinate columns lie in ``[coords_min, coords_max)``.

    As in the reference the comparison runs over columns 0..2 of the coordinate rows and the upper
    bound is exclusive; with the (batch, x, y, z) layout those columns are batch, x, y — callers of the
    reference rely on exactly this, so it is kept.  The result starts a new kernel-map cache."""
    coords, feats = input.coords, input.feats
    keep = torch.ones(coords.shape[0], dtype=torch.bool, device=coords.device)
    if coords_min is not None:
        lo = torch.tensor(coords_min, dtype=coords.dtype, device=coords.device)
        keep &= (coords[:, :3] >= lo).all(dim=1)
    if coords_max is not None:
        hi = torch.tensor(coords_max, dtype=coords.dtype, device=coords.device)
        keep &= (coords[:, :3] < hi).all(dim=1)
    return SparseTensor(feats[keep], coords[keep], input.stride)
