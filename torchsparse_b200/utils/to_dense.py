from typing import Tuple

import torch

__all__ = ["to_dense"]


def to_dense(feats: torch.Tensor, coords: torch.Tensor, spatial_range: Tuple[int, ...]) -> torch.Tensor:
    """Scatter sparse rows into a dense [B,X,Y,Z,C] tensor (torchsparse/utils/to_dense.py:13-64;
    forward only)."""
    from .. import backend

    feats = feats.contiguous()
    coords = coords.contiguous().int()
    outputs = torch.zeros(tuple(spatial_range) + (feats.size(1),), dtype=feats.dtype, device=feats.device)
    backend.to_dense_forward_cuda(feats, coords, spatial_range, outputs)
    return outputs
