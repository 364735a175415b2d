"""Output coordinates of a generative transposed convolution
(torchsparse/nn/functional/conv/kmap/upsample.py:12-38)."""
from typing import Optional, Tuple, Union

import torch

from ....utils.utils import make_ntuple
from ...utils.kernel import get_kernel_offsets

__all__ = ["spupsample_generative"]


def spupsample_generative(_coords: torch.Tensor, stride: Union[int, Tuple[int, ...]] = 2,
                          kernel_size: Union[int, Tuple[int, ...]] = 2, padding=0,
                          spatial_range: Optional[Tuple[int, ...]] = None) -> torch.Tensor:
    """Every input voxel, scaled by the stride, spawns one output voxel per kernel cell (cell offsets of a stride-1,
    dilation-1 kernel); coordinates are clamped to [0, spatial_range - 1] per axis and duplicates removed.  Rows come
    out in lexicographic (b, x, y, z) order, as ``torch.unique(dim=0)`` gives them.  ``padding`` is accepted and
    unused, as in the reference."""
    stride = make_ntuple(stride, ndim=3)
    kernel_size = make_ntuple(kernel_size, ndim=3)
    if spatial_range is None:
        raise AssertionError("spatial range must be specified in generative mode")
    offsets = get_kernel_offsets(kernel_size, 1, 1, device=_coords.device)
    coords = _coords.clone()
    coords[:, 1:] *= torch.tensor(stride, dtype=coords.dtype, device=coords.device)
    coords = coords.unsqueeze(1).repeat(1, offsets.shape[0], 1)
    coords[:, :, 1:] += offsets.to(coords.dtype).unsqueeze(0)
    for i in range(1, coords.shape[-1]):
        coords[:, :, i].clamp_(min=0, max=int(spatial_range[i]) - 1)
    return torch.unique(coords.reshape(-1, coords.shape[-1]), dim=0)
