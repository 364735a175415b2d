"""``spdownsample``: output coordinates of a strided convolution for ``kmap_mode="hashmap"``
(torchsparse/nn/functional/conv/kmap/downsample.py:11-79)."""
from typing import Optional, Tuple, Union

import torch

from .... import backend
from ....utils.utils import make_ntuple

__all__ = ["spdownsample"]


def spdownsample(_coords: torch.Tensor, stride: Union[int, Tuple[int, ...]] = 2,
                 kernel_size: Union[int, Tuple[int, ...]] = 2, padding: Union[int, Tuple[int, ...]] = 0,
                 spatial_range: Optional[Tuple[int, ...]] = None, downsample_mode: str = "spconv") -> torch.Tensor:
    """int32 [M,4] (b,x,y,z), rows in ascending order.

    * every stride equal to 1 or to the kernel size (or ``downsample_mode="minkowski"``): the unique
      rows of floor(coords / stride);
    * otherwise: the outputs reached by the kernel footprints of the inputs, enumerated natively,
      inside the bounds the reference derives (largest coordinate, padding, kernel size, stride)."""
    from ....tensor import get_allow_negative_coordinates

    if downsample_mode not in ("spconv", "minkowski"):
        raise ValueError(f"unknown downsample_mode {downsample_mode!r}")
    stride = make_ntuple(stride, ndim=3)
    kernel_size = make_ntuple(kernel_size, ndim=3)
    padding = make_ntuple(padding, ndim=3)
    if all(stride[k] in (1, kernel_size[k]) for k in range(3)) or downsample_mode == "minkowski":
        coords = _coords.clone()
        div = torch.tensor(stride, dtype=torch.float32, device=_coords.device).unsqueeze(0)
        coords[:, 1:] = torch.div(coords[:, 1:], div).floor().to(coords.dtype)
        return torch.unique(coords, dim=0)
    if _coords.device.type != "cuda":
        raise NotImplementedError("spdownsample with stride != kernel size needs CUDA tensors")
    coords = _coords.contiguous()
    if spatial_range is not None:
        cmax = tuple(int(v) - 1 for v in spatial_range)
    else:
        mx = coords.max(0).values.cpu().tolist()
        cmax = (mx[0],) + tuple((mx[1 + i] + 2 * padding[i] - (kernel_size[i] - 1)) // stride[i] for i in range(3))
    if get_allow_negative_coordinates():
        mn = coords.min(0).values.cpu().tolist()
        cmin = (mn[0],) + tuple(int((mn[1 + i] - 2 * padding[i] + (kernel_size[i] - 1)) / stride[i]) for i in range(3))
    else:
        cmin = (0, 0, 0, 0)
    return backend.downsample_cuda(coords, cmax, cmin, kernel_size, stride, padding)
