from typing import Tuple, Union

import numpy as np
import torch

from ...utils.utils import make_ntuple

__all__ = ["get_kernel_offsets"]


def get_kernel_offsets(size: Union[int, Tuple[int, ...]], stride: Union[int, Tuple[int, ...]] = 1,
                       dilation: Union[int, Tuple[int, ...]] = 1, device="cpu") -> torch.Tensor:
    """Offsets of the kernel cells in weight order: x fastest for an odd kernel volume, z
    fastest for an even one (torchsparse/nn/utils/kernel.py:11-38)."""
    size = make_ntuple(size, ndim=3)
    stride = make_ntuple(stride, ndim=3)
    dilation = make_ntuple(dilation, ndim=3)
    axes = [np.arange(-size[k] // 2 + 1, size[k] // 2 + 1) * stride[k] * dilation[k] for k in range(3)]
    if int(np.prod(size)) % 2 == 1:
        grid = [(x, y, z) for z in axes[2] for y in axes[1] for x in axes[0]]
    else:
        grid = [(x, y, z) for x in axes[0] for y in axes[1] for z in axes[2]]
    return torch.tensor(grid, dtype=torch.int, device=device)
