"""Kernel-cell offsets in weight order (torchsparse/nn/utils/kernel.py:11-38)."""
from itertools import product
from typing import Tuple, Union

import torch

from ...utils.utils import make_ntuple

__all__ = ["get_kernel_offsets"]

_Size = Union[int, Tuple[int, ...]]


def get_kernel_offsets(size: _Size, stride: _Size = 1, dilation: _Size = 1, device="cpu") -> torch.Tensor:
    """int32 [Kvol, 3]: the (x, y, z) displacement of every kernel cell, in the order the rows of a
    ``Conv3d.kernel`` are stored.  Along an axis of extent k the cells sit at -(k-1)//2 ... k//2 (times
    stride and dilation).  The order is x fastest, z slowest when the kernel volume is odd and z fastest,
    x slowest when it is even — the layout the kernel-map builders assume."""
    size, stride, dilation = (make_ntuple(v, ndim=3) for v in (size, stride, dilation))
    per_axis = [[(c - (k - 1) // 2) * s * d for c in range(k)] for k, s, d in zip(size, stride, dilation)]
    volume = size[0] * size[1] * size[2]
    if volume % 2:
        cells = [(x, y, z) for z, y, x in product(per_axis[2], per_axis[1], per_axis[0])]
    else:
        cells = list(product(*per_axis))
    return torch.tensor(cells, dtype=torch.int32, device=device)
