from typing import List, Tuple, Union

import numpy as np
from torch import nn

from ..tensor import SparseTensor
from .. import nn as spnn

__all__ = ["SparseConvBlock", "SparseConvTransposeBlock", "SparseResBlock"]

_KS = Union[int, List[int], Tuple[int, ...]]


class SparseConvBlock(nn.Sequential):
    """conv - BN - ReLU (torchsparse/backbones/modules/blocks.py:12-29)."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: _KS, stride: _KS = 1,
                 dilation: int = 1) -> None:
        super().__init__(
            spnn.Conv3d(in_channels, out_channels, kernel_size, stride=stride, dilation=dilation),
            spnn.BatchNorm(out_channels),
            spnn.ReLU(True),
        )


class SparseConvTransposeBlock(nn.Sequential):
    """transposed conv - BN - ReLU (torchsparse/backbones/modules/blocks.py:32-50)."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: _KS, stride: _KS = 1,
                 dilation: int = 1) -> None:
        super().__init__(
            spnn.Conv3d(in_channels, out_channels, kernel_size, stride=stride, dilation=dilation, transposed=True),
            spnn.BatchNorm(out_channels),
            spnn.ReLU(True),
        )


class SparseResBlock(nn.Module):
    """conv-BN-ReLU-conv-BN plus identity or 1x1-conv-BN shortcut, then ReLU
    (torchsparse/backbones/modules/blocks.py:53-85)."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: _KS, stride: _KS = 1,
                 dilation: int = 1) -> None:
        super().__init__()
        self.main = nn.Sequential(
            spnn.Conv3d(in_channels, out_channels, kernel_size, dilation=dilation, stride=stride),
            spnn.BatchNorm(out_channels),
            spnn.ReLU(True),
            spnn.Conv3d(out_channels, out_channels, kernel_size, dilation=dilation),
            spnn.BatchNorm(out_channels),
        )
        if in_channels != out_channels or np.prod(stride) != 1:
            self.shortcut = nn.Sequential(
                spnn.Conv3d(in_channels, out_channels, 1, stride=stride),
                spnn.BatchNorm(out_channels),
            )
        else:
            self.shortcut = nn.Identity()
        self.relu = spnn.ReLU(True)

    def forward(self, x: SparseTensor) -> SparseTensor:
        return self.relu(self.main(x) + self.shortcut(x))
