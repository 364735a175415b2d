"""Building blocks of the backbones (torchsparse/backbones/modules/blocks.py:12-85).  Child order and
attribute names are the reference's, so its state_dicts load."""
from typing import List, Sequence, Union

from torch import nn

from .. import nn as spnn

__all__ = ["SparseConvBlock", "SparseConvTransposeBlock", "SparseResBlock"]

_Size = Union[int, Sequence[int]]


def _conv_bn(cin: int, cout: int, kernel_size: _Size, *, stride: _Size = 1, dilation: int = 1,
             transposed: bool = False, relu: bool = False) -> List[nn.Module]:
    """[conv, BatchNorm(, ReLU)] — the unit every block here is made of."""
    layers: List[nn.Module] = [
        spnn.Conv3d(cin, cout, kernel_size, stride=stride, dilation=dilation, transposed=transposed),
        spnn.BatchNorm(cout),
    ]
    if relu:
        layers.append(spnn.ReLU(True))
    return layers


def _strided(stride: _Size) -> bool:
    return any(s != 1 for s in ((stride,) if isinstance(stride, int) else stride))


class SparseConvBlock(nn.Sequential):
    """conv → BatchNorm → ReLU."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: _Size, stride: _Size = 1,
                 dilation: int = 1) -> None:
        super().__init__(*_conv_bn(in_channels, out_channels, kernel_size, stride=stride, dilation=dilation, relu=True))


class SparseConvTransposeBlock(nn.Sequential):
    """transposed conv → BatchNorm → ReLU."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: _Size, stride: _Size = 1,
                 dilation: int = 1) -> None:
        super().__init__(*_conv_bn(in_channels, out_channels, kernel_size, stride=stride, dilation=dilation,
                                   transposed=True, relu=True))


class SparseResBlock(nn.Module):
    """ReLU(main(x) + shortcut(x)): main = conv-BN-ReLU-conv-BN; the shortcut is the identity unless the
    channel count or the resolution changes, then a 1x1x1 conv + BN."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: _Size, stride: _Size = 1,
                 dilation: int = 1) -> None:
        super().__init__()
        self.main = nn.Sequential(
            *_conv_bn(in_channels, out_channels, kernel_size, stride=stride, dilation=dilation, relu=True),
            *_conv_bn(out_channels, out_channels, kernel_size, dilation=dilation))
        reshapes = in_channels != out_channels or _strided(stride)
        self.shortcut = nn.Sequential(*_conv_bn(in_channels, out_channels, 1, stride=stride)) if reshapes \
            else nn.Identity()
        self.relu = spnn.ReLU(True)

    def forward(self, x):
        return self.relu(self.main(x) + self.shortcut(x))
