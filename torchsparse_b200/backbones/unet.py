from typing import List

from torch import nn

from ..operators import cat
from ..tensor import SparseTensor
from .. import nn as spnn
from .blocks import SparseConvBlock, SparseConvTransposeBlock, SparseResBlock

__all__ = ["SparseResUNet", "SparseResUNet42"]


class SparseResUNet(nn.Module):
    """Residual sparse U-Net: stem, four stride-2 encoder stages, four transposed-conv decoder
    stages with skip concatenation (torchsparse/backbones/unet.py:14-112).  Module names match
    the reference so its state_dicts load."""

    def __init__(self, stem_channels: int, encoder_channels: List[int], decoder_channels: List[int], *,
                 in_channels: int = 4, width_multiplier: float = 1.0) -> None:
        super().__init__()
        self.stem_channels = stem_channels
        self.encoder_channels = encoder_channels
        self.decoder_channels = decoder_channels
        self.in_channels = in_channels
        self.width_multiplier = width_multiplier
        nc = [int(width_multiplier * c) for c in [stem_channels] + encoder_channels + decoder_channels]
        self.stem = nn.Sequential(
            spnn.Conv3d(in_channels, nc[0], 3), spnn.BatchNorm(nc[0]), spnn.ReLU(True),
            spnn.Conv3d(nc[0], nc[0], 3), spnn.BatchNorm(nc[0]), spnn.ReLU(True),
        )
        self.encoders = nn.ModuleList()
        for k in range(4):
            self.encoders.append(nn.Sequential(
                SparseConvBlock(nc[k], nc[k], 2, stride=2),
                SparseResBlock(nc[k], nc[k + 1], 3),
                SparseResBlock(nc[k + 1], nc[k + 1], 3),
            ))
        self.decoders = nn.ModuleList()
        for k in range(4):
            self.decoders.append(nn.ModuleDict({
                "upsample": SparseConvTransposeBlock(nc[k + 4], nc[k + 5], 2, stride=2),
                "fuse": nn.Sequential(
                    SparseResBlock(nc[k + 5] + nc[3 - k], nc[k + 5], 3),
                    SparseResBlock(nc[k + 5], nc[k + 5], 3),
                ),
            }))

    def _unet_forward(self, x: SparseTensor, encoders, decoders) -> List[SparseTensor]:
        if not encoders and not decoders:
            return [x]
        xd = encoders[0](x)
        outputs = self._unet_forward(xd, encoders[1:], decoders[:-1])
        yd = outputs[-1]
        u = decoders[-1]["upsample"](yd)
        y = decoders[-1]["fuse"](cat([u, x]))
        return [x] + outputs + [y]

    def forward(self, x: SparseTensor) -> List[SparseTensor]:
        return self._unet_forward(self.stem(x), self.encoders, self.decoders)


class SparseResUNet42(SparseResUNet):
    def __init__(self, **kwargs) -> None:
        super().__init__(stem_channels=32, encoder_channels=[32, 64, 128, 256],
                         decoder_channels=[256, 128, 96, 96], **kwargs)
