"""Residual sparse U-Net (torchsparse/backbones/unet.py:14-122): a two-conv stem, four stride-2 encoder
stages and four transposed-conv decoder stages that concatenate the encoder output of the same
resolution.  Attribute names (`stem`, `encoders`, `decoders[k]["upsample" | "fuse"]`) are the
reference's, so its state_dicts load."""
from typing import List

from torch import nn

from ..operators import cat
from .blocks import SparseConvBlock, SparseConvTransposeBlock, SparseResBlock

__all__ = ["SparseResUNet", "SparseResUNet42"]

_LEVELS = 4


class SparseResUNet(nn.Module):
    def __init__(self, stem_channels: int, encoder_channels: List[int], decoder_channels: List[int], *,
                 in_channels: int = 4, width_multiplier: float = 1.0) -> None:
        super().__init__()
        self.stem_channels, self.encoder_channels, self.decoder_channels = (stem_channels, encoder_channels,
                                                                            decoder_channels)
        self.in_channels, self.width_multiplier = in_channels, width_multiplier
        width = [int(width_multiplier * c) for c in (stem_channels, *encoder_channels, *decoder_channels)]
        enc, dec = width[:_LEVELS + 1], width[_LEVELS:]        # enc[k] / dec[k]: channels entering level k

        self.stem = nn.Sequential(*SparseConvBlock(in_channels, enc[0], 3), *SparseConvBlock(enc[0], enc[0], 3))
        self.encoders = nn.ModuleList(
            nn.Sequential(SparseConvBlock(enc[k], enc[k], 2, stride=2),
                          SparseResBlock(enc[k], enc[k + 1], 3),
                          SparseResBlock(enc[k + 1], enc[k + 1], 3))
            for k in range(_LEVELS))
        self.decoders = nn.ModuleList(
            nn.ModuleDict({
                "upsample": SparseConvTransposeBlock(dec[k], dec[k + 1], 2, stride=2),
                # the skip tensor of the same resolution comes from the encoder level mirrored around the bottleneck
                "fuse": nn.Sequential(SparseResBlock(dec[k + 1] + enc[_LEVELS - 1 - k], dec[k + 1], 3),
                                      SparseResBlock(dec[k + 1], dec[k + 1], 3)),
            })
            for k in range(_LEVELS))

    def forward(self, x) -> List:
        """[stem, enc1..enc4, dec1..dec4] outputs (9 tensors)."""
        skips = [self.stem(x)]
        for encoder in self.encoders:
            skips.append(encoder(skips[-1]))
        outputs = list(skips)
        y = skips[-1]
        for k, decoder in enumerate(self.decoders):
            y = decoder["fuse"](cat([decoder["upsample"](y), skips[_LEVELS - 1 - k]]))
            outputs.append(y)
        return outputs


class SparseResUNet42(SparseResUNet):
    def __init__(self, **kwargs) -> None:
        super().__init__(stem_channels=32, encoder_channels=[32, 64, 128, 256],
                         decoder_channels=[256, 128, 96, 96], **kwargs)
