"""Sparse ResNet backbones (torchsparse/backbones/resnet.py:12-66): a list of stages, each a strided
conv block followed by residual blocks; the forward returns the output of every stage."""
from typing import List, Sequence, Tuple, Union

from torch import nn

from .blocks import SparseConvBlock, SparseResBlock

__all__ = ["SparseResNet", "SparseResNet21D"]

_Size = Union[int, Tuple[int, ...]]
StageSpec = Tuple[int, int, _Size, _Size]          # (blocks in the stage, channels, kernel size, stride of its first conv)


def _stage(cin: int, cout: int, n_blocks: int, kernel_size: _Size, stride: _Size) -> nn.Sequential:
    first = SparseConvBlock(cin, cout, kernel_size, stride=stride)
    rest = [SparseResBlock(cout, cout, kernel_size) for _ in range(n_blocks - 1)]
    return nn.Sequential(first, *rest)


class SparseResNet(nn.ModuleList):
    def __init__(self, blocks: Sequence[StageSpec], *, in_channels: int = 4, width_multiplier: float = 1.0) -> None:
        super().__init__()
        self.blocks, self.in_channels, self.width_multiplier = blocks, in_channels, width_multiplier
        widths = [int(channels * width_multiplier) for _, channels, _, _ in blocks]
        for (n_blocks, _, kernel_size, stride), cin, cout in zip(blocks, [in_channels] + widths[:-1], widths):
            self.append(_stage(cin, cout, n_blocks, kernel_size, stride))

    def forward(self, x) -> List:
        per_stage = []
        for stage in self:
            x = stage(x)
            per_stage.append(x)
        return per_stage


class SparseResNet21D(SparseResNet):
    """Five stages, 21 convolutions: the detection backbone with the anisotropic last stage."""

    STAGES: Tuple[StageSpec, ...] = ((3, 16, 3, 1), (3, 32, 3, 2), (3, 64, 3, 2), (3, 128, 3, 2),
                                     (1, 128, (1, 3, 1), (1, 2, 1)))

    def __init__(self, **kwargs) -> None:
        super().__init__(blocks=list(self.STAGES), **kwargs)
