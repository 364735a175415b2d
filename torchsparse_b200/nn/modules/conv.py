import math
from typing import Dict, List, Tuple, Union

import numpy as np
import torch
from torch import nn

from ...tensor import SparseTensor
from ...utils.utils import make_ntuple
from .. import functional as F

__all__ = ["Conv3d"]


class Conv3d(nn.Module):
    """Sparse 3-D convolution (torchsparse/nn/modules/conv.py:22-110).  Parameter ``kernel`` has
    shape [Kvol, Cin, Cout] ([Cin, Cout] for a 1x1x1 stride-1 kernel) in the reference's
    kernel-offset order, so reference state_dicts load unchanged.  Odd kernel dims at
    stride 1 are padded (k-1)/2 automatically; other dims use ``padding``."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: Union[int, List[int], Tuple[int, ...]] = 3,
                 stride: Union[int, List[int], Tuple[int, ...]] = 1, padding: Union[int, Tuple[int, ...]] = 0,
                 dilation: int = 1, bias: bool = False, transposed: bool = False, generative: bool = False,
                 config: Dict = None) -> None:
        super().__init__()
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel_size = make_ntuple(kernel_size, ndim=3)
        self.stride = make_ntuple(stride, ndim=3)
        self.dilation = dilation
        _padding = make_ntuple(padding, 3)
        self.padding = tuple(
            (self.kernel_size[i] - 1) // 2 if (self.kernel_size[i] % 2 == 1 and self.stride[i] == 1) else _padding[i]
            for i in range(3))
        self.transposed = transposed
        self.generative = generative
        if self.generative:
            assert self.transposed
        self._config = config
        self.kernel_volume = int(np.prod(self.kernel_size))
        if self.kernel_volume > 1 or self.stride != (1, 1, 1):
            self.kernel = nn.Parameter(torch.zeros(self.kernel_volume, in_channels, out_channels))
        else:
            self.kernel = nn.Parameter(torch.zeros(in_channels, out_channels))
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_channels))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def extra_repr(self) -> str:
        s = f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}"
        if self.stride != (1, 1, 1):
            s += f", stride={self.stride}"
        if self.dilation != 1:
            s += f", dilation={self.dilation}"
        if self.bias is None:
            s += ", bias=False"
        if self.transposed:
            s += ", transposed=True"
        if self.generative:
            s += ", generative=True"
        return s

    def reset_parameters(self) -> None:
        std = 1 / math.sqrt((self.out_channels if self.transposed else self.in_channels) * self.kernel_volume)
        self.kernel.data.uniform_(-std, std)
        if self.bias is not None:
            self.bias.data.uniform_(-std, std)

    def forward(self, input: SparseTensor) -> SparseTensor:
        return F.conv3d(input, weight=self.kernel, kernel_size=self.kernel_size, bias=self.bias, stride=self.stride,
                        padding=self.padding, dilation=self.dilation, transposed=self.transposed,
                        generative=self.generative, config=self._config, training=self.training)
