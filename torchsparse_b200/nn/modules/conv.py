"""The sparse convolution layer (torchsparse/nn/modules/conv.py:22-110)."""
import math
from typing import Dict, Optional, Sequence, Tuple, Union

import torch
from torch import nn

from ...utils.utils import make_ntuple
from .. import functional as F

__all__ = ["Conv3d"]

_Size = Union[int, Sequence[int]]


def _effective_padding(kernel_size: Tuple[int, ...], stride: Tuple[int, ...], padding: Tuple[int, ...]):
    """An odd kernel extent at stride 1 is centred ((k - 1) / 2 of padding, whatever was asked for);
    every other axis keeps the padding it was given."""
    return tuple((k - 1) // 2 if (k % 2 == 1 and s == 1) else p for k, s, p in zip(kernel_size, stride, padding))


class Conv3d(nn.Module):
    """``kernel`` is [Kvol, Cin, Cout] — or [Cin, Cout] for a 1x1x1 stride-1 layer — with the kernel
    cells in the reference's offset order, so its state_dicts load unchanged.  ``config`` pins the
    dataflow configuration of this layer (see ``F.conv_config``); None follows the global setting."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: _Size = 3, stride: _Size = 1,
                 padding: _Size = 0, dilation: int = 1, bias: bool = False, transposed: bool = False,
                 generative: bool = False, config: Optional[Dict] = None) -> None:
        super().__init__()
        if generative and not transposed:
            raise AssertionError("a generative convolution is a transposed one")
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride = make_ntuple(kernel_size, ndim=3), make_ntuple(stride, ndim=3)
        self.padding = _effective_padding(self.kernel_size, self.stride, make_ntuple(padding, 3))
        self.dilation, self.transposed, self.generative, self._config = dilation, transposed, generative, config
        self.kernel_volume = math.prod(self.kernel_size)
        pointwise = self.kernel_volume == 1 and self.stride == (1, 1, 1)
        shape = (in_channels, out_channels) if pointwise else (self.kernel_volume, in_channels, out_channels)
        self.kernel = nn.Parameter(torch.zeros(*shape))
        self.bias = nn.Parameter(torch.zeros(out_channels)) if bias else None
        self.reset_parameters()

    def reset_parameters(self) -> None:
        """U(-b, b) with b = 1 / sqrt(fan * Kvol), fan = Cout for a transposed layer, else Cin."""
        fan = self.out_channels if self.transposed else self.in_channels
        bound = 1.0 / math.sqrt(fan * self.kernel_volume)
        # in-place under no_grad, not through .data: the version counter moves, so weight copies cached for the
        # tensor-core kernel (packed / padded layouts) are rebuilt
        with torch.no_grad():
            for param in (self.kernel, self.bias):
                if param is not None:
                    param.uniform_(-bound, bound)

    def extra_repr(self) -> str:
        parts = [f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}"]
        if self.stride != (1, 1, 1):
            parts.append(f"stride={self.stride}")
        if self.dilation != 1:
            parts.append(f"dilation={self.dilation}")
        parts += [flag for flag, on in (("bias=False", self.bias is None), ("transposed=True", self.transposed),
                                        ("generative=True", self.generative)) if on]
        return ", ".join(parts)

    def forward(self, input):
        return F.conv3d(input, self.kernel, self.kernel_size, self.bias, self.stride, self.padding, self.dilation,
                        self._config, self.transposed, self.generative, self.training)
