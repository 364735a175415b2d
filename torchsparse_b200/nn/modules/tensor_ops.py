"""Module forms of the whole-tensor operators (torchsparse/nn/modules/{pooling,crop}.py)."""
from typing import Optional, Sequence

from torch import nn

from .. import functional as F

__all__ = ["GlobalAvgPool", "GlobalMaxPool", "SparseCrop"]


class _Functional(nn.Module):
    """A parameter-free module that forwards to one function of the functional namespace."""

    _fn = None

    def forward(self, input):
        return type(self)._fn(input)


class GlobalAvgPool(_Functional):
    _fn = staticmethod(F.global_avg_pool)


class GlobalMaxPool(_Functional):
    _fn = staticmethod(F.global_max_pool)


class SparseCrop(nn.Module):
    """Keeps the voxels inside ``[coords_min, coords_max)`` (see ``F.spcrop`` for the columns compared)."""

    def __init__(self, coords_min: Optional[Sequence[int]] = None, coords_max: Optional[Sequence[int]] = None) -> None:
        super().__init__()
        self.coords_min, self.coords_max = coords_min, coords_max

    def forward(self, input):
        return F.spcrop(input, self.coords_min, self.coords_max)

    def extra_repr(self) -> str:
        return f"coords_min={self.coords_min}, coords_max={self.coords_max}"
