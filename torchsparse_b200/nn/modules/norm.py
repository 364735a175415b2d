from torch import nn

from ...tensor import SparseTensor
from ..utils import fapply

__all__ = ["BatchNorm", "InstanceNorm"]


class BatchNorm(nn.BatchNorm1d):
    """BatchNorm1d over the feature matrix (torchsparse/nn/modules/norm.py:15-17)."""

    def forward(self, input: SparseTensor) -> SparseTensor:
        return fapply(input, super().forward)


class InstanceNorm(nn.InstanceNorm1d):
    def forward(self, input: SparseTensor) -> SparseTensor:
        return fapply(input, super().forward)
