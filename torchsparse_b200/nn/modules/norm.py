import torch
from torch import nn

from ...tensor import SparseTensor
from ..utils import fapply

__all__ = ["BatchNorm", "GroupNorm", "InstanceNorm"]


class BatchNorm(nn.BatchNorm1d):
    """BatchNorm1d over the feature matrix (torchsparse/nn/modules/norm.py:15-17)."""

    def forward(self, input: SparseTensor) -> SparseTensor:
        return fapply(input, super().forward)


class InstanceNorm(nn.InstanceNorm1d):
    def forward(self, input: SparseTensor) -> SparseTensor:
        return fapply(input, super().forward)


class GroupNorm(nn.GroupNorm):
    """Group normalisation per batch sample (torchsparse/nn/modules/norm.py:25-57): the rows of every sample are
    normalised on their own, as ``nn.GroupNorm`` does for one [1, C, rows] input."""

    def forward(self, input: SparseTensor) -> SparseTensor:
        coords, feats = input.coords, input.feats
        batch_size = int(torch.max(coords[:, 0]).item()) + 1 if coords.shape[0] else 0
        num_channels = feats.shape[1]
        nfeats = torch.zeros_like(feats)
        for k in range(batch_size):
            rows = coords[:, 0] == k
            sample = feats[rows].transpose(0, 1).reshape(1, num_channels, -1)
            sample = super().forward(sample)
            nfeats[rows] = sample.reshape(num_channels, -1).transpose(0, 1)
        output = SparseTensor(nfeats, coords, input.stride, spatial_range=input.spatial_range)
        output._caches = input._caches
        return output
