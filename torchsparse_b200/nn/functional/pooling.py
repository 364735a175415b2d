"""Global pooling over the voxels of each batch element
(torchsparse/nn/functional/pooling.py:8-27)."""
import torch

from ...tensor import SparseTensor

__all__ = ["global_avg_pool", "global_max_pool"]


def _batch_reduce(inputs: SparseTensor, reduce: str) -> torch.Tensor:
    feats, batch = inputs.feats, inputs.coords[:, 0].long()
    n_batch = int(batch.max().item()) + 1 if batch.numel() else 0
    out = torch.zeros((n_batch, feats.shape[1]), dtype=feats.dtype, device=feats.device)
    index = batch.unsqueeze(1).expand(-1, feats.shape[1])
    # include_self=False: a batch element's row is the reduction of its own voxels only
    return out.scatter_reduce(0, index, feats, reduce=reduce, include_self=False)


def global_avg_pool(inputs: SparseTensor) -> torch.Tensor:
    """[B, C]: mean of the features of every batch element (one scatter instead of a loop over the batch)."""
    return _batch_reduce(inputs, "mean")


def global_max_pool(inputs: SparseTensor) -> torch.Tensor:
    """[B, C]: per-channel maximum over the voxels of every batch element."""
    return _batch_reduce(inputs, "amax")
