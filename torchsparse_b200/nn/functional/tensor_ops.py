"""Whole-tensor operators of the reference's functional namespace that need no kernel of their own:
batch-wise global pooling, the coordinate-box crop and feature-wise activations
(torchsparse/nn/functional/{pooling,crop,activation}.py)."""
from typing import Callable, Optional, Sequence

import torch
from torch.nn import functional as _tf

from ...tensor import SparseTensor
from ..utils.apply import fapply

__all__ = ["global_avg_pool", "global_max_pool", "spcrop", "relu", "silu", "leaky_relu"]


# ---------------------------------------------------------------------------------- pooling
def _pool_per_batch(x: SparseTensor, how: str) -> torch.Tensor:
    """[B, C] from [N, C]: one scatter-reduce keyed by the batch column instead of a loop over the
    batch with a boolean mask each; a row only reduces its own voxels (include_self=False)."""
    batch = x.coords[:, 0].long()
    rows = int(batch.max().item()) + 1 if batch.numel() else 0
    channels = x.feats.shape[1]
    out = x.feats.new_zeros((rows, channels))
    return out.scatter_reduce(0, batch[:, None].expand(-1, channels), x.feats, reduce=how, include_self=False)


def global_avg_pool(inputs: SparseTensor) -> torch.Tensor:
    """Mean feature vector of every batch element."""
    return _pool_per_batch(inputs, "mean")


def global_max_pool(inputs: SparseTensor) -> torch.Tensor:
    """Per-channel maximum over the voxels of every batch element."""
    return _pool_per_batch(inputs, "amax")


# ---------------------------------------------------------------------------------- crop
def spcrop(input: SparseTensor, coords_min: Optional[Sequence[int]] = None,
           coords_max: Optional[Sequence[int]] = None) -> SparseTensor:
    """Voxels inside the half-open box ``[coords_min, coords_max)``.

    As in the reference, the three bounds are compared with columns 0..2 of the coordinate rows; with
    the (batch, x, y, z) layout those are batch, x and y.  Callers of the reference rely on exactly
    that, so it is kept.  The result starts a kernel-map cache of its own."""
    head = input.coords[:, :3]
    inside = torch.ones(head.shape[0], dtype=torch.bool, device=head.device)
    for bound, accept in ((coords_min, torch.ge), (coords_max, torch.lt)):
        if bound is not None:
            inside &= accept(head, head.new_tensor(list(bound))).all(dim=1)
    return SparseTensor(input.feats[inside], input.coords[inside], input.stride)


# ---------------------------------------------------------------------------------- activations
def _on_feats(fn: Callable[..., torch.Tensor], name: str, **fixed):
    def op(input: SparseTensor, *args, inplace: bool = True, **kwargs) -> SparseTensor:
        return fapply(input, fn, *args, inplace=inplace, **{**fixed, **kwargs})

    op.__name__ = op.__qualname__ = name
    op.__doc__ = f"``{name}`` on the feature matrix; coordinates, stride and kernel-map cache are kept."
    return op


relu = _on_feats(_tf.relu, "relu")
silu = _on_feats(_tf.silu, "silu")
leaky_relu = _on_feats(_tf.leaky_relu, "leaky_relu", negative_slope=0.1)
