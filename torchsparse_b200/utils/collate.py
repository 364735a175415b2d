from typing import Any, List

import numpy as np
import torch

from ..tensor import SparseTensor

__all__ = ["sparse_collate", "sparse_collate_fn"]


def sparse_collate(inputs: List[SparseTensor]) -> SparseTensor:
    """Concatenate scans into one batch, prepending the batch index column
    (torchsparse/utils/collate.py:11-33)."""
    coords, feats = [], []
    stride = inputs[0].stride
    for k, x in enumerate(inputs):
        if isinstance(x.coords, np.ndarray):
            x.coords = torch.tensor(x.coords)
        if isinstance(x.feats, np.ndarray):
            x.feats = torch.tensor(x.feats)
        assert isinstance(x.coords, torch.Tensor), type(x.coords)
        assert isinstance(x.feats, torch.Tensor), type(x.feats)
        assert x.stride == stride, (x.stride, stride)
        batch = torch.full((x.coords.shape[0], 1), k, device=x.coords.device, dtype=torch.int)
        coords.append(torch.cat((batch, x.coords.int()), dim=1))
        feats.append(x.feats)
    return SparseTensor(coords=torch.cat(coords, dim=0), feats=torch.cat(feats, dim=0), stride=stride)


def sparse_collate_fn(inputs: List[Any]) -> Any:
    """Dict-wise collation used as a DataLoader collate_fn (torchsparse/utils/collate.py:36-54)."""
    if not isinstance(inputs[0], dict):
        return inputs
    output = {}
    for name, first in inputs[0].items():
        vals = [inp[name] for inp in inputs]
        if isinstance(first, dict):
            output[name] = sparse_collate_fn(vals)
        elif isinstance(first, np.ndarray):
            output[name] = torch.stack([torch.tensor(v) for v in vals], dim=0)
        elif isinstance(first, torch.Tensor):
            output[name] = torch.stack(vals, dim=0)
        elif isinstance(first, SparseTensor):
            output[name] = sparse_collate(vals)
        else:
            output[name] = vals
    return output
