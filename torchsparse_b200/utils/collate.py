"""Batching of scans (torchsparse/utils/collate.py:11-54)."""
from typing import Any, List

import numpy as np
import torch

from ..tensor import SparseTensor

__all__ = ["sparse_collate", "sparse_collate_fn"]


def _as_tensor(value, what: str) -> torch.Tensor:
    if isinstance(value, np.ndarray):
        return torch.tensor(value)
    if not isinstance(value, torch.Tensor):
        raise AssertionError(f"{what} must be a tensor or an array, got {type(value)}")
    return value


def sparse_collate(inputs: List[SparseTensor]) -> SparseTensor:
    """One batch from per-scan tensors with [N_i, 3] coordinates: scan i's rows get the batch index i
    in a new first column; features are concatenated in the same order.  All scans share a stride."""
    stride = inputs[0].stride
    rows, feats = [], []
    for index, scan in enumerate(inputs):
        scan.coords, scan.feats = _as_tensor(scan.coords, "coords"), _as_tensor(scan.feats, "feats")
        if scan.stride != stride:
            raise AssertionError((scan.stride, stride))
        xyz = scan.coords.int()
        rows.append(torch.cat([xyz.new_full((xyz.shape[0], 1), index), xyz], dim=1))
        feats.append(scan.feats)
    return SparseTensor(torch.cat(feats, dim=0), torch.cat(rows, dim=0), stride)


def sparse_collate_fn(inputs: List[Any]) -> Any:
    """``collate_fn`` for a DataLoader of dicts: nested dicts recurse, SparseTensors are batched, arrays and
    tensors are stacked, anything else stays a list; a list of non-dicts is returned as it is."""
    head = inputs[0]
    if not isinstance(head, dict):
        return inputs
    merged = {}
    for key, sample in head.items():
        column = [item[key] for item in inputs]
        if isinstance(sample, dict):
            merged[key] = sparse_collate_fn(column)
        elif isinstance(sample, SparseTensor):
            merged[key] = sparse_collate(column)
        elif isinstance(sample, np.ndarray):
            merged[key] = torch.stack([torch.tensor(v) for v in column], dim=0)
        elif isinstance(sample, torch.Tensor):
            merged[key] = torch.stack(column, dim=0)
        else:
            merged[key] = column
    return merged
