from typing import Optional

import torch

from ... import backend

__all__ = ["sphash"]


def sphash(coords: torch.Tensor, offsets: Optional[torch.Tensor] = None) -> torch.Tensor:
    """64-bit FNV-1a hash of int32 (b,x,y,z) rows; with ``offsets`` [K,3] the hash of every
    shifted copy, shape [K,N] (torchsparse/nn/functional/hash.py:10-39)."""
    assert coords.dtype == torch.int, coords.dtype
    assert coords.ndim == 2 and coords.shape[1] == 4, coords.shape
    coords = coords.contiguous()
    if offsets is None:
        return backend.hash_cuda(coords)
    assert offsets.dtype == torch.int, offsets.dtype
    assert offsets.ndim == 2 and offsets.shape[1] == 3, offsets.shape
    return backend.kernel_hash_cuda(coords, offsets.contiguous())
