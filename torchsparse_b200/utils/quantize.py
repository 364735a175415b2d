from itertools import repeat
from typing import Tuple, Union

import numpy as np
import torch

__all__ = ["sparse_quantize"]


def sparse_quantize(coords, voxel_size: Union[float, Tuple[float, ...]] = 1, *, return_index: bool = False,
                    return_inverse: bool = False, return_bounds: bool = False):
    """Voxelise point coordinates and keep one entry per voxel, in ascending (x,y,z) order.

    Same contract as torchsparse/utils/quantize.py:24-48 (coords = floor(coords / voxel) as
    int32, ``indices`` = first occurrence of each voxel, ``inverse_indices`` = voxel of each
    point) but computed on the GPU: the input may be a CUDA tensor (results are CUDA
    tensors) or a numpy array / CPU tensor (copied to the current CUDA device, results
    returned as numpy arrays, as the reference returns).  ``return_bounds`` (not in the reference)
    appends ``((min x,y,z), (max x,y,z))`` of the voxel coordinates as host tuples: the count readback
    brings them along for free, and `SparseTensor(..., coord_bounds=...)` can use them to skip its own
    device reduction."""
    from .. import backend

    if isinstance(voxel_size, (float, int)):
        voxel_size = tuple(repeat(voxel_size, 3))
    assert isinstance(voxel_size, tuple) and len(voxel_size) == 3
    as_numpy = not (isinstance(coords, torch.Tensor) and coords.is_cuda)
    if as_numpy:
        arr = np.ascontiguousarray(np.asarray(coords.cpu() if isinstance(coords, torch.Tensor) else coords))
        if arr.dtype not in (np.float32, np.float64):
            arr = arr.astype(np.float64)
        t = torch.from_numpy(arr).cuda(non_blocking=True)
    else:
        t = coords
    vox, idx, inv, bounds = backend.quantize_unique_cuda(t, voxel_size, return_index, return_inverse)
    outs = [vox]
    if return_index:
        outs.append(idx)
    if return_inverse:
        outs.append(inv)
    if as_numpy:
        outs = [o.cpu().numpy() for o in outs]
    if return_bounds:
        outs.append(bounds)
    return outs[0] if len(outs) == 1 else outs
