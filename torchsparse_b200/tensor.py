from typing import Tuple, Union

import torch

from .utils.utils import make_ntuple
from .utils.to_dense import to_dense
from .utils.tensor_cache import (TensorCache, TensorCacheMode, get_global_tensor_cache, set_global_tensor_cache,
                                 get_tensor_cache_mode)

__all__ = ["SparseTensor", "PointTensor", "get_allow_negative_coordinates", "set_allow_negative_coordinates"]

_allow_negative_coordinates = False


def get_allow_negative_coordinates():
    return _allow_negative_coordinates


def set_allow_negative_coordinates(allow_negative_coordinates):
    global _allow_negative_coordinates
    _allow_negative_coordinates = allow_negative_coordinates


class SparseTensor:
    """feats [N,C] + coords int32 [N,4] = (batch,x,y,z) + tensor stride + optional spatial range,
    with a cache of kernel maps shared along the network (torchsparse/tensor.py:29-114)."""

    def __init__(self, feats: torch.Tensor, coords: torch.Tensor, stride: Union[int, Tuple[int, ...]] = 1,
                 spatial_range: Union[int, Tuple[int, ...]] = None, coord_bounds=None) -> None:
        self.feats = feats
        self.coords = coords
        self.stride = make_ntuple(stride, ndim=3)
        self.spatial_range = None if spatial_range is None else make_ntuple(spatial_range, ndim=len(spatial_range))
        if get_tensor_cache_mode() == TensorCacheMode.GLOBAL_TENSOR_CACHE:
            caches = get_global_tensor_cache()
            if caches is None:
                caches = TensorCache()
                set_global_tensor_cache(caches)
            self._caches = caches
        else:
            self._caches = TensorCache()
        if coord_bounds is not None:
            # ((min b,x,y,z), (max b,x,y,z)) known on the host (e.g. from sparse_quantize): kernel-map
            # builds then need no device reduction of the coordinates
            self._caches.cbounds[self.stride] = (tuple(int(v) for v in coord_bounds[0]),
                                                 tuple(int(v) for v in coord_bounds[1]))

    @classmethod
    def _from_parts(cls, feats: torch.Tensor, coords: torch.Tensor, stride: Tuple[int, ...], spatial_range,
                    caches) -> "SparseTensor":
        """The output of a layer: stride and range are already canonical tuples and the cache is the
        input's, so nothing is validated or created."""
        self = cls.__new__(cls)
        self.feats, self.coords, self.stride, self.spatial_range, self._caches = (feats, coords, stride,
                                                                                 spatial_range, caches)
        return self

    @property
    def F(self) -> torch.Tensor:
        return self.feats

    @F.setter
    def F(self, feats: torch.Tensor) -> None:
        self.feats = feats

    @property
    def C(self) -> torch.Tensor:
        return self.coords

    @C.setter
    def C(self, coords: torch.Tensor) -> None:
        self.coords = coords

    @property
    def s(self) -> Tuple[int, ...]:
        return self.stride

    @s.setter
    def s(self, stride: Union[int, Tuple[int, ...]]) -> None:
        self.stride = make_ntuple(stride, ndim=3)

    def cpu(self):
        self.coords, self.feats = self.coords.cpu(), self.feats.cpu()
        return self

    def cuda(self):
        self.coords, self.feats = self.coords.cuda(), self.feats.cuda()
        return self

    def half(self):
        self.feats = self.feats.half()
        return self

    def detach(self):
        self.coords, self.feats = self.coords.detach(), self.feats.detach()
        return self

    def to(self, device, non_blocking: bool = True):
        self.coords = self.coords.to(device, non_blocking=non_blocking)
        self.feats = self.feats.to(device, non_blocking=non_blocking)
        return self

    def dense(self):
        assert self.spatial_range is not None
        return to_dense(self.feats, self.coords, self.spatial_range)

    def __add__(self, other):
        output = SparseTensor(coords=self.coords, feats=self.feats + other.feats, stride=self.stride,
                              spatial_range=self.spatial_range)
        output._caches = self._caches
        return output


class PointTensor:
    """Point features with float coordinates and cached voxel queries (torchsparse/tensor.py:116-145)."""

    def __init__(self, feats, coords, idx_query=None, weights=None):
        self.F = feats
        self.C = coords
        self.idx_query = idx_query if idx_query is not None else {}
        self.weights = weights if weights is not None else {}
        self.additional_features = {"idx_query": {}, "counts": {}}

    def cuda(self):
        self.F, self.C = self.F.cuda(), self.C.cuda()
        return self

    def detach(self):
        self.F, self.C = self.F.detach(), self.C.detach()
        return self

    def to(self, device, non_blocking=True):
        self.F = self.F.to(device, non_blocking=non_blocking)
        self.C = self.C.to(device, non_blocking=non_blocking)
        return self

    def __add__(self, other):
        tensor = PointTensor(self.F + other.F, self.C, self.idx_query, self.weights)
        tensor.additional_features = self.additional_features
        return tensor
