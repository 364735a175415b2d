"""The two tensor containers of the reference's Python surface (torchsparse/tensor.py:29-145).

``SparseTensor`` = features [N, C] + int32 coordinates [N, 4] in (batch, x, y, z) order + the tensor
stride + an optional spatial range, carrying the cache of coordinate maps, kernel maps and hash
tables that the layers of a network share.  ``PointTensor`` = point features with float coordinates
and the voxel queries cached for them."""
from typing import Callable, Optional, Sequence, Tuple, Union

import torch

from .utils.tensor_cache import TensorCache, TensorCacheMode, cache_for_new_tensor
from .utils.to_dense import to_dense
from .utils.utils import make_ntuple

__all__ = ["SparseTensor", "CatSparseTensor", "PointTensor", "get_allow_negative_coordinates",
           "set_allow_negative_coordinates"]

_negative_coordinates = {"allowed": False}


def set_allow_negative_coordinates(allow_negative_coordinates: bool) -> None:
    """When on, kernel-map keys start at the smallest coordinate instead of 0."""
    _negative_coordinates["allowed"] = bool(allow_negative_coordinates)


def get_allow_negative_coordinates() -> bool:
    return _negative_coordinates["allowed"]


class _Alias:
    """Short attribute name of the reference (``F``, ``C``, ``s``) for a field of this class."""

    def __init__(self, field: str, convert: Optional[Callable] = None) -> None:
        self.field, self.convert = field, convert

    def __get__(self, obj, owner=None):
        return self if obj is None else getattr(obj, self.field)

    def __set__(self, obj, value) -> None:
        setattr(obj, self.field, self.convert(value) if self.convert else value)


class SparseTensor:
    F = _Alias("feats")
    C = _Alias("coords")
    s = _Alias("stride", lambda v: make_ntuple(v, ndim=3))

    def __init__(self, feats: torch.Tensor, coords: torch.Tensor, stride: Union[int, Tuple[int, ...]] = 1,
                 spatial_range: Optional[Sequence[int]] = None, coord_bounds=None) -> None:
        """``coord_bounds`` = ((min b, x, y, z), (max b, x, y, z)) when the caller already knows them on
        the host (``sparse_quantize`` returns them): kernel-map builds then need no device reduction."""
        self.feats, self.coords = feats, coords
        self.stride = make_ntuple(stride, ndim=3)
        self.spatial_range = None if spatial_range is None else make_ntuple(spatial_range, ndim=len(spatial_range))
        self._caches = cache_for_new_tensor()
        if coord_bounds is not None:
            lo, hi = coord_bounds
            self._caches.cbounds[self.stride] = (tuple(int(v) for v in lo), tuple(int(v) for v in hi))

    @classmethod
    def _from_parts(cls, feats: torch.Tensor, coords: torch.Tensor, stride: Tuple[int, ...], spatial_range,
                    caches: TensorCache) -> "SparseTensor":
        """The output of a layer: stride and range are already canonical tuples and the cache is the
        input's, so nothing is validated or created."""
        out = cls.__new__(cls)
        out.feats, out.coords, out.stride, out.spatial_range, out._caches = feats, coords, stride, spatial_range, caches
        return out

    # ---- in-place movers (each returns self, as the reference's do)
    def _apply(self, fn: Callable[[torch.Tensor], torch.Tensor], coords_too: bool = True) -> "SparseTensor":
        self.feats = fn(self.feats)
        if coords_too:
            self.coords = fn(self.coords)
        return self

    def cpu(self) -> "SparseTensor":
        return self._apply(torch.Tensor.cpu)

    def cuda(self) -> "SparseTensor":
        return self._apply(torch.Tensor.cuda)

    def detach(self) -> "SparseTensor":
        return self._apply(torch.Tensor.detach)

    def half(self) -> "SparseTensor":
        return self._apply(torch.Tensor.half, coords_too=False)

    def to(self, device, non_blocking: bool = True) -> "SparseTensor":
        return self._apply(lambda t: t.to(device, non_blocking=non_blocking))

    def dense(self) -> torch.Tensor:
        if self.spatial_range is None:
            raise AssertionError("dense() needs a spatial_range")
        return to_dense(self.feats, self.coords, self.spatial_range)

    def __add__(self, other: "SparseTensor") -> "SparseTensor":
        return SparseTensor._from_parts(self.feats + other.feats, self.coords, self.stride, self.spatial_range,
                                        self._caches)


class CatSparseTensor(SparseTensor):
    """A channel concatenation of tensors on the same coordinates that is not written out: ``parts`` holds
    the feature matrices, and ``feats`` concatenates them the first time something asks for it.  Layers
    that can read their input from two matrices (the fused convolutions) take ``parts`` directly."""

    def __init__(self, parts, coords, stride, spatial_range, caches) -> None:
        self.parts = tuple(parts)
        self._feats = None
        self.coords, self.stride, self.spatial_range, self._caches = coords, stride, spatial_range, caches

    @property
    def feats(self) -> torch.Tensor:
        if self._feats is None:
            self._feats = torch.cat(self.parts, dim=1)
        return self._feats

    @feats.setter
    def feats(self, value: torch.Tensor) -> None:
        self._feats, self.parts = value, (value,)


class PointTensor:
    def __init__(self, feats, coords, idx_query=None, weights=None):
        self.F, self.C = feats, coords
        self.idx_query = {} if idx_query is None else idx_query
        self.weights = {} if weights is None else weights
        self.additional_features = {"idx_query": {}, "counts": {}}

    def _apply(self, fn) -> "PointTensor":
        self.F, self.C = fn(self.F), fn(self.C)
        return self

    def cuda(self) -> "PointTensor":
        return self._apply(torch.Tensor.cuda)

    def detach(self) -> "PointTensor":
        return self._apply(torch.Tensor.detach)

    def to(self, device, non_blocking: bool = True) -> "PointTensor":
        return self._apply(lambda t: t.to(device, non_blocking=non_blocking))

    def __add__(self, other: "PointTensor") -> "PointTensor":
        out = PointTensor(self.F + other.F, self.C, self.idx_query, self.weights)
        out.additional_features = self.additional_features
        return out
