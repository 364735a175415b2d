"""The cache a network's layers share (torchsparse/utils/tensor_cache.py:6-60): coordinate maps,
kernel maps and hash tables, keyed by tensor stride — plus the host-side coordinate bounds this
implementation keeps so that kernel-map builds need no device read of ``coords.max``.

Two modes, as in the reference: every new SparseTensor starts its own cache (default), or all
tensors share one process-wide cache until it is cleared."""
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, Optional, Tuple

__all__ = ["TensorCache", "TensorCacheMode", "set_tensor_cache_mode", "get_tensor_cache_mode",
           "get_global_tensor_cache", "set_global_tensor_cache", "clear_global_tensor_cache",
           "cache_for_new_tensor"]

Stride = Tuple[int, ...]
Bounds = Tuple[Tuple[int, ...], Tuple[int, ...]]


@dataclass
class TensorCache:
    cmaps: Dict[Stride, Tuple[Any, Any]] = field(default_factory=dict)       # stride -> (coords, spatial_range)
    kmaps: Dict[Tuple[Any, ...], Any] = field(default_factory=dict)          # (stride, kernel, conv stride, dilation) -> kmap
    hashmaps: Dict[Stride, Tuple[Any, ...]] = field(default_factory=dict)    # stride of the coords held -> (keys, vals)
    cbounds: Dict[Stride, Bounds] = field(default_factory=dict)              # host copy of the actual (min, max)
    hash_bounds: Dict[Stride, Any] = field(default_factory=dict)             # key space of the table at that stride


class TensorCacheMode(Enum):
    SEPARATE_TENSOR_CACHE = 0
    GLOBAL_TENSOR_CACHE = 1


_state: Dict[str, Any] = {"mode": TensorCacheMode.SEPARATE_TENSOR_CACHE, "shared": None}


def get_tensor_cache_mode() -> TensorCacheMode:
    return _state["mode"]


def set_tensor_cache_mode(mode: TensorCacheMode) -> None:
    if not isinstance(mode, TensorCacheMode):
        raise AssertionError("Input must be an instance of TensorCacheMode")
    _state["mode"] = mode


def get_global_tensor_cache() -> Optional[TensorCache]:
    return _state["shared"]


def set_global_tensor_cache(tensor_cache: Optional[TensorCache]) -> None:
    _state["shared"] = tensor_cache


def clear_global_tensor_cache() -> None:
    _state["shared"] = None


def cache_for_new_tensor() -> TensorCache:
    """The cache a freshly constructed SparseTensor gets under the current mode."""
    if _state["mode"] is TensorCacheMode.GLOBAL_TENSOR_CACHE:
        if _state["shared"] is None:
            _state["shared"] = TensorCache()
        return _state["shared"]
    return TensorCache()
