"""Per-network cache of coordinate maps, kernel maps and hash tables
(torchsparse/utils/tensor_cache.py:6-60), plus the host-side coordinate bounds this
implementation keeps so that kernel-map builds need no device read of ``coords.max``."""
from enum import Enum
from typing import Any, Dict, Tuple

__all__ = ["TensorCache", "TensorCacheMode", "set_tensor_cache_mode", "get_tensor_cache_mode",
           "get_global_tensor_cache", "set_global_tensor_cache", "clear_global_tensor_cache"]


class TensorCacheMode(Enum):
    SEPARATE_TENSOR_CACHE = 0
    GLOBAL_TENSOR_CACHE = 1


_tensor_cache_mode = TensorCacheMode.SEPARATE_TENSOR_CACHE
_global_tensor_cache = None


def set_tensor_cache_mode(mode: TensorCacheMode):
    assert isinstance(mode, TensorCacheMode), "Input must be an instance of TensorCacheMode"
    global _tensor_cache_mode
    _tensor_cache_mode = mode


def get_tensor_cache_mode() -> TensorCacheMode:
    return _tensor_cache_mode


class TensorCache:
    def __init__(self) -> None:
        self.cmaps: Dict[Tuple[int, ...], Tuple[Any, Any]] = {}   # stride -> (coords, spatial_range)
        self.kmaps: Dict[Tuple[Any, ...], Any] = {}               # (stride, kernel, conv stride, dilation) -> kmap
        self.hashmaps: Dict[Tuple[int, ...], Tuple[Any, ...]] = {}  # stride of the coords held -> (keys, vals)
        # host-side bounds, keyed by tensor stride
        self.cbounds: Dict[Tuple[int, ...], Tuple[Tuple[int, ...], Tuple[int, ...]]] = {}   # actual (min, max)
        self.hash_bounds: Dict[Tuple[int, ...], Tuple[Tuple[int, ...], Tuple[int, ...]]] = {}  # ravel bounds of the table


def get_global_tensor_cache():
    return _global_tensor_cache


def set_global_tensor_cache(tensor_cache):
    global _global_tensor_cache
    _global_tensor_cache = tensor_cache


def clear_global_tensor_cache():
    global _global_tensor_cache
    _global_tensor_cache = None
