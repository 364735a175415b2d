"""Global convolution presets (torchsparse/nn/functional/conv/conv_mode.py)."""
from enum import Enum

__all__ = ["ConvMode", "get_conv_mode", "set_conv_mode", "get_kmap_mode", "set_kmap_mode", "get_downsample_mode",
           "set_downsample_mode"]

_global_kmap_mode = "hashmap_on_the_fly"
_global_downsample_mode = "spconv"


def get_kmap_mode():
    return _global_kmap_mode


def set_kmap_mode(kmap_mode: str):
    global _global_kmap_mode
    assert kmap_mode in ("hashmap_on_the_fly", "hashmap"), (
        f'Unsupport kmap_mode: {kmap_mode}. Please set kmap_mode to "hashmap_on_the_fly" or "hashmap".')
    _global_kmap_mode = kmap_mode


def get_downsample_mode():
    return _global_downsample_mode


def set_downsample_mode(downsample_mode: str):
    global _global_downsample_mode
    assert downsample_mode in ("spconv", "minkowski"), (
        f'Unsupport downsample_mode {downsample_mode}. Please set downsample_mode to "spconv" or "minkowski".')
    _global_downsample_mode = downsample_mode


class ConvMode(Enum):
    mode0 = 0  # unsorted forward
    mode1 = 1  # sorted forward, one mask split
    mode2 = 2  # sorted forward, three mask splits


_global_conv_mode = ConvMode.mode0


def get_conv_mode():
    return _global_conv_mode


def set_conv_mode(conv_mode):
    global _global_conv_mode
    if isinstance(conv_mode, int):
        assert conv_mode in (0, 1, 2), f"Undefined conv_mode:{conv_mode}"
        conv_mode = ConvMode(conv_mode)
    assert isinstance(conv_mode, ConvMode), "Unsupport conv_mode input type"
    _global_conv_mode = conv_mode
