"""Convolution configuration: dataflow, sorting, mask splits
(torchsparse/nn/functional/conv/conv_config.py:7-94)."""
from enum import Enum

from .conv_mode import ConvMode

__all__ = ["Dataflow", "ConvConfig", "get_default_conv_config", "get_global_conv_config", "set_global_conv_config",
           "clear_global_conv_config"]


class Dataflow(Enum):
    ImplicitGEMM = 0
    GatherScatter = 1
    FetchOnDemand = 2
    CodedCSR = 3


class ConvConfig(dict):
    """A dict whose items are also attributes (``cfg.dataflow`` / ``cfg["dataflow"]``)."""

    def __getattr__(self, name):
        try:
            return self[name]
        except KeyError:
            raise AttributeError(name) from None

    def __setattr__(self, name, value):
        self[name] = value

    def copy(self):
        return ConvConfig(self)


_DEFAULTS = (
    ("dataflow", Dataflow.ImplicitGEMM),
    ("ifsort", False),
    ("kmap_mode", "hashmap_on_the_fly"),
    ("downsample_mode", "spconv"),
    ("split_mask_num", 1),
    ("split_mask_num_bwd", 3),
    ("epsilon", 0.0),
    ("mm_thresh", 0),
    ("FOD_fusion", True),
)

_global_conv_config = None


def keys_check(conv_config) -> None:
    missing = [k for k, _ in _DEFAULTS if k not in conv_config]
    for k, v in _DEFAULTS:
        conv_config.setdefault(k, v)
    if missing:
        print("Warning: Missing fields for ConvConfig. Use default configs for these fields.")


def get_global_conv_config():
    return _global_conv_config


def set_global_conv_config(conv_config):
    global _global_conv_config
    keys_check(conv_config)
    _global_conv_config = conv_config


def clear_global_conv_config():
    global _global_conv_config
    _global_conv_config = None


def get_default_conv_config(conv_mode: ConvMode = ConvMode.mode0, training: bool = False):
    """A fresh config per call (the reference hands out one shared object that conv3d then
    mutates, so a GatherScatter call changes the defaults of later calls)."""
    config = ConvConfig(_DEFAULTS)
    if conv_mode == ConvMode.mode1:
        config.ifsort = True
    elif conv_mode == ConvMode.mode2:
        config.ifsort = True
        config.split_mask_num = 3
    return config
