"""``conv3d``: dataflow choice, kernel-map cache, native forward, output wrapping
(torchsparse/nn/functional/conv/conv.py:15-210)."""
from typing import Dict, List, Optional, Tuple, Union

import torch

from ....tensor import SparseTensor
from ....utils.utils import make_ntuple
from . import conv_config as cc
from .conv_config import Dataflow
from .conv_mode import get_conv_mode
from .func import (FetchOnDemandConvolutionFuntion, GatherScatterConvolutionFuntion,
                   ImplicitGEMMConvolutionFuntion)
from .kmap import build_kernel_map, transpose_kernel_map

__all__ = ["conv3d"]

_FUNCS = {
    Dataflow.ImplicitGEMM: ImplicitGEMMConvolutionFuntion,
    Dataflow.GatherScatter: GatherScatterConvolutionFuntion,
    Dataflow.FetchOnDemand: FetchOnDemandConvolutionFuntion,
}


def conv3d(
    input: SparseTensor,
    weight: torch.Tensor,
    kernel_size: Union[int, List[int], Tuple[int, ...]],
    bias: Optional[torch.Tensor] = None,
    stride: Union[int, List[int], Tuple[int, ...]] = 1,
    padding: Union[int, Tuple[int, ...]] = 0,
    dilation: Union[int, Tuple[int, ...]] = 1,
    config: Dict = None,
    transposed: bool = False,
    generative: bool = False,
    training: bool = False,
) -> SparseTensor:
    feats, coords = input.feats, input.coords
    kernel_size = make_ntuple(kernel_size, ndim=3)
    stride = make_ntuple(stride, ndim=3)
    dilation = make_ntuple(dilation, ndim=3)
    if config is None:
        config = cc.get_global_conv_config()
        if config is None:
            config = cc.get_default_conv_config(conv_mode=get_conv_mode(), training=training)
    dataflow = config["dataflow"]
    if dataflow == Dataflow.CodedCSR:
        raise AssertionError("CodedCSR has not been integrated.")
    if dataflow not in _FUNCS:
        raise ValueError("unsupported dataflow: {}".format(dataflow))
    if dataflow != Dataflow.ImplicitGEMM and config["ifsort"]:
        config = config.copy() if hasattr(config, "copy") else dict(config)
        config["ifsort"] = False  # row sorting only exists for the implicit-GEMM dataflow
    fn = _FUNCS[dataflow]
    caches = input._caches
    # the input's own coordinates are the target of a later transposed conv back to this stride
    caches.cmaps.setdefault(input.stride, (coords, input.spatial_range))

    if kernel_size == (1, 1, 1) and stride == (1, 1, 1) and dilation == (1, 1, 1):
        out_feats = feats.matmul(weight.to(feats.dtype))
        if bias is not None:
            out_feats += bias
        output = SparseTensor(coords=coords, feats=out_feats, stride=input.stride, spatial_range=input.spatial_range)
    elif not transposed:
        key = (input.stride, kernel_size, stride, dilation)
        kmap = caches.kmaps.get(key)
        out_stride = tuple(input.stride[k] * stride[k] for k in range(3))
        if kmap is not None and not _kmap_serves(kmap, config):
            kmap = None
        if kmap is None:
            subm = not any(s > 1 for s in stride)
            hashmap = caches.hashmaps.get(input.stride) if subm else None
            keys, vals = hashmap if hashmap is not None else (None, None)
            kmap = build_kernel_map(
                coords, feats.shape[0], kernel_size, stride, padding, keys, vals, input.spatial_range,
                config["kmap_mode"], dataflow, downsample_mode=config["downsample_mode"], training=training,
                ifsort=config["ifsort"], split_mask_num=config["split_mask_num"],
                split_mask_num_bwd=config["split_mask_num_bwd"], caches=caches, tensor_stride=input.stride)
            kmap["_dataflow"], kmap["_ifsort"], kmap["_split"] = dataflow, config["ifsort"], config["split_mask_num"]
            caches.kmaps[key] = kmap
            ts = kmap["table_stride"]
            caches.hashmaps[ts] = (kmap["hashmap_keys"], kmap["hashmap_vals"])
            caches.hash_bounds[ts] = kmap["table_bounds"]
            if "out_bounds" in kmap:
                caches.cbounds.setdefault(out_stride, kmap["out_bounds"])
        out_feats = fn.apply(feats, weight, kmap, config, False)
        if bias is not None:
            out_feats += bias
        output = SparseTensor(coords=kmap["coords"], feats=out_feats, stride=out_stride,
                              spatial_range=kmap["spatial_range"])
    else:
        if generative:
            raise NotImplementedError("generative transposed convolution is not built")
        tensor_stride = tuple(input.stride[k] // stride[k] for k in range(3))
        kmap = caches.kmaps.get((tensor_stride, kernel_size, stride, dilation))
        kmap = transpose_kernel_map(kmap, config["ifsort"], training=training,
                                    split_mask_num=config["split_mask_num"],
                                    split_mask_num_bwd=config["split_mask_num_bwd"])
        if dataflow != Dataflow.ImplicitGEMM and kmap.get("nbmaps") is None:
            raise ValueError("the cached kernel map was built for another dataflow")
        out_feats = fn.apply(feats, weight, kmap, config, True)
        if bias is not None:
            out_feats += bias
        cmap = caches.cmaps[tensor_stride]
        output = SparseTensor(coords=cmap[0], feats=out_feats, stride=tensor_stride, spatial_range=cmap[1])

    output._caches = caches
    caches.cmaps.setdefault(output.stride, (output.coords, output.spatial_range))
    return output


def _kmap_serves(kmap: Dict, config: Dict) -> bool:
    """A cached map can be reused when it holds what this config's dataflow reads."""
    df = config["dataflow"]
    if df == Dataflow.ImplicitGEMM:
        if not config["ifsort"]:
            return True
        return kmap.get("reorder_out_in_map") is not None and kmap.get("_split") == config["split_mask_num"]
    return kmap.get("_dataflow") == df
