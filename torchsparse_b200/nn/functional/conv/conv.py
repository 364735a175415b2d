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

__all__ = ["conv3d", "acquire_kernel_map", "resolve_config"]

_FUNCS = {
    Dataflow.ImplicitGEMM: ImplicitGEMMConvolutionFuntion,
    Dataflow.GatherScatter: GatherScatterConvolutionFuntion,
    Dataflow.FetchOnDemand: FetchOnDemandConvolutionFuntion,
}

# When set to a list, every strided kernel-map build appends (tensor stride, kernel, stride, padding)
# to it: the inference engine uses the record of a first forward to build those maps up front later.
strided_build_log: Optional[list] = None


def resolve_config(config: Optional[Dict], training: bool = False) -> Dict:
    """Per-layer config > global config > defaults under the global conv mode
    (torchsparse/nn/functional/conv/conv.py:36-42)."""
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
    return config


def _kmap_serves(kmap: Dict, config: Dict) -> bool:
    """A cached map can be reused when it holds what this config's dataflow reads."""
    df = config["dataflow"]
    if df == Dataflow.ImplicitGEMM:
        if not config["ifsort"]:
            return True
        return kmap.get("reorder_out_in_map") is not None and kmap.get("_split") == config["split_mask_num"]
    return kmap.get("_dataflow") == df


def acquire_kernel_map(caches, coords: torch.Tensor, n_rows: int, tensor_stride, spatial_range, kernel_size, stride,
                       padding, dilation, config: Dict, training: bool = False) -> Dict:
    """The kernel map of a (non-transposed) conv on the tensor at `tensor_stride`: looked up in the
    cache, else built and registered together with its hash table and bounds."""
    global strided_build_log
    key = (tensor_stride, kernel_size, stride, dilation)
    kmap = caches.kmaps.get(key)
    if kmap is not None and _kmap_serves(kmap, config):
        return kmap
    subm = not any(s > 1 for s in stride)
    hashmap = caches.hashmaps.get(tensor_stride) if subm else None
    keys, vals = hashmap if hashmap is not None else (None, None)
    kmap = build_kernel_map(
        coords, n_rows, kernel_size, stride, padding, keys, vals, spatial_range, config["kmap_mode"],
        config["dataflow"], downsample_mode=config["downsample_mode"], training=training, ifsort=config["ifsort"],
        split_mask_num=config["split_mask_num"], split_mask_num_bwd=config["split_mask_num_bwd"], caches=caches,
        tensor_stride=tensor_stride)
    kmap["_dataflow"], kmap["_ifsort"], kmap["_split"] = config["dataflow"], config["ifsort"], config["split_mask_num"]
    caches.kmaps[key] = kmap
    ts = kmap["table_stride"]
    caches.hashmaps[ts] = (kmap["hashmap_keys"], kmap["hashmap_vals"])
    caches.hash_bounds[ts] = kmap["table_bounds"]
    if not subm:
        out_stride = tuple(tensor_stride[k] * stride[k] for k in range(3))
        if "out_bounds" in kmap:
            caches.cbounds.setdefault(out_stride, kmap["out_bounds"])
        caches.cmaps.setdefault(out_stride, (kmap["coords"], kmap["spatial_range"]))
        if strided_build_log is not None:
            strided_build_log.append((tensor_stride, kernel_size, stride, padding, dilation))
    return kmap


def _apply(fn, feats, weight, kmap, config, transposed, epilogue):
    # outside autograd (inference) the Function wrapper is pure overhead
    if torch.is_grad_enabled() and (feats.requires_grad or weight.requires_grad):
        return fn.apply(feats, weight, kmap, config, transposed, epilogue)
    return fn.forward(None, feats, weight, kmap, config, transposed, epilogue)


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
    epilogue: Optional[Dict] = None,
) -> SparseTensor:
    """Sparse convolution.  ``epilogue`` (not in the reference) is an optional dict with any of
    ``scale`` / ``bias`` (fp32 [Cout]), ``residual`` ([M, Cout]) and ``relu``: applied to the fp32
    accumulator inside the implicit-GEMM kernel, y = relu(acc * scale + bias + residual); for the
    other dataflows and for 1x1x1 kernels the same arithmetic is done with torch ops."""
    feats, coords = input.feats, input.coords
    kernel_size = make_ntuple(kernel_size, ndim=3)
    stride = make_ntuple(stride, ndim=3)
    dilation = make_ntuple(dilation, ndim=3)
    config = resolve_config(config, training)
    dataflow = config["dataflow"]
    fn = _FUNCS[dataflow]
    caches = input._caches
    # the input's own coordinates are the target of a later transposed conv back to this stride
    caches.cmaps.setdefault(input.stride, (coords, input.spatial_range))
    fused = epilogue is not None and dataflow == Dataflow.ImplicitGEMM
    if fused and torch.is_grad_enabled():
        # the kernel's epilogue has no backward: under autograd the same arithmetic runs as torch ops
        res = epilogue.get("residual")
        if feats.requires_grad or weight.requires_grad or (res is not None and res.requires_grad):
            fused = False

    if kernel_size == (1, 1, 1) and stride == (1, 1, 1) and dilation == (1, 1, 1):
        out_feats = feats.matmul(weight.to(feats.dtype))
        fused = False
        out_coords, out_stride, out_range = coords, input.stride, input.spatial_range
    elif not transposed:
        padding = make_ntuple(padding, ndim=3)
        kmap = acquire_kernel_map(caches, coords, feats.shape[0], input.stride, input.spatial_range, kernel_size,
                                  stride, padding, dilation, config, training)
        out_feats = _apply(fn, feats, weight, kmap, config, False, epilogue if fused else None)
        out_coords = kmap["coords"]
        out_stride = tuple(input.stride[k] * stride[k] for k in range(3))
        out_range = kmap["spatial_range"]
    else:
        tensor_stride = tuple(input.stride[k] // stride[k] for k in range(3))
        if generative:
            # new coordinates are generated from the inputs; the map is built afresh (no table is reused) and the
            # convolution runs as a plain (not transposed) one on it
            # (torchsparse/nn/functional/conv/conv.py:161-203)
            from .kmap import build_kernel_map
            padding = make_ntuple(padding, ndim=3)
            kmap = build_kernel_map(coords, feats.shape[0], kernel_size, stride, padding, None, None,
                                    input.spatial_range, config["kmap_mode"], dataflow,
                                    downsample_mode=config["downsample_mode"], training=training,
                                    ifsort=config["ifsort"], generative=True)
            out_feats = _apply(fn, feats, weight, kmap, config, False, epilogue if fused else None)
            caches.cmaps[tensor_stride] = (kmap["coords"], kmap.get("spatial_range"))
            out_coords, out_range = caches.cmaps[tensor_stride]
            out_stride = tensor_stride
            caches.kmaps = dict()
            caches.hashmaps = dict()
        else:
            kmap = caches.kmaps.get((tensor_stride, kernel_size, stride, dilation))
            kmap = transpose_kernel_map(kmap, config["ifsort"], training=training,
                                        split_mask_num=config["split_mask_num"],
                                        split_mask_num_bwd=config["split_mask_num_bwd"])
            if dataflow != Dataflow.ImplicitGEMM and kmap.get("nbmaps") is None:
                raise ValueError("the cached kernel map was built for another dataflow")
            out_feats = _apply(fn, feats, weight, kmap, config, True, epilogue if fused else None)
            out_coords, out_range = caches.cmaps[tensor_stride]
            out_stride = tensor_stride

    if bias is not None:
        out_feats += bias
    if epilogue is not None and not fused:
        out_feats = _epilogue_torch(out_feats, epilogue)
    output = SparseTensor._from_parts(out_feats, out_coords, out_stride, out_range, caches)
    caches.cmaps.setdefault(out_stride, (out_coords, out_range))
    return output


def _epilogue_torch(x: torch.Tensor, epilogue: Dict) -> torch.Tensor:
    dtype = x.dtype
    scale, bias, residual = epilogue.get("scale"), epilogue.get("bias"), epilogue.get("residual")
    if scale is not None or bias is not None:
        x = x.float()
        if scale is not None:
            x = x * scale
        if bias is not None:
            x = x + bias
    if residual is not None:
        x = x + residual
    if epilogue.get("relu"):
        x = torch.relu(x)
    return x.to(dtype)
