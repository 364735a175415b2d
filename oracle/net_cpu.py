"""CPU execution of a whole sparse network (TEST INFRASTRUCTURE ONLY).

Runs the package's own nn.Modules on CPU tensors by swapping the ``conv3d`` the Conv3d module
calls for a CPU implementation made of the oracle kernel maps (oracle/kmap_oracle.py) and the
reference project's own CPU convolution (oracle/_ref, compiled from
torchsparse/backend/convolution/convolution_gather_scatter_cpu.cpp), falling back to the numpy
restatement of the same gather-matmul-scatter when that build is absent.  The flow mirrors the
reference's CPU path: GatherScatterConvolutionFuntion.forward with CPU tensors
(torchsparse/nn/functional/conv/func/gather_scatter.py:52-85) under conv3d
(torchsparse/nn/functional/conv/conv.py:15-210).

Used as the network-level checker in tests and as the timed CPU baseline of the benchmark.
"""
from __future__ import annotations

import contextlib
import os

import numpy as np
import torch

from . import kmap_oracle as ko

_ref = None


def reference_conv_module():
    """The compiled reference CPU extension, or None."""
    global _ref
    if _ref is None:
        try:
            from . import build_ref
            _ref = build_ref.load()
        except Exception:
            _ref = False
    return _ref or None


def _conv_pairs(feats: torch.Tensor, weight: torch.Tensor, nbmaps, nbsizes, n_out: int, transpose: bool):
    ref = reference_conv_module()
    if ref is not None:
        out = torch.zeros(n_out, weight.shape[-1], dtype=torch.float32)
        ref.conv_forward_gather_scatter_cpu(feats.contiguous(), out, weight.contiguous(),
                                            torch.from_numpy(nbmaps), torch.from_numpy(nbsizes), transpose)
        return out
    y = ko.conv_from_pairs(feats.numpy(), weight.numpy(), nbmaps, nbsizes, n_out, transpose, dtype=np.float32)
    return torch.from_numpy(y)


def conv3d_cpu(input, weight, kernel_size, bias=None, stride=1, padding=0, dilation=1, config=None,
               transposed=False, generative=False, training=False):
    from torchsparse_b200.tensor import SparseTensor
    from torchsparse_b200.utils.utils import make_ntuple

    ks, st = make_ntuple(kernel_size, 3), make_ntuple(stride, 3)
    pd = make_ntuple(padding, 3)
    feats = input.feats.float()
    weight = weight.detach().float()
    caches = input._caches
    caches.cmaps.setdefault(input.stride, (input.coords, input.spatial_range))
    if ks == (1, 1, 1) and st == (1, 1, 1):
        out = feats @ weight
        res = SparseTensor(out if bias is None else out + bias.float(), input.coords, input.stride, input.spatial_range)
    elif not transposed:
        key = (input.stride, ks, st, (1, 1, 1))
        km = caches.kmaps.get(key)
        if km is None:
            km = ko.build_kmap(input.coords.numpy(), ks, st, pd, input.spatial_range)
            km["nbmaps"], km["nbsizes"] = ko.pairs_from_map(km["out_in_map"])
            km["coords_t"] = torch.from_numpy(np.ascontiguousarray(km["coords"]))
            caches.kmaps[key] = km
        out = _conv_pairs(feats, weight, km["nbmaps"], km["nbsizes"], km["sizes"][1], False)
        if bias is not None:
            out = out + bias.float()
        res = SparseTensor(out, km["coords_t"], tuple(input.stride[i] * st[i] for i in range(3)), km["spatial_range"])
    else:
        fine = tuple(input.stride[i] // st[i] for i in range(3))
        km = caches.kmaps[(fine, ks, st, (1, 1, 1))]
        out = _conv_pairs(feats, weight, km["nbmaps"], km["nbsizes"], km["sizes"][0], True)
        if bias is not None:
            out = out + bias.float()
        cm = caches.cmaps[fine]
        res = SparseTensor(out, cm[0], fine, cm[1])
    res._caches = caches
    caches.cmaps.setdefault(res.stride, (res.coords, res.spatial_range))
    return res


@contextlib.contextmanager
def cpu_conv():
    """Inside this context the package's Conv3d modules evaluate on CPU through the oracle."""
    from torchsparse_b200.nn.modules import conv as conv_mod

    class _F:
        conv3d = staticmethod(conv3d_cpu)

    saved = conv_mod.F
    conv_mod.F = _F
    try:
        yield
    finally:
        conv_mod.F = saved


def forward_cpu(model: torch.nn.Module, coords: np.ndarray, feats: np.ndarray, threads: int | None = None):
    """Evaluate `model` (a copy, fp32, eval) on CPU.  Returns the model's output (SparseTensor or list)."""
    import copy

    from torchsparse_b200.tensor import SparseTensor

    if threads:
        torch.set_num_threads(threads)
    m = copy.deepcopy(model).float().cpu().eval()
    x = SparseTensor(torch.from_numpy(np.asarray(feats, dtype=np.float32)), torch.from_numpy(coords.astype(np.int32)))
    with torch.no_grad(), cpu_conv():
        return m(x)


def host_threads() -> int:
    return int(os.environ.get("OMP_NUM_THREADS", 0)) or (os.cpu_count() or 1)
