"""Inference-time fusion: conv + BatchNorm (stored statistics) + ReLU (+ residual add) become one
kernel launch, and the strided kernel maps of a network are built before its first convolution.

The reference runs BatchNorm, ReLU and the residual add as separate torch kernels over the feature
matrix after every convolution (torchsparse/nn/modules/norm.py:15-17, activation.py,
torchsparse/backbones/modules/blocks.py:53-85).  At batch 1 those launches cost more than the
convolutions, so `fuse_for_inference` rewrites a trained model:

* ``Conv3d -> BatchNorm [-> ReLU]`` inside any ``nn.Sequential``  ->  :class:`FusedConv`
  (BatchNorm folded into a per-channel fp32 scale and shift applied to the fp32 accumulator);
* ``SparseResBlock``  ->  :class:`FusedResBlock` (the shortcut is added and the final ReLU applied in
  the second convolution's epilogue).

The rewritten model computes the same function (one rounding instead of three per layer).
:class:`InferenceEngine` additionally remembers, from its first forward, which strided convolutions
the network runs and builds their kernel maps up front on later calls, so that the only
device-to-host reads of a forward (one per strided map) happen before the convolutions are queued.
"""
from typing import Optional

import torch
from torch import nn

from .. import backend, backends
from ..tensor import SparseTensor
from ..utils.utils import make_ntuple
from . import functional as F
from .functional.conv import conv as _conv_impl
from .modules.activation import ReLU
from .modules.conv import Conv3d

__all__ = ["FusedConv", "FusedResBlock", "fuse_for_inference", "InferenceEngine"]


def _fold_bn(conv: Conv3d, bn: Optional[nn.BatchNorm1d]):
    cout = conv.out_channels
    dev = conv.kernel.device
    if bn is None:
        scale = torch.ones(cout, dtype=torch.float32, device=dev)
        shift = torch.zeros(cout, dtype=torch.float32, device=dev)
    else:
        var = bn.running_var.float()
        mean = bn.running_mean.float()
        gamma = bn.weight.float() if bn.weight is not None else torch.ones_like(var)
        beta = bn.bias.float() if bn.bias is not None else torch.zeros_like(var)
        scale = gamma / torch.sqrt(var + bn.eps)
        shift = beta - mean * scale
    if conv.bias is not None:
        shift = shift + conv.bias.float() * scale
    return scale.detach().contiguous(), shift.detach().contiguous()


class FusedConv(nn.Module):
    """conv (+ folded BatchNorm) (+ ReLU); ``forward(x, residual=None)`` adds a residual feature
    matrix before the ReLU."""

    def __init__(self, conv: Conv3d, bn: Optional[nn.BatchNorm1d] = None, relu: bool = False) -> None:
        super().__init__()
        assert not conv.generative
        self.kernel_size, self.stride = make_ntuple(conv.kernel_size, 3), make_ntuple(conv.stride, 3)
        self.padding, self.dilation = conv.padding, make_ntuple(conv.dilation, 3)
        self.transposed, self._config = conv.transposed, conv._config
        self.in_channels, self.out_channels = conv.in_channels, conv.out_channels
        self.relu = relu
        self.kernel = nn.Parameter(conv.kernel.detach(), requires_grad=False)
        scale, shift = _fold_bn(conv, bn)
        self.pointwise = self.kernel.dim() == 2
        if self.pointwise:
            # 1x1x1: a dense matmul; the scale goes into the weights (fp32 product, then one rounding)
            self.kernel = nn.Parameter((self.kernel.float() * scale[None, :]).to(self.kernel.dtype),
                                       requires_grad=False)
            self.register_buffer("shift_lp", shift.to(self.kernel.dtype))
        self.register_buffer("scale", scale)
        self.register_buffer("shift", shift)
        self._plan = None      # per-layer constant launch arguments, made on first use

    def _apply(self, fn, recurse=True):
        # keep the folded scale / shift in fp32 under .half() / .to(dtype)
        scale, shift = self.scale, self.shift
        super()._apply(fn, recurse)
        self.scale = scale.to(self.kernel.device).float()
        self.shift = shift.to(self.kernel.device).float()
        self._plan = None
        return self

    # set by InferenceEngine: layers whose input (output, for transposed convs) tensor stride is at most
    # this value run on row-sorted kernel maps (fewer issued K blocks where the map is very sparse)
    sort_max_stride = 0

    def _layer_config(self, x: SparseTensor):
        if self._config is not None or self.sort_max_stride <= 0:
            return self._config
        # only submanifold convolutions: their map is shared by every layer of the resolution level, so
        # one sort serves many launches; a strided or transposed map is used once and not worth sorting
        if self.transposed or any(s != 1 for s in self.stride) or max(x.stride) > self.sort_max_stride:
            return None
        cfg = _conv_impl.resolve_config(None).copy()
        cfg["ifsort"] = True
        cfg["split_mask_num"] = 1
        return cfg

    def forward(self, x: SparseTensor, residual: Optional[torch.Tensor] = None) -> SparseTensor:
        if self.pointwise:
            out = torch.addmm(self.shift_lp, x.feats, self.kernel)
            if residual is not None:
                out = out + residual
            if self.relu:
                out = torch.relu_(out)
            return SparseTensor._from_parts(out, x.coords, x.stride, x.spatial_range, x._caches)
        layer_config = self._layer_config(x)
        y = self._forward_cached_map(x, residual, layer_config)
        if y is not None:
            return y
        return F.conv3d(x, self.kernel, self.kernel_size, None, self.stride, self.padding, self.dilation,
                        layer_config, self.transposed, False, False,
                        epilogue={"scale": self.scale, "bias": self.shift, "residual": residual, "relu": self.relu})

    def _forward_cached_map(self, x: SparseTensor, residual, layer_config) -> Optional[SparseTensor]:
        """Short path for the common case of a network's inner layers: implicit GEMM on a
        kernel map that is already in the tensor's cache (built by an earlier layer of the level or by
        the engine's prebuild).  Same launch as F.conv3d makes, without its per-call bookkeeping;
        returns None when the case does not apply."""
        config = _conv_impl.resolve_config(layer_config)
        if config["dataflow"] != F.Dataflow.ImplicitGEMM:
            return None
        ifsort = bool(config["ifsort"])
        if ifsort and config["split_mask_num"] != 1:
            return None
        feats = x.feats
        if feats.dtype != self.kernel.dtype or not feats.is_cuda:
            return None
        caches = x._caches
        if self.transposed:
            out_stride = tuple(a // b for a, b in zip(x.stride, self.stride))
            kmap = caches.kmaps.get((out_stride, self.kernel_size, self.stride, self.dilation))
            target = caches.cmaps.get(out_stride)
            if kmap is None or target is None or kmap.get("out_in_map_t") is None:
                return None
            if ifsort and (kmap.get("reorder_out_in_map_t") is None or kmap.get("_split_t") != 1):
                return None
            out_in_map, n_out = kmap["reorder_out_in_map_t" if ifsort else "out_in_map_t"], kmap["sizes"][0]
            reorder_loc = kmap["reorder_loc_t"] if ifsort else None
            out_coords, out_range = target
        else:
            kmap = caches.kmaps.get((x.stride, self.kernel_size, self.stride, self.dilation))
            if kmap is None:
                return None
            if ifsort and (kmap.get("reorder_out_in_map") is None or kmap.get("_split") != 1):
                return None
            out_in_map, n_out = kmap["reorder_out_in_map" if ifsort else "out_in_map"], kmap["sizes"][1]
            reorder_loc = kmap["reorder_loc"] if ifsort else None
            out_coords, out_range = kmap["coords"], kmap["spatial_range"]
            out_stride = tuple(a * b for a, b in zip(x.stride, self.stride))
        if feats.shape[1] % 8 != 0 or not feats.is_contiguous():
            return None     # the 4-channel input layer is padded by the general entry point
        plan = self._plan
        if plan is None or not plan.valid_for(self.kernel, backends.allow_tf32):
            plan = self._plan = backend.IgemmLayerPlan(self.kernel, self.scale, self.shift, backends.allow_tf32)
        out = backend.igemm_plan_launch(plan, feats, out_in_map, n_out, residual, self.relu, reorder_loc)
        caches.cmaps.setdefault(out_stride, (out_coords, out_range))
        return SparseTensor._from_parts(out, out_coords, out_stride, out_range, caches)

    def extra_repr(self) -> str:
        return (f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, stride={self.stride}, "
                f"relu={self.relu}, transposed={self.transposed}")


class FusedResBlock(nn.Module):
    """relu(conv2(relu(conv1(x))) + shortcut(x)) with both BatchNorms folded and the add + ReLU in the
    second convolution's epilogue."""

    def __init__(self, block) -> None:
        super().__init__()
        main = list(block.main)
        self.conv1 = FusedConv(main[0], main[1], relu=True)
        self.conv2 = FusedConv(main[3], main[4], relu=True)
        if isinstance(block.shortcut, nn.Identity):
            self.shortcut = None
        else:
            sc = list(block.shortcut)
            self.shortcut = FusedConv(sc[0], sc[1], relu=False)

    def forward(self, x: SparseTensor) -> SparseTensor:
        # the fused modules carry no hooks: their forward methods are called directly
        res = x.feats if self.shortcut is None else self.shortcut.forward(x).feats
        return self.conv2.forward(self.conv1.forward(x), residual=res)


class _FusedSequential(nn.Sequential):
    """nn.Sequential whose fused members are run through their forward methods directly (no hook
    dispatch per layer: at batch 1 the host, not the GPU, paces a forward pass)."""

    def forward(self, x):
        for m in self._modules.values():
            x = m.forward(x) if type(m) in _DIRECT else m(x)
        return x


def _fuse_sequential(seq: nn.Sequential) -> nn.Sequential:
    mods = list(seq)
    out = []
    i = 0
    while i < len(mods):
        m = mods[i]
        if isinstance(m, Conv3d) and not m.generative:
            bn = mods[i + 1] if i + 1 < len(mods) and isinstance(mods[i + 1], nn.BatchNorm1d) else None
            j = i + (2 if bn is not None else 1)
            relu = j < len(mods) and isinstance(mods[j], (ReLU, nn.ReLU))
            out.append(FusedConv(m, bn, relu))
            i = j + (1 if relu else 0)
        else:
            out.append(fuse_for_inference(m))
            i += 1
    return _FusedSequential(*out)


_DIRECT = (FusedConv, FusedResBlock)


def fuse_for_inference(model: nn.Module) -> nn.Module:
    """Returns a rewritten copy-free view of `model` (parameters are shared, BatchNorm statistics
    are folded at call time) for eval-mode inference.  Modules it does not recognise are kept."""
    from ..backbones.blocks import SparseResBlock

    if isinstance(model, SparseResBlock):
        return FusedResBlock(model)
    if isinstance(model, Conv3d) and not model.generative:
        return FusedConv(model, None, False)
    if isinstance(model, nn.Sequential):
        return _fuse_sequential(model)
    for name, child in list(model.named_children()):
        fused = fuse_for_inference(child)
        if fused is not child:
            model._modules[name] = fused
    return model


class InferenceEngine(nn.Module):
    """Eval-mode wrapper: fused modules, no autograd, strided kernel maps built ahead of the convs."""

    def __init__(self, model: nn.Module, sort_max_stride: int = 0) -> None:
        """`sort_max_stride` > 0: convolutions at tensor strides up to that value use row-sorted kernel
        maps (the reference's sorted implicit GEMM, chosen per resolution level instead of globally)."""
        super().__init__()
        if model.training:
            raise ValueError("InferenceEngine needs a model in eval() mode (BatchNorm statistics are folded)")
        self.model = fuse_for_inference(model)
        for m in self.model.modules():
            if isinstance(m, FusedConv):
                m.sort_max_stride = sort_max_stride
        self._plan = None   # strided conv keys in execution order, learnt on the first call

    def _prebuild(self, x: SparseTensor) -> None:
        caches = x._caches
        caches.cmaps.setdefault(x.stride, (x.coords, x.spatial_range))
        for tensor_stride, ks, st, pad, dil, config in self._plan:
            cm = caches.cmaps.get(tensor_stride)
            if cm is None:
                return   # the plan no longer matches this input; fall back to building on demand
            coords, srange = cm
            _conv_impl.acquire_kernel_map(caches, coords, coords.shape[0], tensor_stride, srange, ks, st, pad, dil,
                                          config, False)

    @torch.no_grad()
    def forward(self, x: SparseTensor):
        if self._plan is None:
            _conv_impl.strided_build_log = []
            try:
                out = self.model(x)
            finally:
                log, _conv_impl.strided_build_log = _conv_impl.strided_build_log, None
            cfg = _conv_impl.resolve_config(None)
            self._plan = [entry + (cfg,) for entry in log]
            return out
        self._prebuild(x)
        return self.model(x)
