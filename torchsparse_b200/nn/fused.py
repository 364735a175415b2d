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
from .functional.conv.kmap import transpose_kernel_map
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
    matrix before the ReLU.  Every kernel shape, the 1x1x1 kernels included, runs on the library's
    implicit-GEMM kernel; an input that is a pending concatenation (CatSparseTensor) is read from its
    two matrices."""

    # set by InferenceEngine: submanifold layers at tensor strides up to sorted_max_stride run on row-sorted,
    # column-major copies of their kernel maps (built once per map, shared by all layers that use it).  Strided
    # and transposed maps serve one layer each and the coarsest level has few rows: there the copy costs more
    # than the offset blocks it saves.
    sorted_maps = False
    sorted_max_stride = 8
    sorted_strided = False      # also the strided and transposed maps (one sorted copy per map and direction)

    def _wants_sorted(self, stride) -> bool:
        if not self.sorted_maps or max(stride) > self.sorted_max_stride:
            return False
        return self.sorted_strided or (not self.transposed and all(s == 1 for s in self.stride))

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

    def invalidate(self) -> None:
        """Forget the cached launch plan and packed weights (call after changing the weights through
        ``.data`` or a raw pointer, which the version counter does not see)."""
        self._plan = None
        for name in ("_tsb_packed", "_tsb_padded"):
            if hasattr(self.kernel, name):
                delattr(self.kernel, name)

    def _kernel3(self) -> torch.Tensor:
        return self.kernel if self.kernel.dim() == 3 else self.kernel.view(1, *self.kernel.shape)

    def _input_kernel(self, channels: int) -> torch.Tensor:
        """[Kvol, Cin, Cout] weights for an input of `channels` channels: the layer's own, or, for an input
        whose channels were zero-padded to the next multiple of 8 (the 4- or 5-channel network input, so that
        its rows are 16-byte multiples), the weights with zero rows for the padding (made once)."""
        kernel = self._kernel3()
        cin = kernel.shape[1]
        if channels != cin and channels == (cin + 7) // 8 * 8:
            return backend._padded_kernel(kernel)
        return kernel

    def forward(self, x: SparseTensor, residual: Optional[torch.Tensor] = None) -> SparseTensor:
        if getattr(x, "dyn", None) is not None:      # a tensor of the static (CUDA graph) engine
            from .static_engine import dyn_conv
            return dyn_conv(self, x, residual)
        y = self._forward_planned(x, residual)
        if y is not None:
            return y
        epilogue = {"scale": self.scale, "bias": self.shift, "residual": residual, "relu": self.relu}
        if self.pointwise:
            feats = x.feats
            out = backend.conv_forward_implicit_gemm_cuda(feats, self._kernel3().to(feats.dtype), None, feats.shape[0],
                                                          self.out_channels, backends.allow_tf32, True, **epilogue) \
                if backend._tensor_core_shape(feats, self._kernel3(), backends.allow_tf32) else \
                _conv_impl._epilogue_torch(feats.matmul(self.kernel.to(feats.dtype)), epilogue)
            return SparseTensor._from_parts(out, x.coords, x.stride, x.spatial_range, x._caches)
        return F.conv3d(x, self.kernel, self.kernel_size, None, self.stride, self.padding, self.dilation,
                        self._config, self.transposed, False, False, epilogue=epilogue)

    def _forward_planned(self, x: SparseTensor, residual) -> Optional[SparseTensor]:
        """The common case: implicit GEMM on the tensor cores through the layer's launch plan.  The kernel
        map comes from the tensor's cache (built by an earlier layer of the level, by the engine's
        prebuild, or here), optionally in its row-sorted column-major form.  Returns None when the case
        does not apply (another dataflow, a shape the tensor-core kernel does not take)."""
        config = _conv_impl.resolve_config(self._config)
        if config["dataflow"] != F.Dataflow.ImplicitGEMM or config["ifsort"]:
            return None
        parts = getattr(x, "parts", None)
        feats, feats2 = (parts[0], parts[1]) if (parts is not None and len(parts) == 2) else (x.feats, None)
        kernel = self._input_kernel(feats.shape[1] + (0 if feats2 is None else feats2.shape[1]))
        if feats.dtype != kernel.dtype or not feats.is_cuda or not feats.is_contiguous():
            return None
        if (feats.shape[1] * feats.element_size()) % 16 != 0:
            return None     # the 4-channel input layer is padded by the general entry point
        if feats2 is not None and (not feats2.is_contiguous() or feats2.dtype != kernel.dtype):
            return None
        if feats.dtype == torch.float32 and not backends.allow_tf32:
            return None
        plan = self._plan
        if plan is None or not plan.valid_for(kernel, backends.allow_tf32):
            try:
                plan = self._plan = backend.IgemmLayerPlan(kernel, self.scale, self.shift, backends.allow_tf32)
            except ValueError:
                return None
        caches = x._caches
        if self.pointwise:
            out = backend.igemm_plan_launch(plan, feats, None, feats.shape[0], residual, self.relu, in_feats2=feats2)
            return SparseTensor._from_parts(out, x.coords, x.stride, x.spatial_range, caches)
        if self.transposed:
            out_stride = tuple(a // b for a, b in zip(x.stride, self.stride))
            kmap = caches.kmaps.get((out_stride, self.kernel_size, self.stride, self.dilation))
            target = caches.cmaps.get(out_stride)
            if kmap is None or target is None:
                return None
            if kmap.get("out_in_map_t") is None:
                transpose_kernel_map(kmap)
            sfx, n_out = "_t", kmap["sizes"][0]
            out_coords, out_range = target
        else:
            caches.cmaps.setdefault(x.stride, (x.coords, x.spatial_range))
            kmap = _conv_impl.acquire_kernel_map(caches, x.coords, feats.shape[0], x.stride, x.spatial_range,
                                                 self.kernel_size, self.stride, make_ntuple(self.padding, 3),
                                                 self.dilation, config, False)
            sfx, n_out = "", kmap["sizes"][1]
            out_coords, out_range = kmap["coords"], kmap["spatial_range"]
            out_stride = tuple(a * b for a, b in zip(x.stride, self.stride))
        out_in_map = kmap["out_in_map" + sfx]
        if self._wants_sorted(x.stride):
            art = kmap.get("_cm" + sfx)
            if art is None:
                art = kmap["_cm" + sfx] = backend.sorted_cm_artefacts_cuda(out_in_map, n_out)
            out = backend.igemm_plan_launch(plan, feats, None, n_out, residual, self.relu, in_feats2=feats2, smap=art)
        else:
            out = backend.igemm_plan_launch(plan, feats, out_in_map, n_out, residual, self.relu, in_feats2=feats2)
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
    """Eval-mode wrapper: fused modules, no autograd, strided kernel maps built ahead of the convs,
    skip concatenations read in place by the layer that follows them."""

    def __init__(self, model: nn.Module, sorted_maps: bool = True, sorted_max_stride: int = 8,
                 sorted_strided: bool = False) -> None:
        """`sorted_maps`: the kernel map of the submanifold layers of a resolution level (tensor stride up to
        `sorted_max_stride`) gets a row-sorted, column-major copy with per-tile offset masks the first time a
        layer uses it (tsb_map_sorted_cm), and all layers sharing the map run on that copy: the 128 rows of a
        tile then share their neighbour pattern and few (tile, offset) blocks remain."""
        super().__init__()
        if model.training:
            raise ValueError("InferenceEngine needs a model in eval() mode (BatchNorm statistics are folded)")
        self.model = fuse_for_inference(model)
        for m in self.model.modules():
            if isinstance(m, FusedConv):
                m.sorted_maps = bool(sorted_maps)
                m.sorted_max_stride = int(sorted_max_stride)
                m.sorted_strided = bool(sorted_strided)
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
        from .. import operators

        was_lazy, operators.lazy = operators.lazy, True
        try:
            if getattr(x, "dyn", None) is not None:
                return self.model(x)
            if self._plan is None:
                _conv_impl.strided_build_log = []
                try:
                    out = self.model(x)
                finally:
                    log, _conv_impl.strided_build_log = _conv_impl.strided_build_log, None
                cfg = _conv_impl.resolve_config(None)
                self._plan = [entry + (cfg,) for entry in log]
                return out
            self._prebuild(x)     # its size readbacks also fetch the convolution kernels' status word
            return self.model(x)
        finally:
            operators.lazy = was_lazy
