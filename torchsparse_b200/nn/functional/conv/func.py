"""The three dataflows as autograd Functions
(torchsparse/nn/functional/conv/func/{implicit_gemm,gather_scatter,fetch_on_demand}.py)."""
from typing import Dict

import torch
from torch.autograd import Function

from .... import backend, backends

__all__ = ["ImplicitGEMMConvolutionFuntion", "GatherScatterConvolutionFuntion", "FetchOnDemandConvolutionFuntion"]


def _cast_pair(input: torch.Tensor, weight: torch.Tensor):
    # either operand in fp16 -> both in fp16 (torchsparse/nn/functional/conv/func/implicit_gemm.py:64-66)
    if torch.float16 in (input.dtype, weight.dtype):
        return input.to(torch.float16), weight.to(torch.float16)
    if input.dtype != weight.dtype:
        return input, weight.to(input.dtype)
    return input, weight


def _remember(ctx, input: torch.Tensor, weight: torch.Tensor, kmap: Dict, transposed: bool) -> None:
    """What backward needs (ctx is None when the forward runs outside autograd)."""
    if ctx is not None:
        ctx.save_for_backward(input, weight)
        ctx.kmap, ctx.transposed = kmap, transposed


class _SparseConvFunction(Function):
    """Backward shared by the three dataflows (torchsparse/nn/functional/conv/func/implicit_gemm.py:108-193):

    * dgrad: the implicit-GEMM *forward* kernel run on grad_output with W transposed per offset and the
      transposed kernel map (input row -> output rows), as the reference does;
    * wgrad: dW[k] = sum over output rows m of X[map[m][k]]^T . dY[m] on the tensor cores (tcgen05, both operands
      read row-major = MN-major; torchsparse/backend/convolution/convolution_backward_wgrad_implicit_gemm_cuda.cu);
      exact fp32 and odd channel counts as one masked product per offset."""

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        from .kmap import transpose_kernel_map

        input, weight = ctx.saved_tensors
        kmap, transposed = ctx.kmap, ctx.transposed
        x, w = _cast_pair(input.contiguous(), weight.contiguous())
        dy = grad_output.contiguous().to(w.dtype)
        kvol, cin, cout = w.shape
        grad_input = grad_weight = None
        if ctx.needs_input_grad[0]:
            if transposed:
                bwd_map = kmap["out_in_map"]               # rows: inputs of the transposed conv
            else:
                bwd_map = transpose_kernel_map(kmap)["out_in_map_t"]
            grad_input = backend.conv_forward_implicit_gemm_cuda(
                dy, w.transpose(1, 2).contiguous(), bwd_map, x.shape[0], cin, backends.allow_tf32,
                backends.allow_fp16).to(input.dtype)
        if ctx.needs_input_grad[1]:
            # dW[k] = sum over output rows m of X[map[m][k]]^T . dY[m] on the map the forward used
            fwd_map = kmap.get("out_in_map_t") if transposed else kmap["out_in_map"]
            if fwd_map is None:
                fwd_map = transpose_kernel_map(kmap)["out_in_map_t"]
            grad_weight = backend.conv_wgrad_implicit_gemm_cuda(x, dy, fwd_map).to(weight.dtype)
        return grad_input, grad_weight, None, None, None, None


class ImplicitGEMMConvolutionFuntion(_SparseConvFunction):
    @staticmethod
    def forward(ctx, input: torch.Tensor, weight: torch.Tensor, kmap: Dict, config: Dict,
                transposed: bool = False, epilogue: Dict = None) -> torch.Tensor:
        if input.device.type != "cuda":
            raise NotImplementedError
        _remember(ctx, input, weight, kmap, transposed)
        sizes = kmap["sizes"]
        sfx = "_t" if transposed else ""
        input, weight = _cast_pair(input.contiguous(), weight.contiguous())
        num_out_feats = sizes[0] if transposed else sizes[1]
        epilogue = epilogue or {}
        if not config["ifsort"]:
            out = backend.conv_forward_implicit_gemm_cuda(
                input, weight, kmap["out_in_map" + sfx], num_out_feats, weight.shape[-1], backends.allow_tf32,
                backends.allow_fp16, **epilogue)
        else:
            out = backend.conv_forward_implicit_gemm_sorted_cuda(
                input, weight, kmap["reorder_out_in_map" + sfx], kmap["reduced_sorted_mask" + sfx],
                kmap["reorder_loc" + sfx], num_out_feats, weight.shape[-1], backends.allow_tf32,
                backends.allow_fp16, **epilogue)
        return out.to(weight.dtype)


class GatherScatterConvolutionFuntion(_SparseConvFunction):
    @staticmethod
    def forward(ctx, input: torch.Tensor, weight: torch.Tensor, kmap: Dict, config: Dict,
                transposed: bool = False, epilogue: Dict = None) -> torch.Tensor:
        if input.device.type != "cuda":
            raise NotImplementedError
        _remember(ctx, input, weight, kmap, transposed)
        sizes = kmap["sizes"]
        input, weight = _cast_pair(input.contiguous(), weight.contiguous())
        sizes_host = kmap.get("nbsizes_host")
        if sizes_host is None:
            sizes_host = kmap["nbsizes"].cpu().tolist()
        out = backend.conv_forward_gather_scatter_cuda(
            input, weight, kmap["nbmaps"], sizes_host, kmap["input_mask"], kmap["output_mask"],
            sizes[0] if transposed else sizes[1], config["epsilon"], int(config["mm_thresh"]), 0, transposed, None,
            backends.allow_tf32)
        return out.to(weight.dtype)


class FetchOnDemandConvolutionFuntion(_SparseConvFunction):
    @staticmethod
    def forward(ctx, input: torch.Tensor, weight: torch.Tensor, kmap: Dict, config: Dict,
                transposed: bool = False, epilogue: Dict = None) -> torch.Tensor:
        if input.device.type != "cuda":
            raise NotImplementedError
        _remember(ctx, input, weight, kmap, transposed)
        sizes = kmap["sizes"]
        input, weight = _cast_pair(input.contiguous(), weight.contiguous())
        nbmaps = kmap["nbmaps"]
        out_size = sizes[0] if transposed else sizes[1]
        if config["FOD_fusion"]:
            out = backend.conv_forward_fetch_on_demand_cuda(
                input, weight, nbmaps, nbmaps.size(1), kmap["nbaddrs"], kmap["qnbaddrs"], out_size,
                kmap["qmapsize"], transposed, backends.allow_tf32, backends.allow_fp16)
        else:
            out = backend.conv_forward_fetch_on_demand_no_fusion_cuda(
                input, weight, nbmaps, torch.tensor(kmap["nbsizes_host"], dtype=torch.int32), nbmaps.size(1),
                out_size, transposed, backends.allow_tf32, backends.allow_fp16)
        return out.to(weight.dtype)
