"""The three dataflows as autograd Functions (forward only)
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


class _ForwardOnly(Function):
    @staticmethod
    def backward(ctx, grad_output):
        raise NotImplementedError("the backward pass (dgrad / wgrad) of the sparse convolution is not built yet")


class ImplicitGEMMConvolutionFuntion(_ForwardOnly):
    @staticmethod
    def forward(ctx, input: torch.Tensor, weight: torch.Tensor, kmap: Dict, config: Dict,
                transposed: bool = False, epilogue: Dict = None) -> torch.Tensor:
        if input.device.type != "cuda":
            raise NotImplementedError
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


class GatherScatterConvolutionFuntion(_ForwardOnly):
    @staticmethod
    def forward(ctx, input: torch.Tensor, weight: torch.Tensor, kmap: Dict, config: Dict,
                transposed: bool = False, epilogue: Dict = None) -> torch.Tensor:
        if input.device.type != "cuda":
            raise NotImplementedError
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


class FetchOnDemandConvolutionFuntion(_ForwardOnly):
    @staticmethod
    def forward(ctx, input: torch.Tensor, weight: torch.Tensor, kmap: Dict, config: Dict,
                transposed: bool = False, epilogue: Dict = None) -> torch.Tensor:
        if input.device.type != "cuda":
            raise NotImplementedError
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
