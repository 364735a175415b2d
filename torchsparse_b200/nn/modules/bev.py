"""Bird's-eye-view heads (torchsparse/nn/modules/bev.py:17-222): collapse one spatial axis of a SparseTensor.

The four modules keep the reference's names, constructor arguments and parameter shapes.  Coordinates are the
(batch, x, y, z) rows of this package's tensors; ``dim`` names the spatial axis that is collapsed (0, 1, 2 = x, y, z),
i.e. coordinate column ``dim + 1``.  (The reference file still indexes the (x, y, z, batch) rows of earlier releases
and reads ``.values()`` / ``.indices()`` of a tensor it has just made dense, so it cannot run on 2.1 tensors; what is
built here is what its docstrings describe.)

The per-height fully connected layers run as a sparse convolution on the implicit-GEMM kernel: the BEV cells are
the output rows, the height index is the kernel offset and ``out_in_map[cell][height]`` is the voxel there, so the
forward, the input gradient and the weight gradient are the convolution's; the reductions and the dense scatters
are the voxelize and to_dense kernels.
"""
import math
from typing import List, Tuple, Union

import torch
from torch import nn

from ...tensor import SparseTensor

__all__ = ["ToBEVConvolution", "ToBEVReduction", "ToDenseBEVConvolution", "ToBEVHeightCompression"]


def _axis(dim: int) -> int:
    if dim not in (0, 1, 2):
        raise ValueError("dim names a spatial axis: 0, 1 or 2")
    return dim


def _height_conv(feats: torch.Tensor, kernel: torch.Tensor, cells: torch.Tensor, offset_index: torch.Tensor,
                 n_offsets: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Sum over the voxels of each cell of ``feats[voxel] @ kernel[offset_index[voxel]]``.

    cells: int [N, 3] (batch, u, v) of every voxel; (cell, offset_index) pairs are unique.  Returns the rows
    [M, Cout] in the lexicographic order of the unique cells, the cells [M, 3] and the voxel -> cell index."""
    from ..functional.conv.func import ImplicitGEMMConvolutionFuntion

    uniq, inverse = torch.unique(cells, dim=0, return_inverse=True)
    n, m = feats.shape[0], uniq.shape[0]
    rows = (m + 127) // 128 * 128
    out_in_map = torch.full((rows, n_offsets), -1, dtype=torch.int32, device=feats.device)
    out_in_map[inverse, offset_index] = torch.arange(n, dtype=torch.int32, device=feats.device)
    kmap = {"out_in_map": out_in_map, "sizes": (n, m)}
    out = ImplicitGEMMConvolutionFuntion.apply(feats, kernel, kmap, {"ifsort": False}, False, None)
    return out, uniq, inverse


def _height_index(input: SparseTensor, dim: int, n_kernels: int) -> torch.Tensor:
    k = torch.div(input.coords[:, dim + 1], int(input.stride[dim]), rounding_mode="floor").long()
    if k.numel() and (int(k.min()) < 0 or int(k.max()) >= n_kernels):
        raise ValueError(f"a voxel lies outside the {n_kernels} height layers of the kernel")
    return k


class ToBEVReduction(nn.Module):
    """Mean of the features over the collapsed axis; the result keeps a zero in that coordinate column."""

    def __init__(self, dim: int = 1) -> None:
        super().__init__()
        self.dim = _axis(dim)

    def extra_repr(self):
        return f"dim = {self.dim}"

    def forward(self, input: SparseTensor) -> SparseTensor:
        from .. import functional as F

        coords = input.coords.clone()
        coords[:, self.dim + 1] = 0
        uniq, inverse = torch.unique(coords, dim=0, return_inverse=True)
        counts = torch.bincount(inverse, minlength=uniq.shape[0]).int()
        feats = F.spvoxelize(input.feats, inverse.int(), counts)
        return SparseTensor(coords=uniq.int(), feats=feats, stride=input.stride)


class ToBEVConvolution(nn.Module):
    """Sparse BEV map: every height layer has its own [in_channels, out_channels] matrix, the products of a
    column are summed.  ``stride`` > 1 also merges stride x stride columns (their voxels keep their own layer's
    matrix); the result lives at tensor stride ``input.stride * stride``."""

    def __init__(self, in_channels: int, out_channels: int, n_kernels: int, stride: int = 1, dim: int = 1,
                 bias: bool = False) -> None:
        super().__init__()
        self.in_channels, self.out_channels, self.n_kernels = in_channels, out_channels, n_kernels
        self.stride, self.dim = int(stride), _axis(dim)
        self.kernel = nn.Parameter(torch.zeros(n_kernels, in_channels, out_channels))
        self.bias = nn.Parameter(torch.zeros(1, out_channels)) if bias else 0
        self.reset_parameters()

    def reset_parameters(self):
        std = 1.0 / math.sqrt(self.in_channels)
        with torch.no_grad():
            self.kernel.uniform_(-std, std)

    def extra_repr(self):
        return "in_channels={}, out_channels={}, n_kernels={}, stride={}".format(
            self.in_channels, self.out_channels, self.n_kernels, self.stride)

    def forward(self, input: SparseTensor) -> SparseTensor:
        coords, s = input.coords, self.stride
        ratio = tuple(int(v) * s for v in input.stride)
        k = _height_index(input, self.dim, self.n_kernels)
        cells = coords.clone()
        cells[:, self.dim + 1] = 0
        kernel, offset_index, n_offsets = self.kernel, k, self.n_kernels
        if s > 1:
            bev = [a for a in range(3) if a != self.dim]
            sub = [torch.div(coords[:, a + 1], int(input.stride[a]), rounding_mode="floor").long() % s for a in bev]
            for a in range(3):
                cells[:, a + 1] = torch.div(cells[:, a + 1], ratio[a], rounding_mode="floor") * ratio[a]
            offset_index = k * (s * s) + sub[0] * s + sub[1]
            kernel = self.kernel.repeat_interleave(s * s, dim=0)
            n_offsets = self.n_kernels * s * s
        out, uniq, inverse = _height_conv(input.feats, kernel, cells, offset_index, n_offsets)
        if isinstance(self.bias, torch.Tensor):       # added per voxel before the sum, as the reference does
            counts = torch.bincount(inverse, minlength=uniq.shape[0]).to(out.dtype)
            out = out + counts[:, None] * self.bias.to(out.dtype)
        return SparseTensor(out, uniq.int(), ratio)


class _DenseBEV(nn.Module):
    """Shared by the two dense heads: BEV shape, offset and the (batch, u, v, height) rows of the voxels."""

    def _setup(self, shape, offset, dim) -> None:
        self.dim = _axis(dim)
        self.register_buffer("offset", torch.IntTensor([[0] + list(offset)]))
        self.register_buffer("shape", shape.int() if isinstance(shape, torch.Tensor) else torch.IntTensor(list(shape)))
        self.bev_dims = [i for i in range(3) if i != self.dim]
        self.bev_shape = self.shape[self.bev_dims]

    def _grid_rows(self, input: SparseTensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """int [N, 4] (batch, u, v, height) in grid cells, and the rows that fall inside the BEV map."""
        stride = torch.tensor([1] + [int(v) for v in input.stride], device=input.coords.device)
        cells = torch.div(input.coords - self.offset.to(input.coords.device), stride, rounding_mode="floor")
        cells = cells[:, [0] + [a + 1 for a in self.bev_dims] + [self.dim + 1]]
        h, w = int(self.bev_shape[0]), int(self.bev_shape[1])
        inside = (cells[:, 1] >= 0) & (cells[:, 1] < h) & (cells[:, 2] >= 0) & (cells[:, 2] < w)
        return cells, inside


class ToDenseBEVConvolution(_DenseBEV):
    """Dense BEV feature map [B, out_channels, H, W]: per-height matrices as in ``ToBEVConvolution``, the sums
    written into a dense map of ``shape`` without the collapsed axis; voxels outside the map are dropped."""

    def __init__(self, in_channels: int, out_channels: int,
                 shape: Union[List[int], Tuple[int, int, int], torch.Tensor], offset: Tuple[int, int, int] = (0, 0, 0),
                 dim: int = 1, bias: bool = False) -> None:
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self._setup(shape, offset, dim)
        self.n_kernels = int(self.shape[self.dim])
        self.kernel = nn.Parameter(torch.zeros(self.n_kernels, in_channels, out_channels))
        self.bias = nn.Parameter(torch.zeros(1, out_channels)) if bias else 0
        self.reset_parameters()

    def extra_repr(self):
        return "in_channels={}, out_channels={}, n_kernels={}".format(self.in_channels, self.out_channels,
                                                                       self.n_kernels)

    def reset_parameters(self):
        std = 1.0 / math.sqrt(self.in_channels)
        with torch.no_grad():
            self.kernel.uniform_(-std, std)

    def forward(self, input: SparseTensor) -> torch.Tensor:
        from ...utils.to_dense import to_dense

        k = _height_index(input, self.dim, self.n_kernels)       # the layer follows the raw coordinate, as in the reference
        cells, inside = self._grid_rows(input)
        batch = int(input.coords[:, 0].max()) + 1 if input.coords.shape[0] else 0
        h, w = int(self.bev_shape[0]), int(self.bev_shape[1])
        feats = input.feats
        if not bool(inside.all()):
            feats, cells, k = feats[inside], cells[inside], k[inside]
        out, uniq, inverse = _height_conv(feats, self.kernel, cells[:, :3].contiguous(), k, self.n_kernels)
        if isinstance(self.bias, torch.Tensor):
            counts = torch.bincount(inverse, minlength=uniq.shape[0]).to(out.dtype)
            out = out + counts[:, None] * self.bias.to(out.dtype)
        rows = torch.cat([uniq, torch.zeros_like(uniq[:, :1])], dim=1).int()
        dense = to_dense(out, rows, (batch, h, w, 1))            # [B, H, W, 1, C]
        return dense.view(batch, h, w, -1).permute(0, 3, 1, 2).contiguous()


class ToBEVHeightCompression(_DenseBEV):
    """Dense [B, Z * channels, H, W]: the features of a column stacked by height layer (heights clamped into
    ``shape[dim]`` layers); voxels outside the map are dropped."""

    def __init__(self, channels: int, shape: Union[List[int], Tuple[int, int, int], torch.Tensor],
                 offset: Tuple[int, int, int] = (0, 0, 0), dim: int = 1) -> None:
        super().__init__()
        self.channels = channels
        self._setup(shape, offset, dim)

    def extra_repr(self) -> str:
        return f"channels={self.channels}"

    def forward(self, input: SparseTensor) -> torch.Tensor:
        from ...utils.to_dense import to_dense

        cells, inside = self._grid_rows(input)
        layers = int(self.shape[self.dim])
        batch = int(input.coords[:, 0].max()) + 1 if input.coords.shape[0] else 0
        h, w = int(self.bev_shape[0]), int(self.bev_shape[1])
        feats = input.feats
        if not bool(inside.all()):
            feats, cells = feats[inside], cells[inside]
        clamped = cells[:, 3].clamp(0, layers - 1)
        if not torch.equal(clamped, cells[:, 3]):
            # voxels above or below the map share its edge layers: their features add up, as in a coalesced scatter
            cells = torch.cat([cells[:, :3], clamped[:, None]], dim=1)
            cells, inverse = torch.unique(cells, dim=0, return_inverse=True)
            feats = feats.new_zeros((cells.shape[0], feats.shape[1])).index_add_(0, inverse, feats)
        dense = to_dense(feats, cells.int(), (batch, h, w, layers))      # [B, H, W, Z, C]
        return dense.view(batch, h, w, -1).permute(0, 3, 1, 2).contiguous()
