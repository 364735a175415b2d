import torch
from torch.autograd import Function

from ... import backend

__all__ = ["spdevoxelize", "calc_ti_weights"]


def calc_ti_weights(coords: torch.Tensor, idx_query: torch.Tensor, scale: float = 1) -> torch.Tensor:
    """Trilinear interpolation weights of the 8 surrounding voxels, zeroed where the voxel is
    absent and renormalised (torchsparse/nn/functional/devoxelize.py:11-49)."""
    with torch.no_grad():
        p = coords
        pf = torch.floor(coords / scale) * scale if scale != 1 else torch.floor(coords)
        pc = pf + scale
        lo = [(p[:, i] - pf[:, i].float()).view(-1, 1) for i in range(3)]   # distance to the lower corner
        hi = [(pc[:, i].float() - p[:, i]).view(-1, 1) for i in range(3)]   # distance to the upper corner
        cols = []
        for corner in range(8):
            fx = lo[0] if corner & 4 else hi[0]
            fy = lo[1] if corner & 2 else hi[1]
            fz = lo[2] if corner & 1 else hi[2]
            cols.append(fx * fy * fz)
        w = torch.cat(cols, dim=1)
        if scale != 1:
            w /= scale ** 3
        w[idx_query == -1] = 0
        w /= torch.sum(w, dim=1).unsqueeze(1) + 1e-8
    return w


class _Devoxelize(Function):
    """Interpolation of voxel features at points and its gradient with respect to the voxel features
    (torchsparse/nn/functional/devoxelize.py:52-101)."""

    @staticmethod
    def forward(ctx, feats: torch.Tensor, coords: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        ctx.save_for_backward(coords, weights)
        ctx.n_vox = feats.shape[0]
        return backend.devoxelize_forward_cuda(feats, coords, weights)

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        coords, weights = ctx.saved_tensors
        grad = backend.devoxelize_backward_cuda(grad_output, coords, weights, ctx.n_vox)
        return grad.to(grad_output.dtype), None, None


def spdevoxelize(feats: torch.Tensor, coords: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """Interpolate voxel features at points: ``coords`` int [N,8] voxel rows (-1 = absent),
    ``weights`` [N,8] (torchsparse/nn/functional/devoxelize.py:52-101)."""
    feats, coords, weights = feats.contiguous(), coords.contiguous().int(), weights.contiguous()
    if torch.is_grad_enabled() and feats.requires_grad:
        return _Devoxelize.apply(feats, coords, weights)
    return backend.devoxelize_forward_cuda(feats, coords, weights)
