import torch

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


def spdevoxelize(feats: torch.Tensor, coords: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """Interpolate voxel features at points: ``coords`` int [N,8] voxel rows (-1 = absent),
    ``weights`` [N,8] (torchsparse/nn/functional/devoxelize.py:52-101; forward only)."""
    return backend.devoxelize_forward_cuda(feats.contiguous(), coords.contiguous().int(), weights.contiguous())
