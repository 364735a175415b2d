"""CPU restatement of the bird's-eye-view heads, test infrastructure only (never imported by the library).

What torchsparse/nn/modules/bev.py:17-222 describes, on (batch, x, y, z) coordinate rows: `dim` is the collapsed
spatial axis (coordinate column dim + 1).  Plain loops over the voxels, float64 accumulation.  Parity unpinned: the
reference file cannot run on 2.1 tensors (it indexes the (x, y, z, batch) rows of earlier releases and reads
.values() of a dense tensor), so there is no reference output to pin against; the cases are small enough to check
by hand."""
import numpy as np


def _cells_sorted(rows):
    uniq = sorted(set(map(tuple, rows)))
    return uniq, {c: i for i, c in enumerate(uniq)}


def bev_reduction(coords, feats, dim):
    """bev.py:17-36 -> (coords [M,4], mean feats [M,C]) in lexicographic cell order."""
    c = coords.copy()
    c[:, dim + 1] = 0
    uniq, index = _cells_sorted(c)
    acc = np.zeros((len(uniq), feats.shape[1]))
    cnt = np.zeros(len(uniq))
    for row, f in zip(c, feats):
        acc[index[tuple(row)]] += f
        cnt[index[tuple(row)]] += 1
    return np.array(uniq, dtype=np.int32).reshape(-1, 4), acc / cnt[:, None]


def bev_convolution(coords, feats, tensor_stride, kernel, bias, dim, stride):
    """bev.py:118-164 -> (coords [M,4], feats [M,Cout], stride): feats[cell] = sum over its voxels of
    f @ kernel[height layer] + bias."""
    ratio = tuple(int(s) * stride for s in tensor_stride)
    c = coords.copy()
    c[:, dim + 1] = 0
    if stride > 1:
        for a in range(3):
            c[:, a + 1] = np.floor_divide(c[:, a + 1], ratio[a]) * ratio[a]
    uniq, index = _cells_sorted(c)
    acc = np.zeros((len(uniq), kernel.shape[2]))
    for row, src, f in zip(c, coords, feats):
        k = int(src[dim + 1]) // int(tensor_stride[dim])
        acc[index[tuple(row)]] += f.astype(np.float64) @ kernel[k].astype(np.float64) + (0 if bias is None else bias[0])
    return np.array(uniq, dtype=np.int32).reshape(-1, 4), acc, ratio


def dense_bev_convolution(coords, feats, tensor_stride, kernel, bias, shape, offset, dim):
    """bev.py:39-115 -> dense [B, Cout, H, W]."""
    bev = [a for a in range(3) if a != dim]
    batch = int(coords[:, 0].max()) + 1
    out = np.zeros((batch, shape[bev[0]], shape[bev[1]], kernel.shape[2]))
    for src, f in zip(coords, feats):
        k = int(src[dim + 1]) // int(tensor_stride[dim])
        u = (int(src[bev[0] + 1]) - offset[bev[0]]) // int(tensor_stride[bev[0]])
        v = (int(src[bev[1] + 1]) - offset[bev[1]]) // int(tensor_stride[bev[1]])
        if 0 <= u < shape[bev[0]] and 0 <= v < shape[bev[1]]:
            out[int(src[0]), u, v] += f.astype(np.float64) @ kernel[k].astype(np.float64) + (0 if bias is None else bias[0])
    return out.transpose(0, 3, 1, 2)


def bev_height_compression(coords, feats, tensor_stride, shape, offset, dim):
    """bev.py:167-222 -> dense [B, Z * C, H, W], layer-major channels, heights clamped into the map."""
    bev = [a for a in range(3) if a != dim]
    batch = int(coords[:, 0].max()) + 1
    out = np.zeros((batch, shape[bev[0]], shape[bev[1]], shape[dim], feats.shape[1]))
    for src, f in zip(coords, feats):
        u = (int(src[bev[0] + 1]) - offset[bev[0]]) // int(tensor_stride[bev[0]])
        v = (int(src[bev[1] + 1]) - offset[bev[1]]) // int(tensor_stride[bev[1]])
        z = min(max((int(src[dim + 1]) - offset[dim]) // int(tensor_stride[dim]), 0), shape[dim] - 1)
        if 0 <= u < shape[bev[0]] and 0 <= v < shape[bev[1]]:
            out[int(src[0]), u, v, z] += f
    return out.reshape(batch, shape[bev[0]], shape[bev[1]], -1).transpose(0, 3, 1, 2)
