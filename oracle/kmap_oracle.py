"""CPU oracle for the sparse-convolution hot path (TEST INFRASTRUCTURE ONLY).

This module restates, in numpy, what the reference computes on its CUDA backend
for the kernel-map / sparse-conv path.  It is the checker that the CUDA kernels
are compared with: only the test-suite, the smoke check and the ``cpu_baseline``
/ ``--impl reference`` legs of the benchmark may import it.  The product package
never does.

Pinning: the reference ships no golden vectors for this path.  Its own test
(tests/python/test_single_layer_conv.py:111-220) pins results through
equivalence with a dense ``torch.nn.Conv3d``; the same equivalence is checked
for this oracle in tests/test_oracle.py and against fixtures in tests/golden/
that were generated from the reference's own CPU convolution sources and its
own numpy ``sparse_quantize``.

Each function cites the reference file:line whose behaviour it follows
(paths relative to the reference project root).
"""
from __future__ import annotations

import numpy as np

CTA_M = 128  # row padding of every map (torchsparse/backend/hashmap/hashmap_cuda.cuh:310)


# --------------------------------------------------------------------------- helpers
def _as3(x):
    if isinstance(x, (int, np.integer)):
        return (int(x),) * 3
    x = tuple(int(v) for v in x)
    assert len(x) == 3
    return x


def pad_rows(n: int, div: int = CTA_M) -> int:
    return (n + div - 1) // div * div


def kernel_digits(kernel_size) -> np.ndarray:
    """Digits (dx,dy,dz) of every kernel index k.

    Odd kernel volume: x is the fastest digit; even volume: z is the fastest
    (torchsparse/backend/others/sparsemapping_cuda.cu:165-170,209-214;
    torchsparse/nn/utils/kernel.py:28-35).
    """
    kx, ky, kz = _as3(kernel_size)
    kvol = kx * ky * kz
    k = np.arange(kvol)
    if kvol % 2 == 1:
        dx = k % kx
        dy = (k // kx) % ky
        dz = k // (kx * ky)
    else:
        dz = k % kz
        dy = (k // kz) % ky
        dx = k // (kz * ky)
    return np.stack([dx, dy, dz], axis=1).astype(np.int64)


def ravel(coords: np.ndarray, cmin, cmax) -> np.ndarray:
    """Mixed-radix index of (b,x,y,z) with radices max-min+1
    (torchsparse/backend/others/sparsemapping_cuda.cu:12-26)."""
    cmin = np.asarray(cmin, dtype=np.int64)
    cmax = np.asarray(cmax, dtype=np.int64)
    sizes = cmax - cmin + 1
    c = coords.astype(np.int64)
    cur = np.zeros(c.shape[0], dtype=np.int64)
    for i in range(4):
        cur = cur * sizes[i] + (c[:, i] - cmin[i])
    return cur


def unravel(keys: np.ndarray, cmin, cmax) -> np.ndarray:
    """Inverse of :func:`ravel` (sparsemapping_cuda.cu:28-42)."""
    cmin = np.asarray(cmin, dtype=np.int64)
    cmax = np.asarray(cmax, dtype=np.int64)
    sizes = cmax - cmin + 1
    cur = keys.astype(np.int64).copy()
    out = np.zeros((keys.shape[0], 4), dtype=np.int64)
    for i in range(3, -1, -1):
        out[:, i] = cmin[i] + cur % sizes[i]
        cur //= sizes[i]
    return out.astype(np.int32)


class _Lookup:
    """Exact-match key -> row lookup (stands in for the GPU hash table:
    value = row, miss = -1; torchsparse/backend/hashmap/hashmap_cuda.cuh:316-347)."""

    def __init__(self, keys: np.ndarray):
        self.order = np.argsort(keys, kind="stable")
        self.sorted = keys[self.order]

    def __call__(self, q: np.ndarray) -> np.ndarray:
        if self.sorted.size == 0:
            return np.full(q.shape, -1, dtype=np.int64)
        pos = np.searchsorted(self.sorted, q)
        pos = np.minimum(pos, self.sorted.size - 1)
        hit = self.sorted[pos] == q
        return np.where(hit, self.order[pos], -1)


def _in_bounds(c: np.ndarray, cmin, cmax) -> np.ndarray:
    ok = np.ones(c.shape[0], dtype=bool)
    for i in (1, 2, 3):
        ok &= (c[:, i] >= cmin[i]) & (c[:, i] <= cmax[i])
    return ok


# --------------------------------------------------------------------------- bounds
def coords_bounds(coords, kernel_size, stride, padding, subm, spatial_range=None, allow_negative=False):
    """coords_min / coords_max as the Python side of the reference derives them
    (torchsparse/nn/functional/conv/kmap/func/hashmap_on_the_fly.py:24-45).

    ``spatial_range`` here is the already-strided *output* range
    (torchsparse/nn/functional/conv/kmap/build_kmap.py:65-72)."""
    ks = np.array(_as3(kernel_size), dtype=np.int64)
    st = np.array(_as3(stride), dtype=np.int64)
    pd = np.array(_as3(padding), dtype=np.int64)
    if spatial_range is not None:
        cmax = np.array([v - 1 for v in spatial_range], dtype=np.int64)
    elif coords.shape[0] == 0:
        cmax = np.zeros(4, dtype=np.int64)
    else:
        cmax = coords.astype(np.int64).max(axis=0)
        if not subm:
            # floor division, as torch's ``//`` on integer tensors
            cmax[1:] = np.floor_divide(cmax[1:] + 2 * pd - (ks - 1), st)
    cmin = np.zeros(4, dtype=np.int64)
    if allow_negative and coords.shape[0]:
        # torchsparse.tensor.get_allow_negative_coordinates() branch (hashmap_on_the_fly.py:39-43):
        # torch.div is a true division; storing it into the int tensor truncates toward zero
        cmin = coords.astype(np.int64).min(axis=0)
        cmin[1:] = np.trunc((cmin[1:] - 2 * pd + (ks - 1)) / st).astype(np.int64)
    return cmin, cmax


# --------------------------------------------------------------------------- maps
def subm_map(coords, kernel_size, cmin, cmax):
    """Submanifold kernel map, all strides 1.  Returns int32 [pad128(N), Kvol].

    Odd kernel volume (sparsemapping_cuda.cu:144-188): for k < Kvol/2 the
    neighbour at coords + (d - (ks-1)/2) is looked up (bounds on x,y,z against
    cmin/cmax) and, when present, written both at [row][k] and mirrored at
    [nbr][Kvol-1-k]; the centre column is the row itself.
    Even kernel volume (sparsemapping_cuda.cu:192-231): offsets are d in
    [0, ks) (not centred), no mirroring.
    """
    ks = _as3(kernel_size)
    kvol = ks[0] * ks[1] * ks[2]
    n = coords.shape[0]
    digits = kernel_digits(ks)
    out = np.full((pad_rows(n), kvol), -1, dtype=np.int32)
    if n == 0:
        return out
    look = _Lookup(ravel(coords, cmin, cmax))
    c64 = coords.astype(np.int64)
    rows = np.arange(n)
    if kvol % 2 == 1:
        half = np.array([(k - 1) // 2 for k in ks], dtype=np.int64)
        out[:n, kvol // 2] = rows
        for k in range(kvol // 2):
            nb = c64.copy()
            nb[:, 1:] += digits[k] - half
            ok = _in_bounds(nb, cmin, cmax)
            idx = np.full(n, -1, dtype=np.int64)
            idx[ok] = look(ravel(nb[ok], cmin, cmax))
            hit = idx >= 0
            out[rows[hit], k] = idx[hit]
            out[idx[hit], kvol - 1 - k] = rows[hit]
    else:
        for k in range(kvol):
            nb = c64.copy()
            nb[:, 1:] += digits[k]
            ok = _in_bounds(nb, cmin, cmax)
            idx = np.full(n, -1, dtype=np.int64)
            idx[ok] = look(ravel(nb[ok], cmin, cmax))
            hit = idx >= 0
            out[rows[hit], k] = idx[hit]
    return out


def _trunc_mod(a, b):
    """C++ ``%`` (sign follows the dividend)."""
    return np.fmod(a, b)


def _trunc_div(a, b):
    """C++ integer ``/`` (rounds toward zero)."""
    q = np.abs(a) // np.abs(b)
    return np.where((a < 0) ^ (b < 0), -q, q)


def downsample_map(coords, kernel_size, stride, padding, cmin, cmax_out):
    """Strided kernel map.  Returns (out_in_map int32 [pad128(M),Kvol],
    out_coords int32 [M,4]).

    Stage 1 (sparsemapping_cuda.cu:60-107): per (input, k') with digit offset
    d' - (ks-1): c = in + pad + offset; kept iff c % stride == 0 (C++ ``%``) on
    every dim, then c /= stride and the result lies within
    [cmin, cmax_out] on x,y,z.  Outputs are the sorted unique ravel indices
    (torch::_unique, sparsemapping_cuda.cu:478), i.e. ascending (b,x,y,z).
    Stage 3 (sparsemapping_cuda.cu:110-126): map[out][Kvol-1-k'] = in.
    """
    ks = np.array(_as3(kernel_size), dtype=np.int64)
    st = np.array(_as3(stride), dtype=np.int64)
    pd = np.array(_as3(padding), dtype=np.int64)
    kvol = int(ks.prod())
    n = coords.shape[0]
    digits = kernel_digits(tuple(ks))
    c64 = coords.astype(np.int64)
    cand_key = np.full((n, kvol), -1, dtype=np.int64)
    for k in range(kvol):
        off = digits[k] - (ks - 1)
        c = c64.copy()
        c[:, 1:] = c64[:, 1:] + pd + off
        ok = np.ones(n, dtype=bool)
        for i in range(3):
            ok &= _trunc_mod(c[:, 1 + i], st[i]) == 0
            c[:, 1 + i] = _trunc_div(c[:, 1 + i], st[i])
        ok &= _in_bounds(c, cmin, cmax_out)
        cand_key[ok, k] = ravel(c[ok], cmin, cmax_out)
    valid = cand_key >= 0
    uniq = np.unique(cand_key[valid])
    m = uniq.shape[0]
    out_coords = unravel(uniq, cmin, cmax_out)
    out_in_map = np.full((pad_rows(m), kvol), -1, dtype=np.int32)
    if m:
        ii, kk = np.nonzero(valid)
        oo = np.searchsorted(uniq, cand_key[ii, kk])
        out_in_map[oo, kvol - 1 - kk] = ii
    return out_in_map, out_coords


def transpose_map(out_in_map, n_rows_pad):
    """map_t[in][k] = out for every map[out][k] = in
    (torchsparse/backend/others/query_cuda.cu:9-15;
    torchsparse/nn/functional/conv/hash/query.py:47-55)."""
    kvol = out_in_map.shape[1]
    out = np.full((n_rows_pad, kvol), -1, dtype=np.int32)
    oo, kk = np.nonzero(out_in_map >= 0)
    out[out_in_map[oo, kk], kk] = oo
    return out


# --------------------------------------------------------------------------- sorted-map artefacts
def derive_bitmask(out_in_map, split_mask_num, valid_n):
    """Per-row neighbour bitmask per split, -1 for rows >= valid_n
    (torchsparse/backend/others/query_cuda.cu:17-31,59-65)."""
    rows, kvol = out_in_map.shape
    split_len = (kvol + split_mask_num - 1) // split_mask_num
    out = np.full((split_mask_num, rows), -1, dtype=np.int32)
    for s in range(split_mask_num):
        lo = s * split_len
        ln = split_len if s != split_mask_num - 1 else kvol - lo
        bits = np.zeros(valid_n, dtype=np.int64)
        for i in range(ln):
            bits += (out_in_map[:valid_n, lo + i] >= 0).astype(np.int64) << i
        out[s, :valid_n] = bits.astype(np.int32)
    return out


def sort_bitmask(bitmask):
    """Descending sort per split; ties keep ascending row order.  The reference
    uses torch.sort (hashmap_on_the_fly.py:96) whose tie order is unspecified, so
    only the sorted values are pinned; a stable order is chosen here."""
    loc = np.argsort(-bitmask.astype(np.int64), axis=1, kind="stable").astype(np.int32)
    sorted_mask = np.take_along_axis(bitmask, loc.astype(np.int64), axis=1)
    return sorted_mask, loc


def reorder_map(out_in_map, reorder_loc):
    """reordered[r][c] = map[loc[split(c)][r]][c]
    (torchsparse/backend/others/reorder_map_cuda.cu:8-23)."""
    rows, kvol = out_in_map.shape
    split = reorder_loc.shape[0]
    split_len = (kvol + split - 1) // split
    out = np.empty_like(out_in_map)
    for c in range(kvol):
        out[:, c] = out_in_map[reorder_loc[c // split_len].astype(np.int64), c]
    return out


def reduce_bitmask(bitmask, tile):
    """OR over each tile of ``tile`` rows
    (torchsparse/backend/others/reduce_bitmask_cuda.cu:14-57)."""
    split, rows = bitmask.shape
    n_red = (rows - 1) // tile + 1
    out = np.zeros((split, n_red), dtype=np.int32)
    for t in range(n_red):
        seg = bitmask[:, t * tile:(t + 1) * tile]
        out[:, t] = np.bitwise_or.reduce(seg, axis=1)
    return out


# --------------------------------------------------------------------------- pair lists (GatherScatter / FetchOnDemand)
def pairs_from_map(out_in_map):
    """nbmaps int32 [P,2] = (in, out) grouped by k, ascending out; nbsizes [Kvol]
    (torchsparse/nn/functional/conv/kmap/func/hashmap_on_the_fly.py:138-141)."""
    res = out_in_map.T  # [Kvol, rows]
    kk, oo = np.nonzero(res != -1)
    nbmaps = np.stack([res[kk, oo], oo], axis=1).astype(np.int32)
    nbsizes = (res != -1).sum(axis=1).astype(np.int32)
    return nbmaps, nbsizes


def scan_quantified(nbsizes, q=128):
    """nbaddrs / qnbaddrs exclusive scans of length Kvol+1
    (torchsparse/backend/others/exclusive_scan_cuda.cu:7-29)."""
    kvol = nbsizes.shape[0]
    a = np.zeros(kvol + 1, dtype=np.int32)
    qa = np.zeros(kvol + 1, dtype=np.int32)
    a[1:] = np.cumsum(nbsizes)
    qa[1:] = np.cumsum((nbsizes + q - 1) // q * q)
    return a, qa


def masks_from_pairs(n_in, n_out, nbmaps, nbsizes):
    """input_mask[k*N+in] = output_mask[k*M+out] = position inside offset k,
    centre offset skipped for odd submanifold maps
    (torchsparse/backend/others/sparsemapping_cuda.cu:235-256)."""
    kvol = nbsizes.shape[0]
    im = np.full(kvol * n_in, -1, dtype=np.int32)
    om = np.full(kvol * n_out, -1, dtype=np.int32)
    start = 0
    for k in range(kvol):
        sz = int(nbsizes[k])
        if not (n_in == n_out and kvol % 2 == 1 and k == kvol // 2):
            seg = nbmaps[start:start + sz]
            pos = np.arange(sz, dtype=np.int32)
            im[k * n_in + seg[:, 0]] = pos
            om[k * n_out + seg[:, 1]] = pos
        start += sz
    return im, om


# --------------------------------------------------------------------------- convolution value
def conv_from_map(feats, weight, out_in_map, n_out, dtype=np.float64):
    """y[m] = sum_{k: map[m][k] >= 0} x[map[m][k]] @ W[k], accumulated in ``dtype``
    (the contraction every dataflow of the reference computes, e.g.
    torchsparse/backend/convolution/convolution_forward_implicit_gemm_cuda.cu:113-129)."""
    x = feats.astype(dtype)
    w = weight.astype(dtype)
    kvol = w.shape[0]
    y = np.zeros((n_out, w.shape[2]), dtype=dtype)
    for k in range(kvol):
        col = out_in_map[:n_out, k]
        rows = np.nonzero(col >= 0)[0]
        if rows.size:
            y[rows] += x[col[rows]] @ w[k]
    return y


def conv_backward_from_map(feats, weight, out_in_map, n_out, grad_out, dtype=np.float64):
    """Gradients of y = conv_from_map(feats, weight, out_in_map, n_out) for an upstream grad_out:
    dX[map[m][k]] += dY[m] @ W[k]^T and dW[k] += X[map[m][k]]^T @ dY[m]
    (the sums the reference's dgrad / wgrad kernels compute,
    torchsparse/nn/functional/conv/func/implicit_gemm.py:108-193)."""
    x = feats.astype(dtype)
    w = weight.astype(dtype)
    dy = grad_out.astype(dtype)
    dx = np.zeros_like(x)
    dw = np.zeros_like(w)
    for k in range(w.shape[0]):
        col = out_in_map[:n_out, k]
        rows = np.nonzero(col >= 0)[0]
        if rows.size:
            np.add.at(dx, col[rows], dy[rows] @ w[k].T)
            dw[k] = x[col[rows]].T @ dy[rows]
    return dx, dw


def conv_from_pairs(feats, weight, nbmaps, nbsizes, n_out, transpose=False, dtype=np.float64):
    """Gather -> matmul -> scatter-add per kernel offset
    (torchsparse/backend/convolution/convolution_gather_scatter_cpu.cpp:38-109)."""
    x = feats.astype(dtype)
    w = weight.astype(dtype)
    y = np.zeros((n_out, w.shape[2]), dtype=dtype)
    start = 0
    for k in range(w.shape[0]):
        sz = int(nbsizes[k])
        seg = nbmaps[start:start + sz]
        i_col, o_col = (1, 0) if transpose else (0, 1)
        np.add.at(y, seg[:, o_col], x[seg[:, i_col]] @ w[k])
        start += sz
    return y


# --------------------------------------------------------------------------- hashing / point ops / quantize
_FNV_OFFSET = np.uint64(14695981039346656037)
_FNV_PRIME = np.uint64(1099511628211)


def fnv_hash(coords, fold60=False):
    """FNV-1a-64 over the four int32 columns.  The CUDA build of the reference
    returns the raw 64-bit value (torchsparse/backend/hash/hash_cuda.cu:9-22);
    its CPU build additionally folds to 60 bits (hash_cpu.cpp:15)."""
    with np.errstate(over="ignore"):
        h = np.full(coords.shape[0], _FNV_OFFSET, dtype=np.uint64)
        for j in range(4):
            h ^= coords[:, j].astype(np.uint32).astype(np.uint64)
            h *= _FNV_PRIME
        if fold60:
            h = (h >> np.uint64(60)) ^ (h & np.uint64(0xFFFFFFFFFFFFFFF))
    return h.view(np.int64)


def kernel_fnv_hash(coords, offsets):
    """Hash of coords + offset for every offset -> [K, N]
    (torchsparse/backend/hash/hash_cuda.cu:26-54: columns 1..3 are shifted,
    column 0 is kept)."""
    out = np.empty((offsets.shape[0], coords.shape[0]), dtype=np.int64)
    for k in range(offsets.shape[0]):
        c = coords.copy()
        c[:, 1:] = coords[:, 1:] + offsets[k]
        out[k] = fnv_hash(c)
    return out


def hash_query(queries, references):
    """Row of each query key inside references, -1 if absent
    (torchsparse/nn/functional/query.py:8-37)."""
    return _Lookup(references)(queries).astype(np.int64)


def count(idx, n):
    """Histogram of non-negative indices (torchsparse/backend/others/count_cuda.cu:10-16)."""
    ok = idx >= 0
    return np.bincount(idx[ok], minlength=n).astype(np.int32)


def voxelize(feats, idx, counts):
    """out[idx[i]] += feats[i] / counts[idx[i]]
    (torchsparse/backend/voxelize/voxelize_cpu.cpp:7-26)."""
    out = np.zeros((counts.shape[0], feats.shape[1]), dtype=np.float64)
    ok = counts[idx] != 0
    np.add.at(out, idx[ok], feats[ok].astype(np.float64) / counts[idx[ok]][:, None])
    return out


def devoxelize(feats, indices, weights):
    """out[i] = sum_k w[i][k] * feats[indices[i][k]] (index -1 contributes 0)
    (torchsparse/backend/devoxelize/devoxelize_cpu.cpp:9-31)."""
    f = feats.astype(np.float64)
    out = np.zeros((indices.shape[0], feats.shape[1]), dtype=np.float64)
    for k in range(8):
        ix = indices[:, k]
        ok = ix >= 0
        out[ok] += weights[ok, k].astype(np.float64)[:, None] * f[ix[ok]]
    return out


def sparse_quantize(coords, voxel_size=1, return_index=False, return_inverse=False):
    """floor(coords / voxel) -> int32, unique by ravel hash in ascending order,
    first-occurrence index and inverse map
    (torchsparse/utils/quantize.py:9-48)."""
    if isinstance(voxel_size, (float, int)):
        voxel_size = (voxel_size,) * 3
    vs = np.array(voxel_size)
    q = np.floor(coords / vs).astype(np.int32)
    x = (q - q.min(axis=0)).astype(np.uint64)
    xmax = x.max(axis=0).astype(np.uint64) + np.uint64(1)
    h = (x[:, 0] * xmax[1] + x[:, 1]) * xmax[2] + x[:, 2]
    _, index, inverse = np.unique(h, return_index=True, return_inverse=True)
    outs = [q[index]]
    if return_index:
        outs.append(index)
    if return_inverse:
        outs.append(inverse)
    return outs[0] if len(outs) == 1 else outs


# --------------------------------------------------------------------------- one-call kernel-map builder
def build_kmap_hashmap_mode(coords, kernel_size, stride=1, padding=0, spatial_range=None):
    """The kernel map of ``kmap_mode="hashmap"``
    (torchsparse/nn/functional/conv/kmap/func/hashmap.py:8-105, kmap/downsample.py:11-79,
    backend/hashmap/hashmap_cuda.cuh:200-254): output coordinates = unique rows of floor(c / stride) when
    every stride is 1 or the kernel size, else the natively enumerated strided outputs; for output row i
    and kernel index k the input at ``out * stride + digit_k - (kernel - 1) // 2`` (x the fastest digit
    for an odd kernel volume, z for an even one), -1 when there is none.  Padding plays no part in the
    lookup.  Coordinates are matched exactly (the reference matches 64-bit FNV hashes of them)."""
    ks, st, pd = _as3(kernel_size), _as3(stride), _as3(padding)
    subm = not any(s > 1 for s in st)
    coords = np.asarray(coords, dtype=np.int32)
    if subm:
        out_coords = coords
    elif all(st[i] in (1, ks[i]) for i in range(3)):
        c = coords.astype(np.int64).copy()
        c[:, 1:] = np.floor(c[:, 1:] / np.array(st, dtype=np.float64)).astype(np.int64)
        out_coords = np.unique(c, axis=0).astype(np.int32)
    else:
        new_range = None
        if spatial_range is not None:               # the strided output range, as build_kmap derives it
            new_range = (spatial_range[0],) + tuple(
                (spatial_range[i + 1] + 2 * pd[i] - (ks[i] - 1) - 1) // st[i] + 1 for i in range(3))
        cmin, cmax = coords_bounds(coords, ks, st, pd, False, new_range)
        out_coords = downsample_map(coords, ks, st, pd, cmin, cmax)[1]
    index = {tuple(int(v) for v in row): i for i, row in enumerate(coords)}
    kvol = ks[0] * ks[1] * ks[2]
    m = out_coords.shape[0]
    out = np.full(((m + 127) // 128 * 128, kvol), -1, dtype=np.int32)
    digits = kernel_digits(ks)
    for i in range(m):
        b, x, y, z = (int(v) for v in out_coords[i])
        for k in range(kvol):
            dx, dy, dz = (int(v) for v in digits[k])
            key = (b, x * st[0] + dx - (ks[0] - 1) // 2, y * st[1] + dy - (ks[1] - 1) // 2,
                   z * st[2] + dz - (ks[2] - 1) // 2)
            out[i, k] = index.get(key, -1)
    return {"out_in_map": out, "coords": out_coords, "sizes": (coords.shape[0], m)}


def build_kmap_generative(coords, kernel_size, stride, padding, spatial_range):
    """The kernel map of a generative transposed convolution
    (torchsparse/nn/functional/conv/kmap/upsample.py:12-38, kmap/func/hashmap.py:37-40, 58-64, 74-83,
    kmap/build_kmap.py:65-72).  ``spatial_range`` is the INPUT tensor's (batch, x, y, z) range; as in the reference the
    generated coordinates are clamped to the range the strided-convolution formula derives from it.  Output rows:
    unique (lexicographic) rows of clamp(coords * stride + cell offset) over the cells of a stride-1 kernel; entry
    (row, k) = the input whose coords * stride equals output + digit_k - (kernel - 1) // 2, else -1."""
    ks, st, pd = _as3(kernel_size), _as3(stride), _as3(padding)
    coords = np.asarray(coords, dtype=np.int32)
    new_range = (spatial_range[0],) + tuple(
        (spatial_range[i + 1] + 2 * pd[i] - (ks[i] - 1) - 1) // st[i] + 1 for i in range(3))
    digits = kernel_digits(ks)
    offs = digits.astype(np.int64) - np.array([(k - 1) // 2 for k in ks], dtype=np.int64)
    scaled = coords.astype(np.int64).copy()
    scaled[:, 1:] *= np.array(st, dtype=np.int64)
    gen = np.repeat(scaled[:, None, :], offs.shape[0], axis=1)
    gen[:, :, 1:] += offs[None, :, :]
    for i in range(1, 4):
        gen[:, :, i] = np.clip(gen[:, :, i], 0, new_range[i] - 1)
    out_coords = np.unique(gen.reshape(-1, 4), axis=0).astype(np.int32)
    index = {tuple(int(v) for v in row): i for i, row in enumerate(scaled)}
    kvol = offs.shape[0]
    m = out_coords.shape[0]
    out = np.full(((m + 127) // 128 * 128, kvol), -1, dtype=np.int32)
    for i in range(m):
        b, x, y, z = (int(v) for v in out_coords[i])
        for k in range(kvol):
            dx, dy, dz = (int(v) for v in offs[k])
            out[i, k] = index.get((b, x + dx, y + dy, z + dz), -1)
    return {"out_in_map": out, "coords": out_coords, "sizes": (coords.shape[0], m), "spatial_range": new_range}


def build_kmap(coords, kernel_size, stride=1, padding=0, spatial_range=None, allow_negative=False):
    """The ``hashmap_on_the_fly`` kernel map as a dict with the reference's keys
    (torchsparse/nn/functional/conv/kmap/func/hashmap_on_the_fly.py:10-109)."""
    ks, st, pd = _as3(kernel_size), _as3(stride), _as3(padding)
    subm = not any(s > 1 for s in st)
    new_range = None
    if spatial_range is not None:
        new_range = (spatial_range[0],) + tuple(
            (spatial_range[i + 1] + 2 * pd[i] - (ks[i] - 1) - 1) // st[i] + 1 for i in range(3))
    cmin, cmax = coords_bounds(coords, ks, st, pd, subm, new_range, allow_negative)
    if subm:
        m = subm_map(coords, ks, cmin, cmax)
        out_coords = coords
    else:
        m, out_coords = downsample_map(coords, ks, st, pd, cmin, cmax)
    return {"out_in_map": m, "coords": out_coords,
            "sizes": (coords.shape[0], out_coords.shape[0]), "spatial_range": new_range}
