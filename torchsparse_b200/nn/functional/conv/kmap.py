"""Kernel-map construction: orchestration of the native map kernels and the host-side
bookkeeping (bounds, table sizing, caches).

Follows torchsparse/nn/functional/conv/kmap/build_kmap.py:19-309 and
kmap/func/hashmap_on_the_fly.py:10-207 in what it produces (same dictionary keys, same
tensors), but is organised for few device->host reads: coordinate bounds live on the host
(one read per tensor stride, cached next to the kernel maps) and a strided build reads
back one 8-int record (the reference reads two scalars and reduces ``coords.max`` on the
device for every build)."""
from typing import Dict, Optional, Tuple, Union

import torch

from .... import backend, backends
from ....utils.utils import make_ntuple, make_divisible
from .conv_config import Dataflow

__all__ = ["build_kernel_map", "transpose_kernel_map", "convert_transposed_out_in_map"]

cta_M = 128


def _next_pow2(n: int) -> int:
    p = 1
    while p < n:
        p <<= 1
    return p


def _table_capacity(n: int) -> int:
    assert backends.hash_rsv_ratio >= 2, (
        f"hash_rsv_ratio should be no less than 2, now {backends.hash_rsv_ratio}.")
    return _next_pow2(max(512, int(backends.hash_rsv_ratio * n)))


def _actual_bounds(coords: torch.Tensor, caches, tensor_stride):
    """(min, max) of the coordinates as host tuples; cached per tensor stride."""
    from ....tensor import get_allow_negative_coordinates

    if caches is not None and tensor_stride in caches.cbounds:
        return caches.cbounds[tensor_stride]
    if coords.shape[0] == 0:
        b = ((0, 0, 0, 0), (0, 0, 0, 0))
    elif get_allow_negative_coordinates():
        mm = torch.stack([coords.min(0).values, coords.max(0).values]).cpu().tolist()
        b = (tuple(mm[0]), tuple(mm[1]))
    else:
        b = ((0, 0, 0, 0), tuple(coords.max(0).values.cpu().tolist()))
    if caches is not None:
        caches.cbounds[tensor_stride] = b
    return b


def convert_transposed_out_in_map(out_in_map: torch.Tensor, size: int) -> torch.Tensor:
    """(torchsparse/nn/functional/conv/hash/query.py:47-55); the -1 fill is fused into the call."""
    out_in_map_t = torch.empty((size, out_in_map.shape[1]), device=out_in_map.device, dtype=torch.int32)
    backend.convert_transposed_out_in_map(out_in_map, out_in_map_t, fill=True)
    return out_in_map_t


def _sorted_artefacts(out_in_map: torch.Tensor, split_mask_num: int, valid_n: int, tile: int = cta_M):
    if split_mask_num == 1:
        return backend.sorted_artefacts_cuda(out_in_map, valid_n, tile)
    bitmask = backend.derive_bitmask_from_out_in_map(out_in_map, split_mask_num, valid_n)
    sorted_mask, reorder_loc = backend.sort_bitmask_cuda(bitmask, out_in_map.shape[1])
    reorder_out_in_map = backend.reorder_out_in_map_cuda(out_in_map, reorder_loc)
    reduced = backend.reduce_bitmask_cuda(sorted_mask, tile)
    return sorted_mask, reorder_loc, reorder_out_in_map, reduced


def build_kernel_map(
    _coords: torch.Tensor,
    input_node_num: int,
    kernel_size: Union[int, Tuple[int, ...]] = 2,
    stride: Union[int, Tuple[int, ...]] = 2,
    padding: Union[int, Tuple[int, ...]] = 0,
    hashmap_keys: Optional[torch.Tensor] = None,
    hashmap_vals: Optional[torch.Tensor] = None,
    spatial_range=None,
    mode: str = "hashmap_on_the_fly",
    dataflow=Dataflow.ImplicitGEMM,
    downsample_mode: str = "spconv",
    training: bool = False,
    ifsort: bool = False,
    generative: bool = False,
    split_mask_num: int = 1,
    split_mask_num_bwd: int = 1,
    *,
    caches=None,
    tensor_stride: Optional[Tuple[int, ...]] = None,
) -> Dict:
    """Build the kernel map of one convolution.  Returns the dictionary of the reference
    (``out_in_map``, ``coords``, ``sizes``, ``hashmap_keys/vals``, ``spatial_range``, sorted
    artefacts, pair lists ...).  ``caches`` / ``tensor_stride`` let the host-side bounds and
    the ravel bounds of a reused table be looked up instead of recomputed."""
    if mode not in ("hashmap_on_the_fly", "hashmap"):
        raise ValueError(f"unknown kmap_mode {mode!r}")
    if generative and mode != "hashmap":
        raise ValueError(
            f"Unsupported kmap_mode: {mode} for generative convolution (please switch to kmap_mode=hashmap).")
    kmap = dict.fromkeys(
        ["out_in_map", "coords", "sizes", "reorder_out_in_map", "reduced_sorted_mask", "reorder_loc", "nbmaps",
         "nbsizes", "input_mask", "output_mask", "nbaddrs", "qnbaddrs", "qmapsize"])
    stride = make_ntuple(stride, ndim=3)
    kernel_size = make_ntuple(kernel_size, ndim=3)
    padding = make_ntuple(padding, ndim=3)
    new_range = None
    if spatial_range is not None:
        new_range = (spatial_range[0],) + tuple(
            (spatial_range[i + 1] + 2 * padding[i] - (kernel_size[i] - 1) - 1) // stride[i] + 1 for i in range(3))
    kmap["spatial_range"] = new_range
    subm = not any(s > 1 for s in stride)
    coords = _coords.contiguous()
    n = coords.shape[0]
    if mode == "hashmap":
        if generative:
            hashmap_keys, hashmap_vals = _generative_map(kmap, coords, kernel_size, stride, padding, new_range)
        else:
            hashmap_keys, hashmap_vals = _hashmap_mode_map(kmap, coords, kernel_size, stride, padding, new_range,
                                                           subm, downsample_mode, caches, tensor_stride)
        return _finish_kernel_map(kmap, n, input_node_num, hashmap_keys, hashmap_vals, dataflow, ifsort,
                                  split_mask_num)
    cmin_act, cmax_act = _actual_bounds(coords, caches, tensor_stride)
    from ....tensor import get_allow_negative_coordinates
    if get_allow_negative_coordinates():
        # lower bound of the key space as the reference derives it
        # (torchsparse/nn/functional/conv/kmap/func/hashmap_on_the_fly.py:39-43): a true division whose
        # result is truncated toward zero when it is stored back into the integer tensor
        cmin_key = (cmin_act[0],) + tuple(
            int((cmin_act[1 + i] - 2 * padding[i] + (kernel_size[i] - 1)) / stride[i]) for i in range(3))
    else:
        cmin_key = (0, 0, 0, 0)

    if subm:
        table_bounds = caches.hash_bounds.get(tensor_stride) if (caches is not None and hashmap_keys is not None) else None
        if table_bounds == _FNV_TABLE:          # a table of the other kmap_mode cannot serve ravel keys
            table_bounds, hashmap_keys, hashmap_vals = None, None, None
        if table_bounds is not None:
            cmin, cmax = table_bounds
        elif new_range is not None:
            cmin, cmax = cmin_key, tuple(v - 1 for v in new_range)
        else:
            cmin, cmax = cmin_key, cmax_act
        to_insert = hashmap_keys is None or table_bounds is None
        if to_insert:
            hashmap_keys, hashmap_vals = backend.new_table(_table_capacity(n), coords.device, cmin, cmax)
        table = backend.table_of(hashmap_keys, hashmap_vals)
        kmap["out_in_map"] = backend.build_kernel_map_subm_hashmap(
            table, coords, cmin, cmax, kernel_size, stride, padding, to_insert, check_status=False)[0]
        kmap["coords"] = _coords
        kmap["table_stride"] = tensor_stride
        kmap["table_bounds"] = (cmin, cmax)
    else:
        if new_range is not None:
            cmax_out = tuple(v - 1 for v in new_range)
        else:
            cmax_out = (cmax_act[0],) + tuple(
                (cmax_act[1 + i] + 2 * padding[i] - (kernel_size[i] - 1)) // stride[i] for i in range(3))
        cmin_out = cmin_key
        uniq, m, out_max = backend.downsample_unique(coords, cmin_out, cmax_out, kernel_size, stride, padding)
        hashmap_keys, hashmap_vals = backend.new_table(_table_capacity(max(n, m)), coords.device, cmin_out, cmax_out)
        table = backend.table_of(hashmap_keys, hashmap_vals)
        out_in_map, out_coords = backend.downsample_finish(table, coords, uniq, m, cmin_out, cmax_out, kernel_size,
                                                           stride, padding, check_status=False)
        kmap["out_in_map"] = out_in_map
        kmap["coords"] = out_coords
        kmap["table_stride"] = (None if tensor_stride is None
                                else tuple(tensor_stride[i] * stride[i] for i in range(3)))
        kmap["table_bounds"] = (cmin_out, cmax_out)
        kmap["out_bounds"] = (cmin_out, out_max if out_max is not None else cmin_out)
    return _finish_kernel_map(kmap, n, input_node_num, hashmap_keys, hashmap_vals, dataflow, ifsort, split_mask_num)


_FNV_TABLE = ("fnv",)    # `table_bounds` marker of a table keyed by coordinate hashes (kmap_mode="hashmap")


def _hashmap_mode_map(kmap, coords, kernel_size, stride, padding, spatial_range, subm, downsample_mode, caches,
                      tensor_stride):
    """kmap_mode="hashmap" (torchsparse/nn/functional/conv/kmap/func/hashmap.py:8-105): output
    coordinates from ``spdownsample``, input coordinates inserted into a table keyed by the FNV-1a hash
    of (x, y, z, b), and one lookup per (output row, kernel offset) at
    ``out * stride + digit - (kernel - 1) // 2``.  A table built for this tensor stride is reused."""
    from .downsample import spdownsample

    out_coords = coords if subm else spdownsample(coords, stride, kernel_size, padding, spatial_range,
                                                  downsample_mode=downsample_mode)
    keys = vals = None
    if caches is not None and caches.hash_bounds.get(tensor_stride) == _FNV_TABLE:
        keys, vals = caches.hashmaps.get(tensor_stride, (None, None))
    to_insert = keys is None
    if to_insert:
        cap = _table_capacity(coords.shape[0])
        keys = torch.zeros(cap, dtype=torch.int64, device=coords.device)
        vals = torch.zeros(cap, dtype=torch.int32, device=coords.device)
    table = backend.GPUHashTable(keys, vals)
    if to_insert:
        table.insert_coords(coords[:, [1, 2, 3, 0]])
    kvol = kernel_size[0] * kernel_size[1] * kernel_size[2]
    kmap["out_in_map"] = table.lookup_coords(out_coords[:, [1, 2, 3, 0]], kernel_size, stride, kvol) - 1
    kmap["coords"] = out_coords
    kmap["table_stride"] = tensor_stride
    kmap["table_bounds"] = _FNV_TABLE
    return keys, vals


def _generative_map(kmap, coords, kernel_size, stride, padding, spatial_range):
    """Kernel map of a generative transposed convolution
    (torchsparse/nn/functional/conv/kmap/func/hashmap.py:37-40, 58-64, 74-83): the output coordinates are generated
    from the inputs (``spupsample_generative``, clamped to ``spatial_range`` - the range the caller derived with the
    strided-convolution formula, as the reference does), the inputs are inserted at ``coords * stride``, and every
    (output row, kernel cell) looks up ``output + cell offset`` with stride 1."""
    from .upsample import spupsample_generative

    out_coords = spupsample_generative(coords, stride, kernel_size, padding, spatial_range)
    cap = _table_capacity(coords.shape[0])
    keys = torch.zeros(cap, dtype=torch.int64, device=coords.device)
    vals = torch.zeros(cap, dtype=torch.int32, device=coords.device)
    table = backend.GPUHashTable(keys, vals)
    scaled = coords.clone()
    scaled[:, 1:] *= torch.tensor(stride, dtype=coords.dtype, device=coords.device)
    table.insert_coords(scaled[:, [1, 2, 3, 0]])
    kvol = kernel_size[0] * kernel_size[1] * kernel_size[2]
    kmap["out_in_map"] = table.lookup_coords(out_coords[:, [1, 2, 3, 0]].contiguous(), kernel_size, (1, 1, 1), kvol) - 1
    kmap["coords"] = out_coords
    kmap["table_stride"] = None
    kmap["table_bounds"] = _FNV_TABLE
    return keys, vals


def _finish_kernel_map(kmap, n, input_node_num, hashmap_keys, hashmap_vals, dataflow, ifsort, split_mask_num):
    """The part of a build that does not depend on how out_in_map was found: sizes, sorted artefacts
    of the implicit GEMM, pair lists and masks of the other dataflows."""
    kmap["hashmap_keys"], kmap["hashmap_vals"] = hashmap_keys, hashmap_vals
    kmap["sizes"] = (input_node_num, kmap["coords"].shape[0])
    out_in_map = kmap["out_in_map"]

    if dataflow == Dataflow.ImplicitGEMM:
        if ifsort:
            sorted_mask, loc, reordered, reduced = _sorted_artefacts(out_in_map, split_mask_num, kmap["sizes"][1])
            kmap["reorder_out_in_map"], kmap["reduced_sorted_mask"] = reordered, reduced
            kmap["reorder_loc"], kmap["sorted_mask"] = loc, sorted_mask
    elif dataflow in (Dataflow.GatherScatter, Dataflow.FetchOnDemand):
        fod = dataflow == Dataflow.FetchOnDemand
        nbmaps, nbsizes, sizes_host, nbaddrs, qnbaddrs, qmapsize = backend.pairs_from_out_in_map(out_in_map, fod)
        kmap["nbmaps"], kmap["nbsizes"], kmap["nbsizes_host"] = nbmaps, nbsizes, sizes_host
        kmap["nbaddrs"], kmap["qnbaddrs"], kmap["qmapsize"] = nbaddrs, qnbaddrs, qmapsize
        if not fod:
            kmap["input_mask"], kmap["output_mask"] = _build_masks(n, kmap["sizes"][1], nbmaps, nbaddrs,
                                                                   len(sizes_host))
    else:
        raise ValueError("[Build kernel map] unsupported dataflow: {}".format(dataflow))

    for key in ("out_in_map_bwd", "reorder_out_in_map_bwd", "reduced_sorted_mask_bwd_wgrad",
                "reduced_sorted_mask_bwd_dgrad", "reorder_loc_bwd"):
        kmap[key] = None
    return kmap


def _build_masks(n_in, n_out, nbmaps, nbaddrs, kvol):
    from ...._lib import lib, check

    dev = nbmaps.device
    input_mask = torch.empty(kvol * n_in, dtype=torch.int32, device=dev)
    output_mask = torch.empty(kvol * n_out, dtype=torch.int32, device=dev)
    check(lib.tsb_build_masks(n_in, n_out, nbmaps.data_ptr(), nbaddrs.data_ptr(), kvol, nbmaps.shape[0],
                              input_mask.data_ptr(), output_mask.data_ptr(),
                              torch.cuda.current_stream().cuda_stream), "build_mask_from_kmap")
    return input_mask, output_mask


def transpose_kernel_map(kmap: Dict, ifsort: bool = False, training: bool = False, split_mask_num: int = 1,
                         split_mask_num_bwd: int = 1) -> Dict:
    """Adds the transposed map (and its sorted artefacts) of a strided conv's kmap, for the
    matching transposed conv (torchsparse/nn/functional/conv/kmap/build_kmap.py:224-309).
    The result is kept in the dictionary, so only the first transposed conv that uses a
    map pays for it (the reference rebuilds it on every call)."""
    if kmap is None:
        raise ValueError("transposed convolution needs the kernel map of the matching strided convolution, "
                         "which must have run earlier on the same tensor cache")
    if kmap.get("out_in_map_t") is None:
        kmap["out_in_map_t"] = convert_transposed_out_in_map(kmap["out_in_map"],
                                                             make_divisible(kmap["sizes"][0], cta_M))
    if ifsort and (kmap.get("reorder_out_in_map_t") is None or kmap.get("_split_t") != split_mask_num):
        _, loc, reordered, reduced = _sorted_artefacts(kmap["out_in_map_t"], split_mask_num, kmap["sizes"][0])
        kmap["reorder_out_in_map_t"], kmap["reduced_sorted_mask_t"], kmap["reorder_loc_t"] = reordered, reduced, loc
        kmap["_split_t"] = split_mask_num
    elif not ifsort:
        kmap.setdefault("reorder_out_in_map_t", None)
        kmap.setdefault("reduced_sorted_mask_t", None)
        kmap.setdefault("reorder_loc_t", None)
    for key in ("out_in_map_bwd_t", "reorder_out_in_map_bwd_t", "reduced_sorted_mask_bwd_wgrad_t",
                "reduced_sorted_mask_bwd_dgrad_t", "reorder_loc_bwd_t"):
        kmap[key] = None
    return kmap
