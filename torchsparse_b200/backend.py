"""Tensor-level operator interface with the names, argument meaning and error
behaviour of the reference's pybind module ``torchsparse.backend``
(torchsparse/backend/pybind_cuda.cu:29-83), implemented over the tsb200 C ABI.

Every function takes CUDA tensors, allocates its outputs with torch's caching
allocator (as the reference's native functions do with ``torch::empty/zeros``),
passes raw pointers plus torch's current stream to the library and raises
``ValueError`` / ``RuntimeError`` on a bad status.  There is no CPU path: CPU
tensors raise.

Differences from the reference that callers can see:
* kernels run on torch's *current* stream, not on the legacy default stream;
* ``coords_min`` / ``coords_max`` / ``kernel_sizes`` / ``stride`` / ``padding`` may
  be host tuples (preferred: no device read) as well as tensors;
* hash-table probes are bounded; a full table raises instead of hanging.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import lib, check, i32x

__all__ = [
    "GPUHashTable", "build_kernel_map_subm_hashmap", "build_kernel_map_downsample_hashmap",
    "build_mask_from_kmap", "convert_transposed_out_in_map", "derive_bitmask_from_out_in_map",
    "reduce_bitmask_cuda", "reorder_out_in_map_cuda", "sort_bitmask_cuda", "sorted_artefacts_cuda",
    "exclusive_scan_quantified_wrapper",
    "conv_forward_implicit_gemm_cuda", "conv_forward_implicit_gemm_sorted_cuda",
    "conv_forward_gather_scatter_cuda", "conv_backward_gather_scatter_cuda", "conv_wgrad_implicit_gemm_cuda",
    "conv_backward_wgrad_implicit_gemm_cuda", "conv_backward_wgrad_implicit_gemm_sorted_cuda",
    "conv_forward_fetch_on_demand_cuda", "downsample_cuda",
    "conv_forward_fetch_on_demand_no_fusion_cuda", "voxelize_forward_cuda", "devoxelize_forward_cuda",
    "voxelize_backward_cuda", "devoxelize_backward_cuda", "hash_cuda", "kernel_hash_cuda", "hash_query_cuda", "count_cuda", "to_dense_forward_cuda", "to_dense_backward_cuda",
    "pairs_from_out_in_map", "quantize_unique_cuda", "tile_mask_cuda", "sorted_cm_artefacts_cuda", "SortedMap",
]

_DTYPES = {torch.float32: _lib.TSB_F32, torch.float16: _lib.TSB_F16, torch.bfloat16: _lib.TSB_BF16}


_observer = None


def set_launch_observer(fn) -> None:
    """Install (or clear with None) a callback ``fn(name, dims, start_event, end_event)`` invoked
    around every convolution launch; used by the benchmark to time kernels on their own stream."""
    global _observer
    _observer = fn


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(lib.tsb_launch_count())


def _stream() -> int:
    # raw handle of torch's current stream on the current device (torch.cuda.current_stream() builds a
    # Stream object and costs ~15 us per call, which adds up over the launches of a network)
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


_status_words = {}


def _dev(device) -> torch.device:
    device = torch.device(device)
    return device if device.index is not None else torch.device("cuda", torch.cuda.current_device())


def _status_word(device: torch.device) -> torch.Tensor:
    """One persistent int32 status word per device for launches whose status nobody reads back
    (the kernels only ever write non-zero error codes into it)."""
    device = _dev(device)
    w = _status_words.get(device)
    if w is None:
        w = _status_words[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return w


def raise_if_kernel_failed(device: torch.device) -> None:
    """Reads the device's shared status word (a device-to-host read: call it where the stream is being waited for
    anyway) and raises if a bounded wait inside a convolution kernel ran out since the last check."""
    w = _status_words.get(_dev(device))
    if w is None:
        return
    v = int(w.item())
    if v:
        w.zero_()
        raise RuntimeError(f"a bounded wait inside a convolution kernel ran out (code {v}); results computed since "
                           "the last check are undefined")


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("torchsparse_b200.backend: CUDA tensors required (there is no CPU fallback)")


def _host_ints(x, n: int) -> Tuple[int, ...]:
    """Tuple of n ints from a tuple/list/int or a tensor (a device tensor costs a sync)."""
    if isinstance(x, torch.Tensor):
        x = x.detach().cpu().view(-1).tolist()
    elif isinstance(x, int):
        x = (x,) * n
    x = tuple(int(v) for v in x)
    if len(x) != n:
        raise ValueError(f"expected {n} integers, got {x}")
    return x


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise RuntimeError(f"unsupported feature dtype {t.dtype}") from None


def _workspace(nbytes: int, device) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def _check_dev_status(status: torch.Tensor, what: str) -> None:
    v = int(status.item())
    if v & _lib.TSB_DEV_TABLE_FULL:
        raise ValueError(
            f"{what}: the capacity of the hash table is not sufficient; enlarge the reserved space "
            "(torchsparse_b200.backends.hash_rsv_ratio)")
    if v & _lib.TSB_DEV_BAD_INDEX:
        raise RuntimeError(f"{what}: inconsistent hash table (an output coordinate was not found)")
    if v & _lib.TSB_DEV_LIMIT:
        raise ValueError(f"{what}: a key does not fit the table's 32-bit keys, or a device-side size went beyond "
                         "the bound stated by the caller")


def pad128(n: int) -> int:
    return (n + 127) // 128 * 128


# --------------------------------------------------------------------------- hash table
class GPUHashTable:
    """Mirror of class GPUHashTable (torchsparse/backend/hashmap/hashmap_cuda.cuh:65-118):
    either borrows ``(keys int64[cap], vals int32[cap])`` or owns a table of ``capacity``."""

    def __init__(self, keys_or_capacity, vals: Optional[torch.Tensor] = None, device=None):
        if isinstance(keys_or_capacity, int):
            dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
            self.keys = torch.zeros(keys_or_capacity, dtype=torch.int64, device=dev)
            self.vals = torch.zeros(keys_or_capacity, dtype=torch.int32, device=dev)
        else:
            self.keys, self.vals = keys_or_capacity, vals
            _need_cuda(self.keys, self.vals)
            if self.keys.dtype != torch.int64 or self.vals.dtype != torch.int32:
                raise ValueError("GPUHashTable expects int64 keys and int32 values")
            if self.keys.numel() != self.vals.numel() or not self.keys.is_contiguous() or not self.vals.is_contiguous():
                raise ValueError("GPUHashTable: keys and vals must be contiguous and of equal length")
        self.capacity = self.keys.numel()
        self.divisor = 128

    def get_capacity(self) -> int:
        return self.capacity

    def insert_vals(self, keys: torch.Tensor) -> None:
        _need_cuda(keys)
        keys = keys.contiguous()
        status = torch.zeros(1, dtype=torch.int32, device=keys.device)
        check(lib.tsb_hash_insert(_p(self.keys), _p(self.vals), self.capacity, _p(keys), keys.numel(), _p(status),
                                  _stream()), "GPUHashTable.insert_vals")
        _check_dev_status(status, "GPUHashTable.insert_vals")

    def lookup_vals(self, keys: torch.Tensor) -> torch.Tensor:
        _need_cuda(keys)
        keys = keys.contiguous()
        n = keys.numel()
        out = torch.zeros(pad128(n), dtype=torch.int32, device=keys.device)
        check(lib.tsb_hash_lookup(_p(self.keys), _p(self.vals), self.capacity, _p(keys), n, _p(out), _stream()),
              "GPUHashTable.lookup_vals")
        return out


    def insert_coords(self, coords: torch.Tensor) -> None:
        """Rows of int32 [n,4] in (x, y, z, batch) order, keyed by their FNV-1a hash, value = row + 1
        (torchsparse/backend/hashmap/hashmap_cuda.cuh:150-171, 273-277; the caller permutes the
        columns, torchsparse/nn/functional/conv/kmap/func/hashmap.py:60)."""
        self.insert_vals(hash_cuda(coords.int()))

    def lookup_coords(self, coords: torch.Tensor, kernel_sizes, strides, kernel_volume: int) -> torch.Tensor:
        """int32 [pad128(n), Kvol]: for row i and kernel index k the value stored for
        ``coords[i] * stride + digit_k - (kernel - 1) // 2`` (input row + 1), 0 when absent
        (torchsparse/backend/hashmap/hashmap_cuda.cuh:200-254, 307-314).  coords in (x, y, z, batch) order."""
        _need_cuda(coords)
        coords = coords.int().contiguous()
        ks, st = _host_ints(kernel_sizes, 3), _host_ints(strides, 3)
        kvol = ks[0] * ks[1] * ks[2]
        if int(kernel_volume) != kvol:
            raise ValueError("kernel_volume does not match kernel_sizes")
        n = coords.shape[0]
        out = torch.empty((pad128(n), kvol), dtype=torch.int32, device=coords.device)
        check(lib.tsb_hash_lookup_coords(_p(self.keys), _p(self.vals), self.capacity, _p(coords), n, _lib.i32x(ks),
                                         _lib.i32x(st), _p(out), _stream()), "GPUHashTable.lookup_coords")
        return out


class GPUHashTable32(GPUHashTable):
    """The table with 32-bit keys (class hashtable32 of torchsparse/backend/hashmap/hashmap_cuda.cuh, the table type of
    build_kernel_map_subm_hashmap_int32 / build_kernel_map_downsample_hashmap_int32,
    torchsparse/backend/others/sparsemapping_cuda.cu:259-300, 347-426): one 8-byte slot per entry, value << 32 | key,
    so an insert is one compare-and-swap and a probe one load.  Every builder that takes a ``GPUHashTable`` takes
    this one too and returns the same maps; key spaces of 2^32 or more raise."""

    def __init__(self, slots_or_capacity, device=None):
        if isinstance(slots_or_capacity, int):
            dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
            self.keys = torch.zeros(slots_or_capacity, dtype=torch.int64, device=dev)
        else:
            self.keys = slots_or_capacity
            _need_cuda(self.keys)
            if self.keys.dtype != torch.int64 or not self.keys.is_contiguous():
                raise ValueError("GPUHashTable32 expects a contiguous int64 tensor of packed slots")
        self.vals = None
        self.capacity = self.keys.numel()
        self.divisor = 128

    def insert_coords(self, coords: torch.Tensor) -> None:
        raise NotImplementedError("coordinate hashes are 64-bit: the hashmap kernel-map mode needs a GPUHashTable")

    def lookup_coords(self, coords, kernel_sizes, strides, kernel_volume):
        raise NotImplementedError("coordinate hashes are 64-bit: the hashmap kernel-map mode needs a GPUHashTable")


def fits_32bit_keys(coords_min, coords_max) -> bool:
    """True when every ravel key (index + 1) of the box [coords_min, coords_max] fits a 32-bit-key table."""
    total = 1
    for lo, hi in zip(coords_min, coords_max):
        total *= max(int(hi) - int(lo) + 1, 1)
    return total < 0xFFFFFFFF


def new_table(capacity: int, device, coords_min=None, coords_max=None):
    """Zeroed ``(keys, vals)`` of a table for ravel keys over the given box: packed 32-bit-key slots (``vals`` is None)
    when ``backends.hash_keys_32bit`` is set and the box allows it, else int64 keys + int32 values."""
    from . import backends

    keys = torch.zeros(capacity, dtype=torch.int64, device=device)
    if backends.hash_keys_32bit and coords_min is not None and fits_32bit_keys(coords_min, coords_max):
        return keys, None
    return keys, torch.zeros(capacity, dtype=torch.int32, device=device)


def table_of(keys: torch.Tensor, vals: Optional[torch.Tensor]):
    """The table object over ``(keys, vals)`` as ``new_table`` returns them."""
    return GPUHashTable32(keys) if vals is None else GPUHashTable(keys, vals)


# --------------------------------------------------------------------------- kernel maps
def downsample_cuda(coords: torch.Tensor, coords_max, coords_min, kernel_sizes, stride, padding) -> torch.Tensor:
    """Output coordinates of a strided convolution, int32 [M,4] in ascending ravel order
    (torchsparse/backend/others/downsample_cuda.cu:147-189): every input voxel proposes the outputs
    its kernel footprint reaches, the proposals are made unique."""
    _need_cuda(coords)
    cmin, cmax = _host_ints(coords_min, 4), _host_ints(coords_max, 4)
    uniq, m, _ = downsample_unique(coords, cmin, cmax, kernel_sizes, stride, padding)
    keys = uniq[:m]
    out = torch.empty((m, 4), dtype=torch.int32, device=coords.device)
    rem = keys
    for dim in (3, 2, 1):                      # unravel: z fastest, then y, x, batch
        size = cmax[dim] - cmin[dim] + 1
        out[:, dim] = (rem % size + cmin[dim]).int()
        rem = rem // size
    out[:, 0] = (rem + cmin[0]).int()
    return out


def build_kernel_map_subm_hashmap(table: GPUHashTable, coords: torch.Tensor, coords_min, coords_max, kernel_sizes,
                                  stride=None, padding=None, to_insert: bool = True,
                                  check_status: bool = True) -> List[torch.Tensor]:
    """Returns ``[out_in_map]`` int32 [pad128(N), Kvol]
    (torchsparse/backend/others/sparsemapping_cuda.cu:303-345)."""
    _need_cuda(coords)
    coords = coords.contiguous()
    n = coords.shape[0]
    ks = _host_ints(kernel_sizes, 3)
    cmin, cmax = _host_ints(coords_min, 4), _host_ints(coords_max, 4)
    kvol = ks[0] * ks[1] * ks[2]
    out = torch.empty((pad128(n), kvol), dtype=torch.int32, device=coords.device)
    status = torch.zeros(1, dtype=torch.int32, device=coords.device) if (to_insert and check_status) else None
    check(lib.tsb_kmap_subm(_p(table.keys), _p(table.vals), table.capacity, _p(coords), n, i32x(cmin), i32x(cmax),
                            i32x(ks), int(bool(to_insert)), _p(out), _p(status), _stream()),
          "build_kernel_map_subm_hashmap")
    if status is not None:
        _check_dev_status(status, "build_kernel_map_subm_hashmap")
    return [out]


def downsample_unique(coords: torch.Tensor, coords_min, coords_max, kernel_sizes, stride, padding):
    """First half of the strided map: sorted unique output keys plus the host-read
    ``(M, output coords max)``.  One device->host read (the reference needs two)."""
    coords = coords.contiguous()
    n = coords.shape[0]
    ks, st, pd = _host_ints(kernel_sizes, 3), _host_ints(stride, 3), _host_ints(padding, 3)
    cmin, cmax = _host_ints(coords_min, 4), _host_ints(coords_max, 4)
    a_ks, a_st = i32x(ks), i32x(st)
    slots = lib.tsb_kmap_down_slots(a_ks, a_st)
    if slots <= 0:
        raise ValueError("build_kernel_map_downsample_hashmap: bad kernel size / stride")
    uniq = torch.empty(max(n * slots, 1), dtype=torch.int64, device=coords.device)
    result = torch.empty(8, dtype=torch.int32, device=coords.device)
    ws = _workspace(lib.tsb_kmap_down_workspace_bytes(n, a_ks, a_st), coords.device)
    check(lib.tsb_kmap_down_unique(_p(coords), n, i32x(cmin), i32x(cmax), a_ks, a_st, i32x(pd), _p(uniq), _p(result),
                                   _p(ws), ws.numel(), _stream()), "build_kernel_map_downsample_hashmap")
    res = result.cpu().tolist()  # the one synchronisation of the strided build
    raise_if_kernel_failed(coords.device)     # the stream is idle now: the status of earlier launches comes cheap
    m = res[0]
    out_max = tuple(res[1:5]) if m > 0 else None
    return uniq, m, out_max


def downsample_finish(table: GPUHashTable, coords: torch.Tensor, uniq: torch.Tensor, m: int, coords_min, coords_max,
                      kernel_sizes, stride, padding, check_status: bool = True):
    coords = coords.contiguous()
    n = coords.shape[0]
    ks, st, pd = _host_ints(kernel_sizes, 3), _host_ints(stride, 3), _host_ints(padding, 3)
    cmin, cmax = _host_ints(coords_min, 4), _host_ints(coords_max, 4)
    kvol = ks[0] * ks[1] * ks[2]
    if table.capacity < m:
        raise ValueError(
            "The capacity of hashtable is not sufficient. Please enlarge reserved space for hashtable "
            "(torchsparse_b200.backends.hash_rsv_ratio)")
    out_coords = torch.empty((m, 4), dtype=torch.int32, device=coords.device)
    out_in_map = torch.empty((pad128(m), kvol), dtype=torch.int32, device=coords.device)
    status = torch.zeros(1, dtype=torch.int32, device=coords.device) if check_status else None
    check(lib.tsb_kmap_down_finish(_p(table.keys), _p(table.vals), table.capacity, _p(coords), n, _p(uniq), m,
                                   i32x(cmin), i32x(cmax), i32x(ks), i32x(st), i32x(pd), _p(out_coords),
                                   _p(out_in_map), _p(status), _stream()), "build_kernel_map_downsample_hashmap")
    if status is not None:
        _check_dev_status(status, "build_kernel_map_downsample_hashmap")
    return out_in_map, out_coords


def build_kernel_map_downsample_hashmap(table: GPUHashTable, coords: torch.Tensor, coords_min, coords_max, kernel_sizes,
                                        stride, padding, to_insert: bool = True) -> List[torch.Tensor]:
    """Returns ``[out_in_map, out_coords]``
    (torchsparse/backend/others/sparsemapping_cuda.cu:429-507).  ``coords_max`` is the
    bound in output space.  The table receives the output coordinates."""
    _need_cuda(coords)
    uniq, m, _ = downsample_unique(coords, coords_min, coords_max, kernel_sizes, stride, padding)
    out_in_map, out_coords = downsample_finish(table, coords, uniq, m, coords_min, coords_max, kernel_sizes, stride,
                                               padding)
    return [out_in_map, out_coords]


def build_kernel_map_subm_hashmap_int32(table: GPUHashTable32, coords: torch.Tensor, coords_min, coords_max,
                                        kernel_sizes, stride=None, padding=None,
                                        to_insert: bool = True) -> List[torch.Tensor]:
    """``build_kernel_map_subm_hashmap`` over a table of 32-bit keys
    (torchsparse/backend/others/sparsemapping_cuda.cu:259-300): same map, half the bytes per probe."""
    if table.vals is not None:
        raise ValueError("build_kernel_map_subm_hashmap_int32 expects a GPUHashTable32")
    return build_kernel_map_subm_hashmap(table, coords, coords_min, coords_max, kernel_sizes, stride, padding,
                                         to_insert)


def build_kernel_map_downsample_hashmap_int32(table: GPUHashTable32, coords: torch.Tensor, coords_min, coords_max,
                                              kernel_sizes, stride, padding,
                                              to_insert: bool = True) -> List[torch.Tensor]:
    """``build_kernel_map_downsample_hashmap`` over a table of 32-bit keys
    (torchsparse/backend/others/sparsemapping_cuda.cu:347-426)."""
    if table.vals is not None:
        raise ValueError("build_kernel_map_downsample_hashmap_int32 expects a GPUHashTable32")
    return build_kernel_map_downsample_hashmap(table, coords, coords_min, coords_max, kernel_sizes, stride, padding,
                                               to_insert)


def convert_transposed_out_in_map(out_in_map: torch.Tensor, out_in_map_t: torch.Tensor, fill: bool = False) -> None:
    """Writes into ``out_in_map_t`` (pre-filled with -1 by the caller unless ``fill``)
    (torchsparse/backend/others/query_cuda.cu:50-54)."""
    _need_cuda(out_in_map, out_in_map_t)
    check(lib.tsb_map_transpose(_p(out_in_map), out_in_map.shape[0], out_in_map.shape[1], _p(out_in_map_t),
                                out_in_map_t.shape[0], int(fill), _stream()), "convert_transposed_out_in_map")


def derive_bitmask_from_out_in_map(out_in_map: torch.Tensor, split_mask_num: int, valid_n: int) -> torch.Tensor:
    """int32 [split, rows] (torchsparse/backend/others/query_cuda.cu:59-65)."""
    _need_cuda(out_in_map)
    rows, kvol = out_in_map.shape
    out = torch.empty((split_mask_num, rows), dtype=torch.int32, device=out_in_map.device)
    check(lib.tsb_bitmask_derive(_p(out_in_map), rows, kvol, split_mask_num, valid_n, _p(out), _stream()),
          "derive_bitmask_from_out_in_map")
    return out


def sort_bitmask_cuda(bitmask: torch.Tensor, kvol: int = 27) -> Tuple[torch.Tensor, torch.Tensor]:
    """Stable descending sort per split -> (sorted_mask, reorder_loc int32).  Stands in for the
    ``torch.sort(bitmask, descending=True)`` of
    torchsparse/nn/functional/conv/kmap/func/hashmap_on_the_fly.py:96."""
    _need_cuda(bitmask)
    split, rows = bitmask.shape
    sorted_mask = torch.empty_like(bitmask)
    loc = torch.empty_like(bitmask)
    ws = _workspace(lib.tsb_bitmask_sort_workspace_bytes(rows, split), bitmask.device)
    check(lib.tsb_bitmask_sort(_p(bitmask), rows, split, kvol, _p(sorted_mask), _p(loc), _p(ws), ws.numel(),
                               _stream()), "sort_bitmask_cuda")
    return sorted_mask, loc


def sorted_artefacts_cuda(out_in_map: torch.Tensor, valid_n: int, m_tile: int):
    """One-call form of derive_bitmask -> sort -> reorder -> reduce for a single split.
    Returns (sorted_mask [1, rows], reorder_loc [1, rows], reordered_map [rows, Kvol],
    reduced_mask [1, ceil(rows / m_tile)]), the same tensors the four separate calls return."""
    _need_cuda(out_in_map)
    rows, kvol = out_in_map.shape
    dev = out_in_map.device
    masks = torch.empty((2, 1, rows), dtype=torch.int32, device=dev)
    reordered = torch.empty_like(out_in_map)
    reduced = torch.empty((1, (rows - 1) // m_tile + 1 if rows else 0), dtype=torch.int32, device=dev)
    ws = _workspace(lib.tsb_map_sorted_workspace_bytes(rows), dev)
    check(lib.tsb_map_sorted_artefacts(_p(out_in_map), rows, kvol, int(valid_n), int(m_tile), _p(masks[0]),
                                       _p(masks[1]), _p(reordered), _p(reduced), _p(ws), ws.numel(), _stream()),
          "sorted_artefacts_cuda")
    return masks[0], masks[1], reordered, reduced


class SortedMap:
    """A kernel map in the form the tensor-core convolution is fastest on (tsb_map_sorted_cm): rows sorted by
    neighbour mask, stored column-major, with per-tile offset masks and the work-item table that splits tiles
    with many offsets into parts.  Built once per kernel map and shared by every layer that uses the map
    (their launches must not overlap on the GPU: they share the scratch of the split tiles)."""

    __slots__ = ("map_cm", "loc", "tile_mask", "items", "n_items", "n_items_max", "rows", "kvol", "flags", "_scratch")

    def scratch(self, cout: int) -> torch.Tensor:
        buf = self._scratch.get(cout)
        if buf is None:
            buf = self._scratch[cout] = torch.empty((self.rows, cout), dtype=torch.float32, device=self.map_cm.device)
        return buf


# a tile of the sorted map with more offsets than this is split into parts that other CTAs can take
# (32: no tile is split)
split_max_offsets = 32


def sorted_cm_artefacts_cuda(out_in_map: torch.Tensor, valid_n: int, valid_n_dev: Optional[torch.Tensor] = None,
                             max_offsets: Optional[int] = None) -> SortedMap:
    """Row-sorted, column-major copy of a row-major kernel map plus its work-item table (tsb_map_sorted_cm).
    ``valid_n_dev`` (int32, device) overrides ``valid_n`` with a count the host does not know."""
    _need_cuda(out_in_map)
    rows, kvol = out_in_map.shape
    dev = out_in_map.device
    max_offsets = int(max_offsets or split_max_offsets)
    m = SortedMap()
    m.rows, m.kvol = rows, kvol
    m.map_cm = torch.empty((kvol, rows), dtype=torch.int32, device=dev)
    m.loc = torch.empty(rows, dtype=torch.int32, device=dev)
    m.tile_mask = torch.empty(max(rows // 128, 1), dtype=torch.int32, device=dev)
    m.n_items_max = int(lib.tsb_map_items_max(rows, kvol, max_offsets))
    m.items = torch.empty((max(m.n_items_max, 1), 4), dtype=torch.int32, device=dev)
    m.n_items = torch.empty(1, dtype=torch.int32, device=dev)
    m.flags = torch.zeros(max(rows // 128, 1) * 16, dtype=torch.int32, device=dev)
    m._scratch = {}
    ws = _workspace(lib.tsb_map_sorted_cm_workspace_bytes(rows), dev)
    check(lib.tsb_map_sorted_cm(_p(out_in_map), rows, kvol, int(valid_n), _p(valid_n_dev), _p(m.loc), _p(m.map_cm),
                                _p(m.tile_mask), max_offsets, rows // 128, _p(m.items), _p(m.n_items), _p(ws),
                                ws.numel(), _stream()),
          "sorted_cm_artefacts_cuda")
    return m


def reduce_bitmask_cuda(bitmask: torch.Tensor, m_tile: int) -> torch.Tensor:
    """int32 [split, ceil(rows/tile)] (torchsparse/backend/others/reduce_bitmask_cuda.cu:60-87)."""
    _need_cuda(bitmask)
    if m_tile % 4 != 0:
        raise RuntimeError("[Bitmask reduce] reduce tile size must be multiple of 4.")
    split, rows = bitmask.shape
    n_red = (rows - 1) // m_tile + 1
    out = torch.empty((split, n_red), dtype=torch.int32, device=bitmask.device)
    check(lib.tsb_bitmask_reduce(_p(bitmask), rows, split, m_tile, _p(out), _stream()), "reduce_bitmask_cuda")
    return out


def reorder_out_in_map_cuda(out_in_map: torch.Tensor, reorder_loc: torch.Tensor) -> torch.Tensor:
    """(torchsparse/backend/others/reorder_map_cuda.cu:25-47)."""
    _need_cuda(out_in_map, reorder_loc)
    rows, kvol = out_in_map.shape
    out = torch.empty_like(out_in_map)
    check(lib.tsb_map_reorder(_p(out_in_map), rows, kvol, _p(reorder_loc.contiguous()), reorder_loc.shape[0], _p(out),
                              _stream()), "reorder_out_in_map_cuda")
    return out


def exclusive_scan_quantified_wrapper(k_vol: int, nbsizes: torch.Tensor, nbaddrs: torch.Tensor,
                                      qnbaddrs: torch.Tensor) -> torch.Tensor:
    """Writes the two scans into its arguments and returns a dummy tensor
    (torchsparse/backend/others/exclusive_scan_cuda.cu:31-44)."""
    _need_cuda(nbsizes, nbaddrs, qnbaddrs)
    check(lib.tsb_scan_quantified(k_vol, _p(nbsizes), _p(nbaddrs), _p(qnbaddrs), _stream()),
          "exclusive_scan_quantified_wrapper")
    return torch.zeros(1)


def pairs_from_out_in_map(out_in_map: torch.Tensor, transposed_layout: bool):
    """Pair lists of the GatherScatter / FetchOnDemand dataflows from an out_in_map, in one
    counting pass and one fill pass (replaces the torch ``nonzero``/``sum``/gather chain of
    torchsparse/nn/functional/conv/kmap/func/hashmap_on_the_fly.py:138-141).

    Returns (nbmaps int32 [P,2] or [2,P], nbsizes int32 [Kvol] device, nbsizes host list,
    nbaddrs int32 [Kvol+1], qnbaddrs int32 [Kvol+1], qmapsize int)."""
    _need_cuda(out_in_map)
    rows, kvol = out_in_map.shape
    dev = out_in_map.device
    scans = torch.empty(3 * (kvol + 1), dtype=torch.int32, device=dev)
    nbsizes, nbaddrs, qnbaddrs = scans[:kvol], scans[kvol + 1:2 * kvol + 2], scans[2 * kvol + 2:]
    check(lib.tsb_pairs_count(_p(out_in_map), rows, kvol, _p(nbsizes), _p(nbaddrs), _p(qnbaddrs), _stream()),
          "pairs_from_out_in_map")
    host = scans.cpu().tolist()  # one synchronisation; the reference reads nbsizes on the host too
    sizes_host = host[:kvol]
    n_pairs = host[2 * kvol + 1]
    qmapsize = host[-1]
    shape = (2, n_pairs) if transposed_layout else (n_pairs, 2)
    nbmaps = torch.empty(shape, dtype=torch.int32, device=dev)
    ws = _workspace(lib.tsb_pairs_fill_workspace_bytes(rows, kvol), dev)
    check(lib.tsb_pairs_fill(_p(out_in_map), rows, kvol, _p(nbaddrs), n_pairs, int(transposed_layout), _p(nbmaps),
                             _p(ws), ws.numel(), _stream()), "pairs_from_out_in_map")
    return nbmaps, nbsizes, sizes_host, nbaddrs, qnbaddrs, qmapsize


def build_mask_from_kmap(n_points: int, n_out_points: int, nbmaps: torch.Tensor,
                         nbsizes: torch.Tensor) -> List[torch.Tensor]:
    """Returns ``[input_mask, output_mask]``
    (torchsparse/backend/others/sparsemapping_cuda.cu:510-548)."""
    _need_cuda(nbmaps, nbsizes)
    nbmaps = nbmaps.int().contiguous()
    kvol = nbsizes.numel()
    dev = nbmaps.device
    nbaddrs = torch.zeros(kvol + 1, dtype=torch.int32, device=dev)
    nbaddrs[1:] = torch.cumsum(nbsizes.int(), 0)
    n_pairs = nbmaps.shape[0]
    input_mask = torch.empty(kvol * n_points, dtype=torch.int32, device=dev)
    output_mask = torch.empty(kvol * n_out_points, dtype=torch.int32, device=dev)
    check(lib.tsb_build_masks(n_points, n_out_points, _p(nbmaps), _p(nbaddrs), kvol, n_pairs, _p(input_mask),
                              _p(output_mask), _stream()), "build_mask_from_kmap")
    return [input_mask, output_mask]


# --------------------------------------------------------------------------- convolution
# Weights packed K-major for the tensor-core kernel are cached ON the weight tensor object, tagged
# with its version counter, so an inference loop packs each layer once and an in-place update
# through torch invalidates the copy.  Writes through ``.data`` or raw pointers do NOT move the version
# counter: after such a write call ``FusedConv.invalidate()`` / delete the ``_tsb_packed`` and ``_tsb_padded``
# attributes of the weight tensor, or turn the cache off.
cache_packed_weights = True
# When True every tensor-core launch is followed by a read of its device status word (a sync).
check_kernel_status = False


def _packed_weight(kernel: torch.Tensor, code: int, tf32: bool = False) -> Optional[torch.Tensor]:
    if code == _lib.TSB_F32 and not tf32:
        return None          # exact fp32 runs on the CUDA cores, which read the weights as they are
    tag = (kernel._version, kernel.data_ptr())
    hit = getattr(kernel, "_tsb_packed", None)
    if hit is not None and hit[0] == tag:
        return hit[1]
    kvol, cin, cout = kernel.shape
    packed = torch.empty(lib.tsb_conv_packed_weight_bytes(kvol, cin, cout, code), dtype=torch.uint8,
                         device=kernel.device)
    check(lib.tsb_conv_pack_weight(_p(kernel), kvol, cin, cout, code, _p(packed), _stream()), "pack_weight")
    # the packed copy is published to every later launch, also on other streams: it is complete first
    # (once per weight tensor and version)
    torch.cuda.current_stream().synchronize()
    try:
        kernel._tsb_packed = (tag, packed)
    except (AttributeError, RuntimeError):
        pass
    return packed


def _padded_kernel(kernel: torch.Tensor) -> torch.Tensor:
    """[Kvol, Cin, Cout] with Cin zero-padded to a multiple of 8; cached on the weight tensor."""
    tag = (kernel._version, kernel.data_ptr())
    hit = getattr(kernel, "_tsb_padded", None)
    if hit is not None and hit[0] == tag:
        return hit[1]
    cin = kernel.shape[1]
    padded = torch.nn.functional.pad(kernel, (0, 0, 0, (-cin) % 8)).contiguous()
    torch.cuda.current_stream().synchronize()     # published to launches on other streams: complete first
    try:
        kernel._tsb_padded = (tag, padded)
    except (AttributeError, RuntimeError):
        pass
    return padded


def _tensor_core_shape(in_feats: torch.Tensor, kernel: torch.Tensor, allow_tf32: bool) -> bool:
    """Shapes the tcgen05 kernel takes (include/tsb200.h, tsb_conv_igemm_fwd)."""
    kvol, cin, cout = kernel.shape
    if in_feats.dtype == torch.float32 and not allow_tf32:
        return False
    return (cin * in_feats.element_size()) % 16 == 0 and cout % 8 == 0 and kvol <= 32


def _math_mode(t: torch.Tensor, allow_tf32: bool) -> int:
    return _lib.TSB_MATH_TF32 if (t.dtype == torch.float32 and allow_tf32) else _lib.TSB_MATH_FP32


def _prep_feats(in_feats: torch.Tensor, kernel: torch.Tensor, allow_fp16: bool):
    _need_cuda(in_feats, kernel)
    if in_feats.dtype != kernel.dtype:
        raise RuntimeError("input features and kernel must share a dtype")
    if in_feats.dtype == torch.float16 and not allow_fp16:
        raise RuntimeError("fp16 convolution requested but allow_fp16 is off")
    if kernel.dim() != 3:
        raise ValueError("kernel must be [Kvol, Cin, Cout]")
    if in_feats.shape[1] != kernel.shape[1]:
        raise ValueError("Input feature size and kernel size mismatch")
    return in_feats.contiguous(), kernel.contiguous()


# Launch-configuration overrides of the tensor-core kernel for tuning runs (0 = chosen by the library):
# N tile, 128-byte channel chunks per pipeline stage, stages, CTAs per SM.
igemm_tuning = {"n_tile": 0, "cpb": 0, "stages": 0, "ctas": 0, "gather": 0, "grid": 0}


def tile_mask_cuda(out_in_map: torch.Tensor, n_rows: int, row_stride: Optional[int] = None,
                   col_stride: Optional[int] = None, n_rows_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """uint32-as-int32 [ceil(n_rows / 128)]: the kernel offsets present in each 128-row tile of a map whose
    entry (row, k) lies at ``row * row_stride + k * col_stride`` (default: row-major [rows, Kvol])."""
    _need_cuda(out_in_map)
    kvol = out_in_map.shape[1] if row_stride is None else None
    if row_stride is None:
        row_stride, col_stride = out_in_map.shape[1], 1
    else:
        kvol = out_in_map.shape[0] if col_stride != 1 else out_in_map.shape[1]
    out = torch.empty(max(1, (n_rows + 127) // 128), dtype=torch.int32, device=out_in_map.device)
    check(lib.tsb_map_tile_mask(_p(out_in_map), n_rows, kvol, row_stride, col_stride, _p(n_rows_dev), _p(out), _stream()),
          "tile_mask_cuda")
    return out


def _tile_mask_of(out_in_map: torch.Tensor, n_rows: int) -> Optional[torch.Tensor]:
    """Tile masks of a row-major map, derived once and kept on the map tensor (a kernel map is shared
    by the layers of a resolution level; the masks are rebuilt if the tensor is modified in place)."""
    if out_in_map.shape[1] > 32 or not out_in_map.is_contiguous():
        return None
    tag = (out_in_map._version, out_in_map.data_ptr(), n_rows)
    hit = getattr(out_in_map, "_tsb_tile_mask", None)
    if hit is not None and hit[0] == tag:
        return hit[1]
    mask = tile_mask_cuda(out_in_map, n_rows)
    try:
        out_in_map._tsb_tile_mask = (tag, mask)
    except (AttributeError, RuntimeError):
        pass
    return mask


def _apply_tuning(d) -> None:
    d.cfg_n_tile, d.cfg_cpb = igemm_tuning["n_tile"], igemm_tuning["cpb"]
    d.cfg_stages, d.cfg_ctas = igemm_tuning["stages"], igemm_tuning["ctas"]
    d.cfg_gather, d.cfg_grid = igemm_tuning["gather"], igemm_tuning["grid"]


def conv_forward_implicit_gemm_cuda(in_feats: torch.Tensor, kernel: torch.Tensor, out_in_map: Optional[torch.Tensor],
                                    num_out_feats: int, num_out_channels: int, allow_tf32: bool = False,
                                    allow_fp16: bool = True, *, scale: Optional[torch.Tensor] = None,
                                    bias: Optional[torch.Tensor] = None,
                                    residual: Optional[torch.Tensor] = None, relu: bool = False,
                                    reorder_loc: Optional[torch.Tensor] = None,
                                    tile_mask: Optional[torch.Tensor] = None,
                                    in_feats2: Optional[torch.Tensor] = None,
                                    map_strides: Optional[Tuple[int, int]] = None,
                                    k_range: Optional[Tuple[int, int]] = None,
                                    acc_in: Optional[torch.Tensor] = None, acc_out: Optional[torch.Tensor] = None,
                                    n_out_dev: Optional[torch.Tensor] = None,
                                    out: Optional[torch.Tensor] = None, dst_rows: int = 0,
                                    smap: Optional["SortedMap"] = None) -> Optional[torch.Tensor]:
    """Implicit-GEMM forward
    (torchsparse/backend/convolution/convolution_forward_implicit_gemm_cuda.cu:1527-1987).
    ``scale`` / ``bias`` (fp32 [Cout]), ``residual`` and ``relu`` are an optional fused epilogue
    (y = relu(acc * scale + bias + residual), one rounding) that the reference does not have.
    The remaining keywords are the options of ``tsb_conv_igemm_run`` (include/tsb200.h): a second feature
    matrix whose channels follow those of ``in_feats``, a map with other strides (or ``None`` with a
    1x1x1 kernel: row m reads input row m), a range of kernel offsets, fp32 partial sums in / out, a
    device-side row count and a caller-owned output.  ``smap`` (a :class:`SortedMap`) stands for the map, its
    strides, row order and work-item table in one argument."""
    from . import backends
    if (in_feats.dtype == torch.float32 and kernel.dtype == torch.float32 and not allow_tf32
            and backends.fp32_by_split_tf32 and in_feats2 is None and acc_in is None and acc_out is None
            and k_range is None and kernel.dim() == 3 and kernel.shape[1] % 4 == 0 and kernel.shape[2] % 8 == 0
            and kernel.shape[0] <= 32 and in_feats.shape[0] > 0 and num_out_feats > 0
            and in_feats.shape[1] == kernel.shape[1]
            and num_out_feats * kernel.shape[1] * kernel.shape[2] >= _SPLIT_TF32_MIN_WORK):
        return _conv_fp32_by_split_tf32(in_feats, kernel, out_in_map, num_out_feats, num_out_channels,
                                        dict(scale=scale, bias=bias, residual=residual, relu=relu, out=out),
                                        dict(reorder_loc=reorder_loc, tile_mask=tile_mask, map_strides=map_strides,
                                             n_out_dev=n_out_dev, dst_rows=dst_rows, smap=smap))
    if smap is not None:
        out_in_map, reorder_loc, tile_mask, map_strides = smap.map_cm, smap.loc, smap.tile_mask, (1, smap.rows)
    in_feats, kernel = _prep_feats_cat(in_feats, in_feats2, kernel, allow_fp16)
    if in_feats2 is not None:
        in_feats2 = in_feats2.contiguous()
    kvol, cin, cout = kernel.shape
    if num_out_channels != cout:
        raise ValueError("num_out_channels does not match the kernel")
    if in_feats.dtype != torch.float32 and cin % 8 != 0 and cout % 8 == 0 and kvol <= 32 and in_feats2 is None:
        # rows that are not 16-byte multiples (the 4- or 5-channel input layer): zero-pad the channels
        # once so that the layer takes the tensor-core kernel instead of the CUDA-core one
        kernel = _padded_kernel(kernel)
        in_feats = torch.nn.functional.pad(in_feats, (0, kernel.shape[1] - cin))
        cin = kernel.shape[1]
    if out_in_map is None:
        if kvol != 1:
            raise ValueError("a convolution without a kernel map needs a 1x1x1 kernel")
    else:
        _need_cuda(out_in_map)
        if map_strides is None and (out_in_map.shape[1] != kvol or out_in_map.shape[0] < num_out_feats):
            raise ValueError("out_in_map shape does not match kernel volume / output rows")
    code = _dtype_code(in_feats)
    if out is None and acc_out is None:
        out = torch.empty((num_out_feats if not dst_rows else dst_rows, cout), dtype=in_feats.dtype,
                          device=in_feats.device)
    if bias is not None:
        bias = bias.float().contiguous()
    if scale is not None:
        scale = scale.float().contiguous()
    if residual is not None:
        residual = residual.to(in_feats.dtype).contiguous()
    tensor_cores = code != _lib.TSB_F32 or bool(allow_tf32)
    packed = _packed_weight(kernel, code, bool(allow_tf32)) if (cache_packed_weights and tensor_cores) else None
    if check_kernel_status:
        status = torch.zeros(1, dtype=torch.int32, device=in_feats.device)
    else:
        status = _status_word(in_feats.device)
    if tile_mask is None and tensor_cores and out_in_map is not None and map_strides is None and kvol > 1:
        tile_mask = _tile_mask_of(out_in_map, num_out_feats)
    # what is not supplied is made in the workspace: packed weights, tile masks
    ws = None
    if packed is None or (tile_mask is None and out_in_map is not None):
        ws = _workspace(lib.tsb_conv_igemm_workspace_bytes(kvol, cin, cout, code)
                        + lib.tsb_map_tile_mask_bytes(num_out_feats), in_feats.device)
    if _observer is not None:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
    d = _lib.new_igemm_desc()
    d.dtype, d.math, d.relu = code, _math_mode(in_feats, allow_tf32), int(relu)
    d.in_feats, d.in_feats2, d.weight, d.packed_weight = _p(in_feats), _p(in_feats2), _p(kernel), _p(packed)
    d.out_in_map, d.reorder_loc, d.tile_mask, d.out_feats = _p(out_in_map), _p(reorder_loc), _p(tile_mask), _p(out)
    d.scale, d.bias, d.residual = _p(scale), _p(bias), _p(residual)
    d.acc_in, d.acc_out, d.n_out_dev, d.dev_status = _p(acc_in), _p(acc_out), _p(n_out_dev), _p(status)
    d.workspace, d.workspace_bytes = _p(ws), 0 if ws is None else ws.numel()
    d.n_in, d.n_out, d.dst_rows = in_feats.shape[0], num_out_feats, int(dst_rows)
    if map_strides is not None:
        d.map_row_stride, d.map_col_stride = map_strides
    d.kvol, d.cin, d.cout = kvol, cin, cout
    d.c1 = in_feats.shape[1] if in_feats2 is not None else 0
    if k_range is not None:
        d.k_lo, d.k_hi = k_range
    if smap is not None and k_range is None:
        d.items, d.n_items_dev, d.n_items = _p(smap.items), _p(smap.n_items), smap.n_items_max
        d.split_scratch, d.split_flags = _p(smap.scratch(cout)), _p(smap.flags)
    _apply_tuning(d)
    rc = lib.tsb_conv_igemm_run(_lib.C.byref(d), _stream())
    if rc == 2:
        # shapes the tensor-core kernel does not take (exact fp32, odd row sizes): the CUDA-core kernel
        # behind the flat entry point, which has none of the options above
        if (in_feats2 is not None or map_strides is not None or k_range is not None or acc_in is not None
                or acc_out is not None or n_out_dev is not None or out_in_map is None):
            check(rc, "conv_forward_implicit_gemm_cuda (these options need a tensor-core shape)")
        rc = lib.tsb_conv_igemm_fwd(_p(in_feats), _p(kernel), _p(packed), _p(out_in_map), _p(reorder_loc),
                                    _p(tile_mask), _p(out), in_feats.shape[0], num_out_feats, kvol, cin, cout, code,
                                    _math_mode(in_feats, allow_tf32), _p(scale), _p(bias), _p(residual), int(relu),
                                    _p(status), _p(ws), 0 if ws is None else ws.numel(), _stream())
    check(rc, "conv_forward_implicit_gemm_cuda")
    if _observer is not None:
        ev1.record()
        _observer("igemm", (in_feats.shape[0], num_out_feats, kvol, cin, cout, code, out_in_map,
                            tile_mask, k_range), ev0, ev1)
    if check_kernel_status and int(status.item()) != 0:
        raise RuntimeError(f"conv_forward_implicit_gemm_cuda: a bounded wait inside the kernel ran out "
                           f"(code {int(status.item())}); the output is undefined")
    return out


# rows x Cin x Cout below which the ten launches of the split path cost more than the CUDA-core kernel
# (measured: 10 k rows x 16 x 16 take 0.15 ms split against 0.03 ms, 100 k rows x 64 x 64 0.40 ms against 0.75 ms)
_SPLIT_TF32_MIN_WORK = 200_000_000


def _split_tf32(t: torch.Tensor):
    """t = hi + lo with hi exactly representable in TF32 (the low 13 mantissa bits cleared)."""
    hi = (t.contiguous().view(torch.int32) & -8192).view(torch.float32)
    return hi, t - hi


def _conv_fp32_by_split_tf32(in_feats, kernel, out_in_map, num_out_feats, cout, epilogue, common):
    """fp32 convolution of fp32 operands on the tensor cores: three TF32 launches over the split operands, the
    partial sums kept in fp32 between them (smallest terms first), the epilogue in the last launch.  Every product
    of two TF32 numbers is exact in fp32, so what is dropped is x_lo * w_lo (relative 2^-22) and the rounding of
    x_lo, w_lo to TF32 (relative 2^-21): the result stays within the 1e-5 relative error asked of fp32 paths."""
    x_hi, x_lo = _split_tf32(in_feats)
    w_hi, w_lo = _split_tf32(kernel)
    rows = int(common.get("dst_rows") or 0) or num_out_feats
    acc1 = torch.empty((rows, cout), dtype=torch.float32, device=in_feats.device)
    acc2 = torch.empty_like(acc1)
    conv_forward_implicit_gemm_cuda(x_lo, w_hi, out_in_map, num_out_feats, cout, True, acc_out=acc1, **common)
    conv_forward_implicit_gemm_cuda(x_hi, w_lo, out_in_map, num_out_feats, cout, True, acc_in=acc1, acc_out=acc2, **common)
    return conv_forward_implicit_gemm_cuda(x_hi, w_hi, out_in_map, num_out_feats, cout, True, acc_in=acc2, **epilogue,
                                           **common)


def _prep_feats_cat(in_feats, in_feats2, kernel, allow_fp16):
    """_prep_feats for an input that may be the channel concatenation of two matrices."""
    if in_feats2 is None:
        return _prep_feats(in_feats, kernel, allow_fp16)
    _need_cuda(in_feats, in_feats2, kernel)
    if in_feats.dtype != kernel.dtype or in_feats2.dtype != kernel.dtype:
        raise RuntimeError("input features and kernel must share a dtype")
    if in_feats.shape[0] != in_feats2.shape[0]:
        raise ValueError("the two feature matrices must have the same rows")
    if kernel.dim() != 3 or in_feats.shape[1] + in_feats2.shape[1] != kernel.shape[1]:
        raise ValueError("Input feature size and kernel size mismatch")
    return in_feats.contiguous(), kernel.contiguous()


class IgemmLayerPlan:
    """The arguments of tsb_conv_igemm_run that do not change between calls of one inference layer
    (weights, packed weights, fp32 scale / shift, sizes), resolved once into a descriptor.
    :func:`igemm_plan_launch` then costs one output allocation and one foreign call; argument checks
    happened when the plan was made.  The plan keeps the tensors alive and is remade when the weights
    are replaced or modified."""

    __slots__ = ("kernel", "packed", "scale", "bias", "tag", "desc", "cin", "cout", "dtype", "device", "allow_tf32")

    def __init__(self, kernel: torch.Tensor, scale: Optional[torch.Tensor], bias: Optional[torch.Tensor],
                 allow_tf32: bool, relu: bool = False):
        _need_cuda(kernel)
        if kernel.dim() != 3:
            raise ValueError("kernel must be [Kvol, Cin, Cout]")
        kernel = kernel.contiguous()
        kvol, cin, cout = kernel.shape
        code = _dtype_code(kernel)
        if (cin * kernel.element_size()) % 16 != 0 or cout % 8 != 0 or kvol > 32:
            raise ValueError("IgemmLayerPlan needs feature rows that are 16-byte multiples and Cout % 8 == 0")
        if code == _lib.TSB_F32 and not allow_tf32:
            raise ValueError("IgemmLayerPlan is for the tensor-core kernel (16-bit tensors or TF32)")
        self.tag = (kernel._version, kernel.data_ptr(), bool(allow_tf32))
        self.allow_tf32 = bool(allow_tf32)
        self.kernel = kernel
        self.packed = _packed_weight(kernel, code, bool(allow_tf32))
        self.scale = None if scale is None else scale.float().contiguous()
        self.bias = None if bias is None else bias.float().contiguous()
        self.cin, self.cout, self.dtype = cin, cout, kernel.dtype
        self.device = kernel.device if kernel.device.index is not None else torch.device("cuda", kernel.get_device())
        d = self.desc = _lib.new_igemm_desc()
        d.dtype = code
        d.math = _lib.TSB_MATH_TF32 if (kernel.dtype == torch.float32 and allow_tf32) else _lib.TSB_MATH_FP32
        d.relu = int(relu)
        d.weight, d.packed_weight = kernel.data_ptr(), _p(self.packed)
        d.scale, d.bias = _p(self.scale), _p(self.bias)
        d.dev_status = _status_word(self.device).data_ptr()
        d.kvol, d.cin, d.cout = kvol, cin, cout

    def valid_for(self, kernel: torch.Tensor, allow_tf32: bool) -> bool:
        return self.tag == (kernel._version, kernel.data_ptr(), bool(allow_tf32))


def igemm_plan_launch(plan: IgemmLayerPlan, in_feats: torch.Tensor, out_in_map: Optional[torch.Tensor],
                      num_out_feats: int, residual: Optional[torch.Tensor], relu: bool,
                      reorder_loc: Optional[torch.Tensor] = None, tile_mask: Optional[torch.Tensor] = None,
                      in_feats2: Optional[torch.Tensor] = None, map_strides: Optional[Tuple[int, int]] = None,
                      n_out_dev: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                      smap: Optional["SortedMap"] = None) -> torch.Tensor:
    """conv_forward_implicit_gemm_cuda for a layer with an :class:`IgemmLayerPlan` (same kernel launch).
    Falls back to the checked entry point when launches are being observed or their status read back."""
    if _observer is not None or check_kernel_status:
        return conv_forward_implicit_gemm_cuda(in_feats, plan.kernel, out_in_map, num_out_feats, plan.cout,
                                               plan.allow_tf32, True, scale=plan.scale, bias=plan.bias,
                                               residual=residual, relu=relu, reorder_loc=reorder_loc,
                                               tile_mask=tile_mask, in_feats2=in_feats2, map_strides=map_strides,
                                               n_out_dev=n_out_dev, out=out, smap=smap)
    if smap is not None:
        out_in_map, reorder_loc, tile_mask, map_strides = smap.map_cm, smap.loc, smap.tile_mask, (1, smap.rows)
    c1 = in_feats.shape[1]
    if in_feats.dtype != plan.dtype or not in_feats.is_contiguous():
        raise ValueError("input features do not match the layer plan (dtype or layout)")
    if in_feats2 is not None:
        if in_feats2.dtype != plan.dtype or not in_feats2.is_contiguous() or c1 + in_feats2.shape[1] != plan.cin:
            raise ValueError("input features do not match the layer plan (second matrix)")
    elif c1 != plan.cin:
        raise ValueError("input features do not match the layer plan (channel count)")
    if residual is not None and (residual.dtype != plan.dtype or not residual.is_contiguous()):
        residual = residual.to(plan.dtype).contiguous()
    if out is None:
        out = torch.empty((num_out_feats, plan.cout), dtype=plan.dtype, device=plan.device)
    ws = None
    if tile_mask is None and out_in_map is not None and plan.desc.kvol > 1:
        if map_strides is None:
            tile_mask = _tile_mask_of(out_in_map, num_out_feats)
        if tile_mask is None:
            ws = _workspace(lib.tsb_conv_igemm_workspace_bytes(plan.desc.kvol, plan.cin, plan.cout, plan.desc.dtype)
                            + lib.tsb_map_tile_mask_bytes(num_out_feats), plan.device)
    d = plan.desc
    d.relu = int(relu)
    d.in_feats, d.in_feats2 = in_feats.data_ptr(), (None if in_feats2 is None else in_feats2.data_ptr())
    d.c1 = c1 if in_feats2 is not None else 0
    d.out_in_map = None if out_in_map is None else out_in_map.data_ptr()
    d.reorder_loc = None if reorder_loc is None else reorder_loc.data_ptr()
    d.tile_mask = None if tile_mask is None else tile_mask.data_ptr()
    d.out_feats = out.data_ptr()
    d.residual = None if residual is None else residual.data_ptr()
    d.n_out_dev = None if n_out_dev is None else n_out_dev.data_ptr()
    d.workspace, d.workspace_bytes = (None, 0) if ws is None else (ws.data_ptr(), ws.numel())
    d.n_in, d.n_out = in_feats.shape[0], num_out_feats
    d.map_row_stride, d.map_col_stride = map_strides if map_strides is not None else (0, 0)
    if smap is not None:
        d.items, d.n_items_dev, d.n_items = smap.items.data_ptr(), smap.n_items.data_ptr(), smap.n_items_max
        d.split_scratch, d.split_flags = smap.scratch(plan.cout).data_ptr(), smap.flags.data_ptr()
    else:
        d.items, d.n_items_dev, d.n_items, d.split_scratch, d.split_flags = None, None, 0, None, None
    _apply_tuning(d)
    rc = lib.tsb_conv_igemm_run(_lib.C.byref(d), torch._C._cuda_getCurrentRawStream(plan.device.index))
    if rc != 0:
        check(rc, "conv_forward_implicit_gemm_cuda")
    return out


def conv_wgrad_implicit_gemm_cuda(gathered: torch.Tensor, rows: torch.Tensor, out_in_map: torch.Tensor,
                                  tile_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[k][a][b] = sum over map rows m of gathered[out_in_map[m][k]][a] * rows[m][b], fp32 [Kvol, Cg, Cd]
    (tsb_conv_wgrad_igemm: tcgen05 with both operands read MN-major, fp32 accumulators in TMEM, the row range
    divided among CTAs; fp32 tensors and channel counts that are not multiples of 8 / 16 run the CUDA-core kernel
    behind the same entry).  With the forward map, gathered = input features and rows = output gradients give dW."""
    _need_cuda(gathered, rows, out_in_map)
    n_rows, kvol = rows.shape[0], out_in_map.shape[1]
    cg, cd = gathered.shape[1], rows.shape[1]
    if out_in_map.shape[0] < n_rows:
        raise ValueError("the map has fewer rows than the row matrix")
    dev = rows.device
    if rows.dtype != gathered.dtype:
        rows = rows.to(gathered.dtype)
    if gathered.dtype not in _DTYPES:
        raise RuntimeError("unsupported dtype")
    if n_rows == 0 or gathered.shape[0] == 0:
        return torch.zeros((kvol, cg, cd), dtype=torch.float32, device=dev)
    gathered, rows, out_in_map = gathered.contiguous(), rows.contiguous(), out_in_map.contiguous()
    if tile_mask is None:
        tile_mask = _tile_mask_of(out_in_map, n_rows)
    out = torch.empty((kvol, cg, cd), dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev) if check_kernel_status else _status_word(dev)
    ws = _workspace(lib.tsb_conv_wgrad_igemm_workspace_bytes(n_rows), dev)
    rc = lib.tsb_conv_wgrad_igemm(_p(gathered), _p(rows), _p(out_in_map), _p(tile_mask), _p(out), gathered.shape[0],
                                  n_rows, 0, 0, kvol, cg, cd, _dtype_code(gathered), _p(status), _p(ws), ws.numel(),
                                  _stream())
    check(rc, "conv_wgrad_implicit_gemm_cuda")
    if check_kernel_status and int(status.item()) != 0:
        raise RuntimeError(f"conv_wgrad_implicit_gemm_cuda: a bounded wait inside the kernel ran out "
                           f"(code {int(status.item())}); the output is undefined")
    return out


def conv_backward_wgrad_implicit_gemm_cuda(_in_feats: torch.Tensor, _kernel: torch.Tensor, _out_in_map: torch.Tensor,
                                           split_k_iters: int = 32, allow_tf32: bool = False,
                                           allow_fp16: bool = True) -> torch.Tensor:
    """The reference's entry (torchsparse/backend/convolution/convolution_backward_wgrad_implicit_gemm_cuda.cu:1614,
    called at torchsparse/nn/functional/conv/func/implicit_gemm.py:178 with grad_output, input and the map of the
    input rows): returns [Kvol * Cout, Cin] = sum over input rows n of grad_output[map[n][k]]^T . input[n].
    ``split_k_iters`` is accepted and ignored (the library divides the row range itself)."""
    if torch.float16 in (_in_feats.dtype, _kernel.dtype) and allow_fp16:
        _in_feats, _kernel = _in_feats.half(), _kernel.half()
    out = conv_wgrad_implicit_gemm_cuda(_in_feats, _kernel, _out_in_map)
    return out.reshape(-1, _kernel.shape[1]).to(_kernel.dtype)


def conv_backward_wgrad_implicit_gemm_sorted_cuda(_in_feats: torch.Tensor, _kernel: torch.Tensor,
                                                  _out_in_map: torch.Tensor, _reduced_mask: torch.Tensor,
                                                  _reorder_loc: torch.Tensor, split_k_iters: int = 32,
                                                  allow_tf32: bool = False, allow_fp16: bool = True) -> torch.Tensor:
    """The sorted form (convolution_backward_wgrad_implicit_gemm_sorted_cuda.cu:1744): row r of the reordered map
    belongs to input row ``_reorder_loc[0][r]``.  The input rows are put in map order once and the unsorted entry
    does the rest; ``_reduced_mask`` is not needed (the per-tile offset masks are derived from the map)."""
    loc = (_reorder_loc[0] if _reorder_loc.dim() == 2 else _reorder_loc).long()
    n = _kernel.shape[0]
    rows = _kernel.index_select(0, loc[:n].clamp(min=0))
    return conv_backward_wgrad_implicit_gemm_cuda(_in_feats, rows, _out_in_map, split_k_iters, allow_tf32, allow_fp16)


def conv_backward_gather_scatter_cuda(in_feat: torch.Tensor, grad_in_feat: torch.Tensor, grad_out_feat: torch.Tensor,
                                      kernel: torch.Tensor, grad_kernel: torch.Tensor, neighbor_map: torch.Tensor,
                                      neighbor_offset, transpose: bool = False) -> None:
    """Gradients of the gather-scatter convolution, written into ``grad_in_feat`` and ``grad_kernel``
    (torchsparse/backend/convolution/convolution_gather_scatter_cuda.cu:640-800): the input gradient is the
    same pair-list convolution run from the outputs back to the inputs with every W[k] transposed, the weight
    gradient is X[in_k]^T . dY[out_k] per offset (the pair list turned into a map of the output rows)."""
    _need_cuda(in_feat, grad_in_feat, grad_out_feat, kernel, grad_kernel, neighbor_map)
    sizes = [int(v) for v in (neighbor_offset.tolist() if isinstance(neighbor_offset, torch.Tensor) else neighbor_offset)]
    nbmaps = neighbor_map.int().contiguous()
    n_a, n_b = (grad_out_feat.shape[0], in_feat.shape[0]) if transpose else (in_feat.shape[0], grad_out_feat.shape[0])
    masks = build_mask_from_kmap(n_a, n_b, nbmaps, torch.tensor(sizes, dtype=torch.int32, device=nbmaps.device))
    gx = conv_forward_gather_scatter_cuda(grad_out_feat.to(kernel.dtype), kernel.transpose(1, 2).contiguous(), nbmaps,
                                          sizes, masks[0], masks[1], in_feat.shape[0], transpose=not transpose,
                                          allow_tf32=False)
    grad_in_feat.copy_(gx)
    # weight gradient: the pair list as a map of the output rows (entry (row, k) = the input row paired with it at
    # offset k), then the kernel behind tsb_conv_wgrad_igemm
    x_col, y_col = (1, 0) if transpose else (0, 1)
    kvol = len(sizes)
    offset_of_pair = torch.repeat_interleave(torch.arange(kvol, device=nbmaps.device),
                                             torch.tensor(sizes, device=nbmaps.device))
    rows_pad = (grad_out_feat.shape[0] + 127) // 128 * 128
    as_map = torch.full((rows_pad, kvol), -1, dtype=torch.int32, device=nbmaps.device)
    as_map[nbmaps[:, y_col].long(), offset_of_pair] = nbmaps[:, x_col]
    grad_kernel.copy_(conv_wgrad_implicit_gemm_cuda(in_feat, grad_out_feat, as_map))


def conv_forward_implicit_gemm_sorted_cuda(in_feats: torch.Tensor, kernel: torch.Tensor, out_in_map: torch.Tensor,
                                           reduced_mask: torch.Tensor, reorder_loc: torch.Tensor, num_out_feats: int,
                                           num_out_channels: int, allow_tf32: bool = False,
                                           allow_fp16: bool = True, **epilogue) -> torch.Tensor:
    """Sorted implicit-GEMM forward
    (torchsparse/backend/convolution/convolution_forward_implicit_gemm_sorted_cuda.cu:1755-2230).
    ``out_in_map`` is the row-reordered map; output row r is stored at ``reorder_loc[s][r]``.
    With split_mask_num > 1 each split covers its own column range with its own row order; the
    splits are accumulated in fp32 here instead of being rounded and summed."""
    split = reorder_loc.shape[0] if reorder_loc.dim() == 2 else 1
    loc = reorder_loc.reshape(split, -1).contiguous()
    if split == 1:
        return conv_forward_implicit_gemm_cuda(in_feats, kernel, out_in_map, num_out_feats, num_out_channels,
                                               allow_tf32, allow_fp16, reorder_loc=loc[0], **epilogue)
    kvol = kernel.shape[0]
    split_len = (kvol + split - 1) // split
    if not _tensor_core_shape(in_feats, kernel, allow_tf32):
        # exact fp32 (CUDA cores): one launch per split over a slice of the map, summed in fp32
        acc = None
        for s in range(split):
            lo, hi = s * split_len, min(kvol, (s + 1) * split_len)
            part = conv_forward_implicit_gemm_cuda(in_feats, kernel[lo:hi].contiguous(),
                                                   out_in_map[:, lo:hi].contiguous(), num_out_feats,
                                                   num_out_channels, allow_tf32, allow_fp16, reorder_loc=loc[s])
            acc = part if acc is None else acc + part
        from .nn.functional.conv.conv import _epilogue_torch
        return _epilogue_torch(acc, epilogue) if epilogue else acc
    # one launch per split over its own columns and row order; the partial sums stay in fp32 and the
    # last launch applies the epilogue and rounds once
    acc = torch.empty((num_out_feats, num_out_channels), dtype=torch.float32, device=in_feats.device)
    masks = _tile_mask_of(out_in_map, out_in_map.shape[0])
    out = None
    for s in range(split):
        lo, hi = s * split_len, min(kvol, (s + 1) * split_len)
        last = s == split - 1
        out = conv_forward_implicit_gemm_cuda(
            in_feats, kernel, out_in_map, num_out_feats, num_out_channels, allow_tf32, allow_fp16,
            reorder_loc=loc[s], tile_mask=masks, k_range=(lo, hi), acc_in=acc if s > 0 else None,
            acc_out=None if last else acc, **(epilogue if last else {}))
    return out


def conv_forward_gather_scatter_cuda(in_feats: torch.Tensor, kernel: torch.Tensor, nbmaps: torch.Tensor,
                                     nbsizes_cpu: torch.Tensor, input_mask: torch.Tensor, output_mask: torch.Tensor,
                                     output_size: int, epsilon: float = 0.0, mm_thresh: int = 0, conv_mode: int = 0,
                                     transpose: bool = False, buffer: Optional[torch.Tensor] = None,
                                     allow_tf32: bool = False) -> torch.Tensor:
    """Gather -> grouped GEMM -> scatter
    (torchsparse/backend/convolution/convolution_gather_scatter_cuda.cu:279-311).
    ``epsilon`` / ``mm_thresh`` / ``conv_mode`` / ``buffer`` steer the reference's cuBLAS
    grouping heuristics; this implementation has one grouped GEMM and ignores them."""
    in_feats, kernel = _prep_feats(in_feats, kernel, True)
    _need_cuda(nbmaps, input_mask, output_mask)
    kvol, cin, cout = kernel.shape
    sizes = [int(v) for v in (nbsizes_cpu.tolist() if isinstance(nbsizes_cpu, torch.Tensor) else nbsizes_cpu)]
    if len(sizes) != kvol:
        raise ValueError("nbsizes does not match the kernel volume")
    n_pairs = sum(sizes)
    nbmaps = nbmaps.int().contiguous()
    out = torch.empty((output_size, cout), dtype=in_feats.dtype, device=in_feats.device)
    code = _dtype_code(in_feats)
    ws = _workspace(lib.tsb_conv_gs_workspace_bytes(n_pairs, kvol, cin, cout, code), in_feats.device)
    mask = input_mask if transpose else output_mask
    check(lib.tsb_conv_gs_fwd(_p(in_feats), _p(kernel), _p(nbmaps), i32x(sizes), _p(mask), _p(out),
                              in_feats.shape[0], output_size, kvol, cin, cout, code, _math_mode(in_feats, allow_tf32),
                              int(bool(transpose)), _p(ws), ws.numel(), _stream()),
          "conv_forward_gather_scatter_cuda")
    return out


def conv_forward_fetch_on_demand_cuda(in_feats: torch.Tensor, kernel: torch.Tensor, nbmaps: torch.Tensor,
                                      mapsize: int, nbaddrs: torch.Tensor, qnbaddrs: torch.Tensor, output_size: int,
                                      qmapsize, transpose: bool = False, allow_tf32: bool = False,
                                      allow_fp16: bool = True) -> torch.Tensor:
    """Fused fetch-on-demand forward
    (torchsparse/backend/convolution/convolution_forward_fetch_on_demand_cuda.cu:1981-2133)."""
    in_feats, kernel = _prep_feats(in_feats, kernel, allow_fp16)
    _need_cuda(nbmaps, nbaddrs, qnbaddrs)
    kvol, cin, cout = kernel.shape
    nbmaps = nbmaps.int().contiguous()
    out = torch.empty((output_size, cout), dtype=in_feats.dtype, device=in_feats.device)
    code = _dtype_code(in_feats)
    ws = _workspace(lib.tsb_conv_fod_workspace_bytes(output_size, int(qmapsize), kvol, cin, cout, code),
                    in_feats.device)
    check(lib.tsb_conv_fod_fwd(_p(in_feats), _p(kernel), _p(nbmaps), int(mapsize), _p(nbaddrs), _p(qnbaddrs),
                               int(qmapsize), _p(out), in_feats.shape[0], output_size, kvol, cin, cout, code,
                               _math_mode(in_feats, allow_tf32), int(bool(transpose)), _p(ws), ws.numel(), _stream()),
          "conv_forward_fetch_on_demand_cuda")
    return out


def conv_forward_fetch_on_demand_no_fusion_cuda(in_feats: torch.Tensor, kernel: torch.Tensor, nbmaps: torch.Tensor,
                                                nbsizes_cpu: torch.Tensor, mapsize: int, output_size: int,
                                                transpose: bool = False, allow_tf32: bool = False,
                                                allow_fp16: bool = True) -> torch.Tensor:
    """Per-offset variant of the reference (convolution_forward_fetch_on_demand_cuda.cu:2136-2260).
    Here it derives the scans and runs the same fused launch: the result is identical."""
    kvol = kernel.shape[0]
    sizes = nbsizes_cpu.to(device=in_feats.device, dtype=torch.int32).contiguous()
    nbaddrs = torch.empty(kvol + 1, dtype=torch.int32, device=in_feats.device)
    qnbaddrs = torch.empty(kvol + 1, dtype=torch.int32, device=in_feats.device)
    exclusive_scan_quantified_wrapper(kvol, sizes, nbaddrs, qnbaddrs)
    qmapsize = sum((int(v) + 127) // 128 * 128 for v in nbsizes_cpu.tolist())
    return conv_forward_fetch_on_demand_cuda(in_feats, kernel, nbmaps, mapsize, nbaddrs, qnbaddrs, output_size,
                                             qmapsize, transpose, allow_tf32, allow_fp16)


# --------------------------------------------------------------------------- point / voxel ops
def hash_cuda(coords: torch.Tensor) -> torch.Tensor:
    """(torchsparse/backend/hash/hash_cuda.cu:66-72)."""
    _need_cuda(coords)
    coords = coords.contiguous()
    out = torch.empty(coords.shape[0], dtype=torch.int64, device=coords.device)
    check(lib.tsb_coord_hash(_p(coords), coords.shape[0], _p(out), _stream()), "hash_cuda")
    return out


def kernel_hash_cuda(coords: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
    """(torchsparse/backend/hash/hash_cuda.cu:74-83)."""
    _need_cuda(coords, offsets)
    coords, offsets = coords.contiguous(), offsets.contiguous()
    out = torch.empty((offsets.shape[0], coords.shape[0]), dtype=torch.int64, device=coords.device)
    check(lib.tsb_kernel_hash(_p(coords), coords.shape[0], _p(offsets), offsets.shape[0], _p(out), _stream()),
          "kernel_hash_cuda")
    return out


def hash_query_cuda(queries: torch.Tensor, references: torch.Tensor, indices: Optional[torch.Tensor] = None):
    """Row of each query hash inside ``references`` plus one (0 = absent), like the
    reference entry (torchsparse/backend/others/query_cuda.cu:33-47)."""
    _need_cuda(queries, references)
    queries, references = queries.contiguous(), references.contiguous()
    out = torch.empty(queries.numel(), dtype=torch.int64, device=queries.device)
    ws = _workspace(lib.tsb_hash_query_workspace_bytes(references.numel()), queries.device)
    check(lib.tsb_hash_query(_p(queries), queries.numel(), _p(references), references.numel(), _p(out), _p(ws),
                             ws.numel(), _stream()), "hash_query_cuda")
    return out + 1


def count_cuda(idx: torch.Tensor, s: int) -> torch.Tensor:
    """(torchsparse/backend/others/count_cuda.cu:25-31)."""
    _need_cuda(idx)
    idx = idx.int().contiguous()
    out = torch.empty(int(s), dtype=torch.int32, device=idx.device)
    check(lib.tsb_count(_p(idx), idx.numel(), _p(out), int(s), _stream()), "count_cuda")
    return out


def voxelize_forward_cuda(feats: torch.Tensor, idx: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    """Average pooling of point features into voxels; fp32 accumulation, returned in the
    feature dtype (torchsparse/backend/voxelize/voxelize_cuda.cu:78-95)."""
    _need_cuda(feats, idx, counts)
    feats, idx, counts = feats.contiguous(), idx.int().contiguous(), counts.int().contiguous()
    n, c = feats.shape
    out = torch.empty((counts.shape[0], c), dtype=torch.float32, device=feats.device)
    check(lib.tsb_voxelize_fwd(_p(feats), _p(idx), _p(counts), n, counts.shape[0], c, _dtype_code(feats), _p(out),
                               _stream()), "voxelize_forward_cuda")
    return out.to(feats.dtype)


def devoxelize_forward_cuda(feat: torch.Tensor, indices: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """(torchsparse/backend/devoxelize/devoxelize_cuda.cu:61-78)."""
    _need_cuda(feat, indices, weight)
    feat, indices, weight = feat.contiguous(), indices.int().contiguous(), weight.float().contiguous()
    n, c = indices.shape[0], feat.shape[1]
    out = torch.empty((n, c), dtype=feat.dtype, device=feat.device)
    check(lib.tsb_devoxelize_fwd(_p(feat), _p(indices), _p(weight), n, c, _dtype_code(feat), _p(out), _stream()),
          "devoxelize_forward_cuda")
    return out


def voxelize_backward_cuda(grad_out: torch.Tensor, idx: torch.Tensor, counts: torch.Tensor, n: int) -> torch.Tensor:
    """Gradient of voxelize_forward_cuda with respect to the point features, fp32 [n, C]
    (torchsparse/backend/voxelize/voxelize_cuda.cu:97-114)."""
    _need_cuda(grad_out, idx, counts)
    grad_out, idx, counts = grad_out.float().contiguous(), idx.int().contiguous(), counts.int().contiguous()
    c = grad_out.shape[1]
    out = torch.empty((int(n), c), dtype=torch.float32, device=grad_out.device)
    check(lib.tsb_voxelize_bwd(_p(grad_out), _p(idx), _p(counts), int(n), counts.shape[0], c, _p(out), _stream()),
          "voxelize_backward_cuda")
    return out


def devoxelize_backward_cuda(grad_out: torch.Tensor, indices: torch.Tensor, weight: torch.Tensor, n_vox: int) -> torch.Tensor:
    """Gradient of devoxelize_forward_cuda with respect to the voxel features, fp32 [n_vox, C]
    (torchsparse/backend/devoxelize/devoxelize_cuda.cu:80-98)."""
    _need_cuda(grad_out, indices, weight)
    grad_out, indices, weight = grad_out.float().contiguous(), indices.int().contiguous(), weight.float().contiguous()
    n, c = grad_out.shape
    out = torch.empty((int(n_vox), c), dtype=torch.float32, device=grad_out.device)
    check(lib.tsb_devoxelize_bwd(_p(grad_out), _p(indices), _p(weight), n, int(n_vox), c, _p(out), _stream()),
          "devoxelize_backward_cuda")
    return out


def to_dense_forward_cuda(feats: torch.Tensor, coords: torch.Tensor, spatial_range, outputs: torch.Tensor) -> None:
    """Scatter into the caller's zero-initialised dense tensor
    (torchsparse/backend/voxelize/voxelize_cuda.cu:116-127)."""
    _need_cuda(feats, coords, outputs)
    rng = _host_ints(spatial_range, 4)
    feats, coords = feats.contiguous(), coords.int().contiguous()
    check(lib.tsb_to_dense_fwd(_p(feats), _p(coords), feats.shape[0], feats.shape[1], i32x(rng), _dtype_code(feats),
                               _p(outputs), _stream()), "to_dense_forward_cuda")


def to_dense_backward_cuda(top_grad: torch.Tensor, coords: torch.Tensor, spatial_range, bottom_grad: torch.Tensor) -> None:
    """Gather of the dense gradient into the caller's [N, C] tensor
    (torchsparse/backend/voxelize/voxelize_cuda.cu:129-141)."""
    _need_cuda(top_grad, coords, bottom_grad)
    rng = _host_ints(spatial_range, 4)
    top_grad, coords = top_grad.contiguous(), coords.int().contiguous()
    check(lib.tsb_to_dense_bwd(_p(top_grad), _p(coords), bottom_grad.shape[0], bottom_grad.shape[1], i32x(rng),
                               _dtype_code(bottom_grad), _p(bottom_grad), _stream()), "to_dense_backward_cuda")


def quantize_unique_cuda(xyz: torch.Tensor, voxel_size: Sequence[float], return_index: bool, return_inverse: bool):
    """GPU twin of ``sparse_quantize`` (torchsparse/utils/quantize.py:24-48): returns
    (coords int32 [Nv,3], first_index int64 [Nv] or None, inverse int64 [Np] or None)."""
    import ctypes
    _need_cuda(xyz)
    if xyz.dtype not in (torch.float32, torch.float64):
        xyz = xyz.double()
    xyz = xyz.contiguous()
    n = xyz.shape[0]
    dev = xyz.device
    q_all = torch.empty((n, 3), dtype=torch.int32, device=dev)
    uniq = torch.empty((n, 3), dtype=torch.int32, device=dev)
    first = torch.empty(n, dtype=torch.int64, device=dev) if return_index else None
    inv = torch.empty(n, dtype=torch.int64, device=dev) if return_inverse else None
    result = torch.zeros(8, dtype=torch.int32, device=dev)
    ws = _workspace(lib.tsb_quantize_workspace_bytes(n), dev)
    vox = (ctypes.c_double * 3)(*[float(v) for v in voxel_size])
    check(lib.tsb_quantize_unique(_p(xyz), int(xyz.dtype == torch.float64), n, vox, _p(q_all), _p(uniq), _p(first),
                                  _p(inv), _p(result), _p(ws), ws.numel(), _stream()), "quantize_unique_cuda")
    res = result.cpu().tolist()        # the one synchronisation: voxel count + coordinate bounds
    raise_if_kernel_failed(dev)
    nv = res[0]
    bounds = (tuple(res[1:4]), tuple(res[4:7])) if nv else ((0, 0, 0), (0, 0, 0))
    return uniq[:nv], (first[:nv] if first is not None else None), inv, bounds
