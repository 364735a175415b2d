"""A whole scan -> logits forward recorded once and replayed as one CUDA graph.

The reference drives every layer from Python and reads sizes back from the device while it builds
kernel maps (torchsparse/nn/functional/conv/kmap/func/hashmap_on_the_fly.py:33,
torchsparse/backend/others/sparsemapping_cuda.cu:435,477); at batch 1 the host, not the GPU, sets the
pace.  Here nothing in the forward depends on a number the host would have to read: every buffer is
allocated for an upper bound of its rows, the real row counts and coordinate bounds live in device memory
("level records", include/tsb200.h) and every kernel reads them there.  The sequence of launches is then
the same for every input, so it is captured into a CUDA graph once and each later scan costs one graph
launch on the host.

`DynSparseTensor` is the tensor type of this mode (features / coordinates padded to `n_max` rows plus the
level record); the fused modules of `torchsparse_b200.nn.fused` dispatch on it, so the model code that runs
under capture is the model's own `forward`.  Results equal the eager engine's for the valid rows."""
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .. import backend, backends
from .._lib import lib, check, i32x, TSB_DEV_TABLE_FULL, TSB_DEV_BAD_INDEX, TSB_DEV_LIMIT
from ..tensor import SparseTensor
from ..utils.utils import make_ntuple

__all__ = ["DynInfo", "DynSparseTensor", "StaticEngine", "dyn_conv"]


def _next_pow2(n: int) -> int:
    p = 1
    while p < n:
        p <<= 1
    return p


def _bits_for(cells: int) -> int:
    """Bits that hold every key below `cells` plus a sentinel above them."""
    return max(1, int(cells + 1).bit_length())


class DynInfo:
    """What a tensor of the static mode carries besides features and coordinates: the level record (int32[16],
    device; [0] = rows), the row bound its buffers are allocated for, and the engine-wide settings."""

    __slots__ = ("rec", "n_max", "ctx")

    def __init__(self, rec: torch.Tensor, n_max: int, ctx: "_Context") -> None:
        self.rec, self.n_max, self.ctx = rec, n_max, ctx


class _Context:
    """Settings shared by all levels of one engine: the static bound of the voxel grid (for the number of key
    bits that get sorted), the status word the kernels report into, whether maps are row-sorted."""

    def __init__(self, max_extent: Sequence[int], batch: int, status: torch.Tensor, sorted_maps: bool,
                 row_cap: int) -> None:
        self.max_extent = tuple(int(v) for v in max_extent)
        self.batch = int(batch)
        self.status = status
        self.sorted_maps = sorted_maps
        self.row_cap = int(row_cap)      # no level is given buffers for more rows than this
        # Kernel maps depend on coordinates only, so they can be built ahead of the convolutions, on a stream of
        # their own.  `log` (a list, or None) collects the map requests of a forward in network order; a later
        # forward that was given them as its plan builds every map on the side stream first and lets each
        # convolution wait for the event recorded behind the map it reads.
        self.log: Optional[List[Tuple]] = None

    def key_bits(self, tensor_stride: Sequence[int]) -> int:
        cells = self.batch
        for ext, s in zip(self.max_extent, tensor_stride):
            cells *= ext // s + 2
        return _bits_for(cells)


class DynSparseTensor(SparseTensor):
    """SparseTensor whose buffers hold `dyn.n_max` rows of which the first `dyn.rec[0]` (a number in device
    memory) are real."""

    def __init__(self, feats: torch.Tensor, coords: torch.Tensor, stride, dyn: DynInfo, caches=None,
                 spatial_range=None) -> None:
        super().__init__(feats, coords, stride, spatial_range)
        if caches is not None:
            self._caches = caches
        self.dyn = dyn


def _out_tensor(feats, coords, stride, dyn: DynInfo, caches) -> DynSparseTensor:
    out = DynSparseTensor.__new__(DynSparseTensor)
    out.feats, out.coords, out.stride, out.spatial_range, out._caches, out.dyn = feats, coords, stride, None, caches, dyn
    return out


def _level_table(caches, stride, n_max: int, device, key_bits: int):
    """(keys, vals, capacity, fresh) of the hash table of a tensor stride; vals is None for a table of 32-bit keys
    (packed slots), taken whenever the level's key space allows it."""
    from .. import backends

    tables = caches.__dict__.setdefault("dyn_tables", {})
    hit = tables.get(stride)
    if hit is not None:
        return hit + (False,)
    cap = _next_pow2(max(512, 2 * n_max))
    keys = torch.empty(cap, dtype=torch.int64, device=device)
    vals = None if (backends.hash_keys_32bit and key_bits <= 32) else torch.empty(cap, dtype=torch.int32, device=device)
    tables[stride] = (keys, vals, cap)
    return keys, vals, cap, True


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _subm_map(x: DynSparseTensor, kernel_size) -> Dict:
    caches, dyn = x._caches, x.dyn
    key = (x.stride, kernel_size, (1, 1, 1), (1, 1, 1))
    kmap = caches.kmaps.get(key)
    if kmap is not None:
        return kmap
    dev = x.coords.device
    kvol = kernel_size[0] * kernel_size[1] * kernel_size[2]
    keys, vals, cap, fresh = _level_table(caches, x.stride, dyn.n_max, dev, dyn.ctx.key_bits(x.stride))
    out_in_map = torch.empty((backend.pad128(dyn.n_max), kvol), dtype=torch.int32, device=dev)
    check(lib.tsb_kmap_subm_dyn(keys.data_ptr(), _ptr(vals), cap, x.coords.data_ptr(), dyn.n_max,
                                dyn.rec.data_ptr(), i32x(kernel_size), int(fresh), out_in_map.data_ptr(),
                                dyn.ctx.status.data_ptr(), backend._stream()), "tsb_kmap_subm_dyn")
    kmap = {"out_in_map": out_in_map, "coords": x.coords, "dyn_in": dyn, "dyn_out": dyn}
    caches.kmaps[key] = kmap
    return kmap


def _down_map(x: DynSparseTensor, kernel_size, stride, padding) -> Dict:
    caches, dyn = x._caches, x.dyn
    key = (x.stride, kernel_size, stride, (1, 1, 1))
    kmap = caches.kmaps.get(key)
    if kmap is not None:
        return kmap
    dev = x.coords.device
    kvol = kernel_size[0] * kernel_size[1] * kernel_size[2]
    slots = lib.tsb_kmap_down_slots(i32x(kernel_size), i32x(stride))
    if slots <= 0:
        raise ValueError("bad kernel size / stride")
    m_max = min(dyn.n_max * slots, dyn.ctx.row_cap)     # more outputs than this are reported (TSB_DEV_LIMIT)
    out_stride = tuple(a * b for a, b in zip(x.stride, stride))
    keys, vals, cap, _ = _level_table(caches, out_stride, m_max, dev, dyn.ctx.key_bits(out_stride))
    out_coords = torch.empty((m_max, 4), dtype=torch.int32, device=dev)
    out_in_map = torch.empty((backend.pad128(m_max), kvol), dtype=torch.int32, device=dev)
    map_t = torch.empty((backend.pad128(dyn.n_max), kvol), dtype=torch.int32, device=dev)
    rec_out = torch.empty(16, dtype=torch.int32, device=dev)
    nbytes = lib.tsb_kmap_down_dyn_workspace_bytes(dyn.n_max, i32x(kernel_size), i32x(stride))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    check(lib.tsb_kmap_down_dyn(keys.data_ptr(), _ptr(vals), cap, x.coords.data_ptr(), dyn.n_max,
                                dyn.rec.data_ptr(), i32x(kernel_size), i32x(stride), i32x(padding),
                                dyn.ctx.key_bits(out_stride), m_max, out_coords.data_ptr(), out_in_map.data_ptr(),
                                map_t.data_ptr(), rec_out.data_ptr(), dyn.ctx.status.data_ptr(), ws.data_ptr(),
                                ws.numel(), backend._stream()), "tsb_kmap_down_dyn")
    dyn_out = DynInfo(rec_out, m_max, dyn.ctx)
    kmap = {"out_in_map": out_in_map, "out_in_map_t": map_t, "coords": out_coords, "dyn_in": dyn, "dyn_out": dyn_out}
    caches.kmaps[key] = kmap
    caches.cmaps.setdefault(out_stride, (out_coords, None))
    caches.__dict__.setdefault("dyn_levels", {})[out_stride] = dyn_out
    return kmap


def _sorted(kmap: Dict, sfx: str, valid: DynInfo) -> "backend.SortedMap":
    art = kmap.get("_cm" + sfx)
    if art is None:
        art = kmap["_cm" + sfx] = backend.sorted_cm_artefacts_cuda(kmap["out_in_map" + sfx], valid.n_max, valid.rec)
    return art


def _map_for(coords: torch.Tensor, stride, dyn: DynInfo, caches, request):
    """The kernel map a layer asks for (built on first use, cached on the tensor cache) together with the form the
    convolution reads it in: the row-sorted column-major copy, or the per-tile offset masks of the map as built.
    request = (tensor stride, kernel size, conv stride, padding, dilation, transposed, sorted)."""
    _, ks, st, pad, dil, transposed, want_sorted = request
    if transposed:
        out_stride = tuple(a // b for a, b in zip(stride, st))
        kmap = caches.kmaps.get((out_stride, ks, st, dil))
        if kmap is None:
            raise ValueError("transposed convolution needs the kernel map of the matching strided convolution")
        sfx, dyn_out = "_t", kmap["dyn_in"]
        out_coords = caches.cmaps[out_stride][0]
    else:
        level = _out_tensor(None, coords, stride, dyn, caches)
        if any(v != 1 for v in st):
            kmap = _down_map(level, ks, st, pad)
            sfx, dyn_out = "", kmap["dyn_out"]
            out_coords, out_stride = kmap["coords"], tuple(a * b for a, b in zip(stride, st))
        else:
            kmap = _subm_map(level, ks)
            sfx, dyn_out, out_coords, out_stride = "", dyn, coords, stride
    if want_sorted:
        art = _sorted(kmap, sfx, dyn_out)
    else:
        art = kmap.get("_tmask" + sfx)
        if art is None:
            art = kmap["_tmask" + sfx] = backend.tile_mask_cuda(kmap["out_in_map" + sfx], dyn_out.n_max,
                                                                n_rows_dev=dyn_out.rec)
    return kmap, sfx, dyn_out, out_coords, out_stride, art


def _prebuild_maps(x: DynSparseTensor, plan: Sequence[Tuple], side: torch.cuda.Stream) -> torch.cuda.Event:
    """Builds every kernel map of `plan` (the requests of an earlier forward, in network order) on `side`, which
    branches off the current stream here; behind each map an event is recorded that its first reader waits for.
    Returns the event that closes the branch: the caller's stream must wait for it before it ends."""
    caches, main = x._caches, torch.cuda.current_stream(x.coords.device)
    caches.__dict__.setdefault("dyn_levels", {}).setdefault(x.stride, x.dyn)
    caches.cmaps.setdefault(x.stride, (x.coords, None))
    side.wait_stream(main)
    with torch.cuda.stream(side):
        seen = set()
        for request in plan:
            stride, transposed = request[0], request[5]
            level = caches.cmaps.get(stride)
            dyn = caches.__dict__["dyn_levels"].get(stride)
            if level is None or dyn is None:
                break                       # not the network the plan was taken from: the layers build on demand
            kmap, sfx, *_ = _map_for(level[0], stride, dyn, caches, request)
            key = (id(kmap), sfx, request[6])
            if key not in seen:
                seen.add(key)
                ev = torch.cuda.Event()
                ev.record(side)
                kmap["_ready" + sfx] = ev    # a later form of the same map (sorted / masks) moves the event back
        done = torch.cuda.Event()
        done.record(side)
    return done


def dyn_conv(layer, x: DynSparseTensor, residual: Optional[torch.Tensor]) -> DynSparseTensor:
    """A fused convolution layer (torchsparse_b200.nn.fused.FusedConv) on a tensor of the static mode."""
    dyn, caches = x.dyn, x._caches
    parts = getattr(x, "parts", None)
    feats, feats2 = (parts[0], parts[1]) if (parts is not None and len(parts) == 2) else (x.feats, None)
    kernel = layer._input_kernel(feats.shape[1] + (0 if feats2 is None else feats2.shape[1]))
    plan = layer._plan
    if plan is None or not plan.valid_for(kernel, backends.allow_tf32):
        plan = layer._plan = backend.IgemmLayerPlan(kernel, layer.scale, layer.shift, backends.allow_tf32)
    caches.__dict__.setdefault("dyn_levels", {}).setdefault(x.stride, dyn)
    caches.cmaps.setdefault(x.stride, (x.coords, None))
    if layer.pointwise:
        out = torch.empty((dyn.n_max, plan.cout), dtype=plan.dtype, device=plan.device)
        backend.igemm_plan_launch(plan, feats, None, dyn.n_max, residual, layer.relu, in_feats2=feats2,
                                  n_out_dev=dyn.rec, out=out)
        return _out_tensor(out, x.coords, x.stride, dyn, caches)
    want_sorted = bool(dyn.ctx.sorted_maps and layer._wants_sorted(x.stride))
    request = (x.stride, layer.kernel_size, layer.stride, make_ntuple(layer.padding, 3), layer.dilation,
               bool(layer.transposed), want_sorted)
    if dyn.ctx.log is not None:
        dyn.ctx.log.append(request)
    kmap, sfx, dyn_out, out_coords, out_stride, art = _map_for(x.coords, x.stride, dyn, caches, request)
    ready = kmap.pop("_ready" + sfx, None)
    if ready is not None:                  # built on the side stream: its first reader waits, later ones follow it
        torch.cuda.current_stream(plan.device).wait_event(ready)
    out = torch.empty((dyn_out.n_max, plan.cout), dtype=plan.dtype, device=plan.device)
    if want_sorted:
        backend.igemm_plan_launch(plan, feats, None, dyn_out.n_max, residual, layer.relu, in_feats2=feats2,
                                  smap=art, n_out_dev=dyn_out.rec, out=out)
    else:
        backend.igemm_plan_launch(plan, feats, kmap["out_in_map" + sfx], dyn_out.n_max, residual, layer.relu,
                                  tile_mask=art, in_feats2=feats2, n_out_dev=dyn_out.rec, out=out)
    return _out_tensor(out, out_coords, out_stride, dyn_out, caches)


class StaticEngine:
    """points [n_points, C] (fp32) -> `post(model(SparseTensor))`, captured as one CUDA graph.

    `model` is a network of fused modules (`fuse_for_inference` / `InferenceEngine`), `post` turns its output
    into one tensor (e.g. a linear head on the finest features).  `max_points` bounds the points of a scan
    (and so the voxels of every level), `max_extent` the voxel coordinates at stride 1 (x, y, z; e.g. sensor
    range / voxel size): it fixes how many key bits the sorts cover, and a scan that exceeds it is reported by
    `check()`, not silently mishandled.  Point coordinates must be >= 0 (shift them by the lower corner of the
    sensor range).  A scan with fewer than `max_points` points is padded with copies of its first point, which
    the voxel deduplication removes again.

    The captured launches carry the stream's scheduling slot of the convolution kernel: replays of one engine
    must not overlap on the GPU (use one engine per stream).  `conv_grid` bounds the persistent CTAs of every
    convolution launch (0: all resident slots of the device): with several engines kept busy on their own streams
    a share of the device per launch (e.g. 56 of 296 slots with eight engines on a B200) lets launches of different
    engines run side by side, where full-device launches would wait for each other's last CTAs.
    `overlap_maps=False` records the forward as one chain (maps built where the first layer needs them)."""

    def __init__(self, model: torch.nn.Module, post: Callable, *, max_points: int, point_channels: int,
                 voxel_size: float, max_extent: Sequence[int], device: torch.device,
                 dtype: torch.dtype = torch.float16, pad_channels: int = 8, sorted_maps: bool = True,
                 stream: Optional[torch.cuda.Stream] = None, row_cap: Optional[int] = None,
                 conv_grid: int = 0, overlap_maps: bool = True) -> None:
        self.model, self.post = model, post
        self.max_points, self.c_in, self.c_pad = int(max_points), int(point_channels), int(pad_channels)
        self.voxel = (float(voxel_size),) * 3 if isinstance(voxel_size, (int, float)) else tuple(voxel_size)
        self.device, self.dtype = device, dtype
        self.sorted_maps = sorted_maps
        # a strided convolution whose kernel is larger than its stride can create more outputs than inputs
        # (up to 8x for k3 s2); buffers of the coarser levels are bounded by this many rows
        self.row_cap = int(row_cap) if row_cap is not None else 2 * self.max_points
        self.conv_grid = int(conv_grid)
        self.max_extent = tuple(int(v) for v in max_extent)
        self.stream = stream if stream is not None else torch.cuda.Stream(device)
        # kernel maps are built on a second stream that branches off `stream` behind the quantisation and joins it
        # again before the forward ends: in the recorded graph the map builds of the deeper levels (about a hundred
        # short, latency-bound launches) run beside the convolutions of the earlier ones instead of between them
        self.side = torch.cuda.Stream(device) if overlap_maps else None
        self._map_plan: Optional[List[Tuple]] = None
        self.points = torch.zeros((self.max_points, self.c_in), dtype=torch.float32, device=device)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.out: Optional[torch.Tensor] = None
        self.rec: Optional[torch.Tensor] = None
        self.status: Optional[torch.Tensor] = None

    # ---- the recorded computation
    def _forward(self) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        import ctypes

        dev, n = self.device, self.max_points
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        ctx = _Context(self.max_extent, 1, status, self.sorted_maps, self.row_cap)
        xyz = self.points[:, :3].contiguous()
        q_all = torch.empty((n, 3), dtype=torch.int32, device=dev)
        uniq = torch.empty((n, 3), dtype=torch.int32, device=dev)
        first = torch.empty(n, dtype=torch.int64, device=dev)
        result = torch.zeros(8, dtype=torch.int32, device=dev)
        ws = torch.empty(lib.tsb_quantize_workspace_bytes(n), dtype=torch.uint8, device=dev)
        vox = (ctypes.c_double * 3)(*self.voxel)
        cells = 1
        for e in self.max_extent:
            cells *= e + 1
        stream = backend._stream()
        check(lib.tsb_quantize_unique_bits(xyz.data_ptr(), 0, n, vox, _bits_for(cells), q_all.data_ptr(), uniq.data_ptr(),
                                           first.data_ptr(), None, result.data_ptr(), ws.data_ptr(), ws.numel(), stream),
              "tsb_quantize_unique_bits")
        coords = torch.empty((n, 4), dtype=torch.int32, device=dev)
        feats = torch.empty((n, self.c_pad), dtype=self.dtype, device=dev)
        check(lib.tsb_voxel_inputs(self.points.data_ptr(), self.c_in, first.data_ptr(), uniq.data_ptr(), result.data_ptr(),
                                   0, n, coords.data_ptr(), feats.data_ptr(), self.c_pad, backend._dtype_code(feats), stream),
              "tsb_voxel_inputs")
        rec = torch.empty(16, dtype=torch.int32, device=dev)
        check(lib.tsb_level_record_from_quantize(result.data_ptr(), 0, rec.data_ptr(), status.data_ptr(), stream),
              "tsb_level_record_from_quantize")
        x = DynSparseTensor(feats, coords, 1, DynInfo(rec, n, ctx))
        done = None
        if self.side is not None and self._map_plan is not None:
            done = _prebuild_maps(x, self._map_plan, self.side)
        elif self.side is not None:
            ctx.log = []
        out = self.post(self.model(x))
        if done is not None:
            torch.cuda.current_stream(dev).wait_event(done)      # the branch joins: nothing of it outlives the forward
        elif ctx.log is not None:
            self._map_plan = ctx.log
        return out, rec, status

    def capture(self) -> "StaticEngine":
        """One eager pass (packs weights, makes launch plans, loads kernels), then the recording."""
        from .. import operators

        torch.cuda.synchronize(self.device)
        was_lazy, operators.lazy = operators.lazy, True
        # no per-launch status reads or observers while recording (they would synchronise)
        was_checked, backend.check_kernel_status = backend.check_kernel_status, False
        observer, backend._observer = backend._observer, None
        grid, backend.igemm_tuning["grid"] = backend.igemm_tuning["grid"], self.conv_grid or backend.igemm_tuning["grid"]
        try:
            with torch.no_grad(), torch.cuda.stream(self.stream):
                self._forward()
                self.stream.synchronize()
                if self.side is not None:       # once more with the maps on their own stream, as it will be recorded
                    self._forward()
                    torch.cuda.synchronize(self.device)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.stream):
                    self.out, self.rec, self.status = self._forward()
                self.graph = g
        finally:
            operators.lazy = was_lazy
            backend.check_kernel_status, backend._observer = was_checked, observer
            backend.igemm_tuning["grid"] = grid
        torch.cuda.synchronize(self.device)
        return self

    # ---- per scan
    def load(self, points: torch.Tensor) -> None:
        """Copies a scan (device tensor, or pinned host tensor: the copy is asynchronous) into the engine's
        input buffer on the engine's stream."""
        n = points.shape[0]
        if n > self.max_points or points.shape[1] != self.c_in:
            raise ValueError(f"scan of shape {tuple(points.shape)} does not fit ({self.max_points}, {self.c_in})")
        with torch.cuda.stream(self.stream):
            self.points[:n].copy_(points, non_blocking=True)
            if n < self.max_points:
                self.points[n:] = self.points[0]

    def run(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """Replays the graph on the engine's stream.  Returns (output [max rows, ...], level record): the first
        `record[0]` rows of the output are the scan's; both are the engine's own buffers, overwritten by the next
        replay."""
        if self.graph is None:
            self.capture()
        with torch.cuda.stream(self.stream):
            self.graph.replay()
        return self.out, self.rec

    def __call__(self, points: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        self.load(points)
        return self.run()

    def check(self) -> None:
        """Reads the status word of the last replay (a synchronisation) and raises on a reported problem."""
        v = int(self.status.item())
        if v & TSB_DEV_LIMIT:
            raise RuntimeError("StaticEngine: the scan exceeds the engine's bounds (max_extent / max_points), or has "
                               "negative coordinates")
        if v & TSB_DEV_TABLE_FULL:
            raise RuntimeError("StaticEngine: a hash table overflowed")
        if v & TSB_DEV_BAD_INDEX:
            raise RuntimeError("StaticEngine: inconsistent hash table (an output coordinate was not found)")
        w = int(backend._status_word(self.device).item())
        if w:
            raise RuntimeError(f"StaticEngine: a bounded wait inside a convolution kernel ran out (code {w})")
