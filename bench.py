#!/usr/bin/env python
"""Benchmark of the sparse-convolution hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c4]

Workload c2 (BASELINE config 2, the one the metric is quoted on): a MinkUNet-class residual sparse U-Net (the
reference's own SparseResUNet42, width 1.0, plus a 19-way linear head) in fp16 inference on one synthetic
LiDAR-like scan per GPU per step (64 rings x 2048 azimuths, 120k rays + 20% box points, 0.05 m voxels).
One step = voxelisation (sparse_quantize on the GPU) -> 9 kernel maps -> 42 sparse convolutions + 7 pointwise
ones (BatchNorm / ReLU / skip folded in) -> logits.  The whole step is one CUDA graph (StaticEngine: every
size lives in device memory, the kernel maps on a second branch of the graph), replayed per scan; consecutive
scans rotate over eight engines on eight streams whose convolution launches are bounded to 56 CTAs each, so that
several scans are in flight on the GPU.  With N GPUs every rank runs its own scans (weak scaling, scans are independent) and the logits are
all-gathered over NCCL once per step.

Prints ONE JSON line (rank 0):
  value     scans/s with the points already resident in HBM: median over `--repeats` timed passes of K steps
            (one CUDA-event pair around each pass, barrier + synchronize on both sides, max over ranks)
  e2e       the same from pinned host memory: H2D copy of the points and D2H copy of the logits + their row
            count inside the timed region
  roofline  over ALL convolution launches of a step, timed one by one (event pair per launch, queued behind a spin
            kernel) in a serial eager pass over the same scans: useful FLOPs, algorithmic bytes, sum of the
            per-launch roofline minima; `dominant` = the layer shape with the largest total time; `levels` = per
            resolution level; `side_by_side` = the same launches alone with eight scans in flight
  step_roofline  roofline-minimum time of a whole step / measured time of a step
  kmap_build_ms  the kernel-map builds of one scan (5 submanifold, 4 strided + transposed) and the row-sorted
            copies, timed in isolation, with the algorithmic bandwidth of each
  batch32   BASELINE config 3 as written: 32 scans, 32 / N per rank collated into one batch, one gather
  cpu_baseline   the reference project's own CPU convolution (oracle/_ref) driving the same network on the full
            scan, at one thread and at all host threads
`--workload c4` runs BASELINE config 4 (SparseResNet21D, batch 16 sharded 16 / N per rank) and prints its line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

VOXEL = 0.05
NUM_CLASSES = 19
METRIC = "minkunet_fp16_scans_per_sec"
SCAN_POOL = 4           # distinct scans rotated through the timed steps
MAX_POINTS = 144_000    # points of one scan (120k rays + 20 % box points): bound of every level's rows
# voxel grid bound at 0.05 m: 2 x 80 m range in x and y, 25 m in z (sensor range of the generator, with margin)
MAX_EXTENT = (3328, 3328, 512)
L2_FLUSH_BYTES = 256 << 20
# persistent CTAs per convolution launch (of 296 slots) when several engines keep the GPU busy.  Measured with 20 scans
# per timed pass: 8 engines x 56 CTAs 510 scans/s, 7 to 14 engines x 40-56 CTAs 500-506, 20 x 28 485; with 24 scans per
# pass 12 engines x 40 CTAs reach 520 (the last round of a pass is then full)
CONV_GRID_SHARED = 56
C4_VOXEL = (0.1, 0.1, 0.2)
C4_RANGE = (1080, 1080, 40)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "tensor_tflops": p["bf16_tflops"],
                "tensor_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "source": "measured (MEASURED_PEAKS.json: copy bandwidth; 16-bit GEMM burst figure for kernels "
                          "timed one by one, sustained figure for the whole step)"}
    return {"hbm_gbs": 6650.0, "tensor_tflops": 1590.0, "tensor_tflops_sustained": 1400.0,
            "source": "fallback (6.65 TB/s, 1.59 PFLOP/s burst, 1.4 sustained)"}


# --------------------------------------------------------------------------------------- models
class SegNet(torch.nn.Module):
    """SparseResUNet42 + linear classifier on the finest decoder output."""

    def __init__(self):
        super().__init__()
        from torchsparse_b200.backbones import SparseResUNet42

        self.backbone = SparseResUNet42(in_channels=4, width_multiplier=1.0)
        self.head = torch.nn.Linear(96, NUM_CLASSES)

    def forward(self, x):
        return self.head(self.backbone(x)[-1].feats)


class DetNet(torch.nn.Module):
    """SparseResNet21D (BASELINE config 4): the output is the coarsest stage's feature matrix."""

    def __init__(self):
        super().__init__()
        from torchsparse_b200.backbones import SparseResNet21D

        self.backbone = SparseResNet21D(in_channels=5)

    def forward(self, x):
        return self.backbone(x)[-1].feats


def init_model(model):
    torch.manual_seed(0)
    for m in model.modules():   # random Kaiming-style init, non-trivial BN statistics
        if hasattr(m, "kernel"):
            fan_in = m.kernel.shape[-2] * (m.kernel.shape[0] if m.kernel.dim() == 3 else 1)
            torch.nn.init.normal_(m.kernel, std=(2.0 / fan_in) ** 0.5)
        if isinstance(m, torch.nn.BatchNorm1d):
            torch.nn.init.uniform_(m.weight, 0.8, 1.2)
            torch.nn.init.uniform_(m.bias, -0.1, 0.1)
            m.running_mean.uniform_(-0.1, 0.1)
            m.running_var.uniform_(0.8, 1.2)
    return model.eval()


def make_model(device=None, half=True, engine=True, sorted_maps=True, kind="seg", sorted_max_stride=8,
               sorted_strided=False):
    torch.manual_seed(0)
    model = init_model(SegNet() if kind == "seg" else DetNet())
    if device is not None:
        model = model.to(device)
        if half:
            model = model.half()
        if engine:
            from torchsparse_b200.nn import InferenceEngine
            model.backbone = InferenceEngine(model.backbone, sorted_maps=sorted_maps, sorted_max_stride=sorted_max_stride,
                                             sorted_strided=sorted_strided)
    return model


def scan_points(seed: int) -> np.ndarray:
    from torchsparse_b200.utils.synthetic import lidar_scan

    pts = lidar_scan(seed)
    pts[:, :3] -= pts[:, :3].min(0, keepdims=True)
    return pts


def c4_points(seed: int) -> np.ndarray:
    """Multi-sweep detection scan cropped to the config-4 region, shifted so that the region starts at 0."""
    from torchsparse_b200.utils.synthetic import multisweep_scan

    pts = multisweep_scan(seed)
    pts[:, 0] += 54.0
    pts[:, 1] += 54.0
    pts[:, 2] += 5.0
    return pts


# --------------------------------------------------------------------------------------- our arm
def scan_tensor(pts_dev: torch.Tensor, voxel=VOXEL, pad_to: int = 8):
    """points [Np, C] on the device -> (voxel coords int32 [Nv,3], features fp16 [Nv, C padded], max coords)."""
    from torchsparse_b200.utils import sparse_quantize

    vox, idx, (vmin, vmax) = sparse_quantize(pts_dev[:, :3], voxel, return_index=True, return_bounds=True)
    feats = torch.index_select(pts_dev, 0, idx).half()
    if feats.shape[1] % pad_to:
        feats = torch.nn.functional.pad(feats, (0, (-feats.shape[1]) % pad_to))
    return vox, feats, vmax


def forward_scan(model, pts_dev: torch.Tensor):
    """One scan through the eager engine (the public-API path without graph capture) -> logits [Nv, 19]."""
    import torchsparse_b200 as ts

    vox, feats, vmax = scan_tensor(pts_dev)
    coords = torch.nn.functional.pad(vox, (1, 0))              # batch index 0 in front
    bounds = ((0, 0, 0, 0), (0,) + tuple(vmax))                # the points were shifted to start at the origin
    return model(ts.SparseTensor(feats, coords, coord_bounds=bounds))


def forward_batch(model, scans_dev, voxel, spatial_range):
    """A batch of scans collated into one tensor with a common spatial range -> the model's output matrix."""
    import torchsparse_b200 as ts
    from torchsparse_b200.utils.collate import sparse_collate

    items = []
    for p in scans_dev:
        vox, feats, _ = scan_tensor(p, voxel)
        items.append(ts.SparseTensor(feats, vox))
    x = sparse_collate(items)
    x.spatial_range = (len(scans_dev),) + tuple(spatial_range)
    return model(x)


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(gpu_index)],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, v in zip(names, f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.remove(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def conv_algorithmic(dims, pairs: int):
    """Algorithmic work of one conv launch: useful FLOPs and bytes (features, weights, map once)."""
    n_in, n_out, kvol, cin, cout, code = dims[:6]
    e = 4 if code == 0 else 2
    flops = 2.0 * pairs * cin * cout
    m_pad = (n_out + 127) // 128 * 128
    byts = n_in * cin * e + n_out * cout * e + kvol * cin * cout * e + (m_pad * kvol * 4 if kvol > 1 else 0)
    return flops, byts


def launch_counts(dims):
    """(valid (row, offset) pairs, issued (128-row tile, offset) blocks) of one observed conv launch."""
    n_out, kvol, m, tmask = dims[1], dims[2], dims[6], dims[7]
    if m is None:                       # 1x1x1: every row reads itself
        return n_out, (n_out + 127) // 128
    if tmask is not None:
        tm = tmask.cpu().numpy().astype(np.uint32)
        blocks = int(sum(bin(int(v)).count("1") for v in tm))
    else:
        blocks = ((n_out + 127) // 128) * kvol
    pairs = int((m >= 0).sum().item())      # pad rows / columns hold -1 in either layout
    return pairs, blocks


def make_engines(model, device, n_eng, sorted_maps=True, conv_grid=0, overlap_maps=True):
    from torchsparse_b200.nn import StaticEngine

    head = model.head
    return [StaticEngine(model.backbone, lambda outs: head(outs[-1].feats), max_points=MAX_POINTS, point_channels=4,
                         voxel_size=VOXEL, max_extent=MAX_EXTENT, device=device, sorted_maps=sorted_maps,
                         conv_grid=conv_grid, overlap_maps=overlap_maps).capture()
            for _ in range(n_eng)]


def conv_only_ms(model, resident, device, n_eng, conv_grid, steps, flush):
    """ms per scan of the convolution launches alone with `n_eng` scans in flight: every engine replays a graph of the
    eager engine's forward on a tensor whose kernel maps are already cached, i.e. the conv launches and the head,
    nothing else; same L2 flush per scan and same launch bound as the timed step.  Median of 5 passes."""
    import torchsparse_b200 as ts
    from torchsparse_b200 import backend

    keep, engines = [], []
    grid, backend.igemm_tuning["grid"] = backend.igemm_tuning["grid"], conv_grid
    try:
        with torch.no_grad():
            for i in range(n_eng):
                vox, feats, vmax = scan_tensor(resident[i % len(resident)])
                coords = torch.nn.functional.pad(vox, (1, 0))
                bounds = ((0, 0, 0, 0), (0,) + tuple(vmax))
                x = ts.SparseTensor(feats, coords, coord_bounds=bounds)
                model(x)                                   # builds and caches every map of this scan
                torch.cuda.synchronize()

                def again(x=x, feats=feats, coords=coords, bounds=bounds):
                    y = ts.SparseTensor(feats, coords, coord_bounds=bounds)
                    y._caches = x._caches
                    return model(y)

                stream = torch.cuda.Stream(device)
                with torch.cuda.stream(stream):
                    again()
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    out = again()
                engines.append((g, stream))
                keep.append((x, out, again))               # the cached maps must outlive the graphs
    finally:
        backend.igemm_tuning["grid"] = grid
    main = torch.cuda.current_stream()
    times = []
    for _ in range(6):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(main)
        for _, st in engines:
            st.wait_event(e0)
        for i in range(steps):
            g, st = engines[i % n_eng]
            with torch.cuda.stream(st):
                flush.fill_(i & 0xFF)
                g.replay()
        for _, st in engines:
            done = torch.cuda.Event()
            done.record(st)
            main.wait_event(done)
        e1.record(main)
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / steps)
    del engines, keep
    return statistics.median(times[1:])


def event_ms(fn, stream, reps, barrier):
    """`reps` calls of fn(), each bracketed by a barrier + synchronize and one CUDA-event pair on `stream`."""
    out = []
    for _ in range(reps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        fn(e0)
        e1.record(stream)
        barrier()
        out.append(e0.elapsed_time(e1))
    return out


def run_ours(args, rank: int, world: int, device: torch.device):
    import torch.distributed as dist
    import torchsparse_b200 as ts   # fails loudly when libtsb200.so is missing
    from torchsparse_b200 import backend
    from torchsparse_b200.sharding import PaddedGather

    model = make_model(device, sorted_maps=not args.unsorted, sorted_max_stride=args.sorted_max_stride,
                       sorted_strided=args.sorted_strided)
    scans = [scan_points(1000 * rank + i) for i in range(SCAN_POOL)]
    host = [torch.from_numpy(s).pin_memory() for s in scans]
    resident = [h.to(device) for h in host]
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    main = torch.cuda.current_stream()
    n_eng = max(1, args.streams)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    engines = make_engines(model, device, n_eng, not args.unsorted, args.conv_grid, not args.serial_maps)
    # kernels of this library per replay: a further capture (weights are packed by now) runs the forward twice, or
    # three times when the maps go to a side branch (eager, eager with the branch, recording)
    launches0 = backend.launch_count()
    make_engines(model, device, 1, not args.unsorted, args.conv_grid, not args.serial_maps)
    launches_per_step = (backend.launch_count() - launches0) // (2 if args.serial_maps else 3)
    comm_stream = torch.cuda.Stream(device) if world > 1 else None
    gather = PaddedGather(MAX_POINTS, NUM_CLASSES, torch.float16, device) if world > 1 else None
    pinned_out = [torch.empty((MAX_POINTS, NUM_CLASSES), dtype=torch.float16).pin_memory() for _ in range(n_eng)]
    pinned_rec = [torch.empty(16, dtype=torch.int32).pin_memory() for _ in range(n_eng)]

    def steps(e0, n_steps, e2e):
        """n_steps scans, consecutive ones on alternating engines / streams; every stream first waits for e0."""
        for eng in engines:
            eng.stream.wait_event(e0)
        if comm_stream is not None:
            comm_stream.wait_event(e0)
        for i in range(n_steps):
            eng = engines[i % n_eng]
            with torch.cuda.stream(eng.stream):
                flush.fill_(i & 0xFF)                      # L2 flush between steps, inside the timed region
            eng.load(host[i % SCAN_POOL] if e2e else resident[i % SCAN_POOL])
            out, rec = eng.run()
            if world > 1:
                done = torch.cuda.Event()
                done.record(eng.stream)
                comm_stream.wait_event(done)
                with torch.cuda.stream(comm_stream):
                    gather(out, rec[:1])                   # rows padded to the bound, the count travels with them
                    back = torch.cuda.Event()
                    back.record(comm_stream)
                eng.stream.wait_event(back)                # the engine's output buffer is free again
            if e2e:
                with torch.cuda.stream(eng.stream):
                    pinned_out[i % n_eng].copy_(out, non_blocking=True)
                    pinned_rec[i % n_eng].copy_(rec, non_blocking=True)
        for s in [e.stream for e in engines] + ([comm_stream] if comm_stream is not None else []):
            done = torch.cuda.Event()
            done.record(s)
            main.wait_event(done)

    def timed(e2e: bool, reps: int):
        with torch.no_grad():
            barrier()
            e = torch.cuda.Event(); e.record(main)
            steps(e, args.warmup, e2e)
            t_host0 = time.perf_counter()
            ms = event_ms(lambda e0: steps(e0, args.steps, e2e), main, reps, barrier)
            host_ms = (time.perf_counter() - t_host0) * 1e3 / max(1, reps * args.steps)
        t = torch.tensor(ms, dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)       # per pass: the slowest rank
        return [float(v) for v in t.tolist()], host_ms

    sampler = ClockSampler(device.index or 0) if rank == 0 else None
    passes, host_wall_ms = timed(False, args.repeats)
    e2e_passes = []
    if not args.no_e2e:
        e2e_passes, _ = timed(True, args.repeats)
    clocks = sampler.stop() if sampler else None     # sampled over both timed passes
    for eng in engines:
        eng.check()

    # ---- batch of 32 scans sharded over the ranks (BASELINE config 3 as written)
    batch32 = None
    if not args.no_batch32:
        batch32 = run_batch(args, rank, world, device, model, barrier, kind="seg", total=32)

    # ---- per-launch durations: the same scans through the eager engine, serially on one stream, with an event
    # pair around every convolution launch
    records = []
    cur = {"step": 0, "k": 0}

    def observer(name, dims, ev0, ev1):
        records.append((cur["step"], cur["k"], dims, ev0, ev1))
        cur["k"] += 1

    with torch.no_grad():
        for i in range(3):
            forward_scan(model, resident[i % SCAN_POOL])
        torch.cuda.synchronize()
        serial_ms = 0.0
        for i in range(args.steps):
            # the whole eager forward (maps built with their host reads), timed as one piece
            flush.fill_(i & 0xFF)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            vox, feats, vmax = scan_tensor(resident[i % SCAN_POOL])
            coords = torch.nn.functional.pad(vox, (1, 0))
            bounds = ((0, 0, 0, 0), (0,) + tuple(vmax))
            x = ts.SparseTensor(feats, coords, coord_bounds=bounds)
            model(x)
            e1.record()
            torch.cuda.synchronize()
            serial_ms += e0.elapsed_time(e1)
            # the conv launches once more on the cached maps, queued behind a spin kernel and an L2 flush: the host
            # runs ahead of the GPU, so the event pair around a launch holds the kernel's time and nothing of the host's
            cur["step"], cur["k"] = i, 0
            y = ts.SparseTensor(feats, coords, coord_bounds=bounds)
            y._caches = x._caches
            torch.cuda._sleep(40_000_000)
            flush.fill_(i & 0xFF)
            backend.set_launch_observer(observer)
            try:
                model(y)
            finally:
                backend.set_launch_observer(None)
            torch.cuda.synchronize()
    kmap_ms = None if args.no_kmap else kmap_build_ms(model, resident[0], device)
    side_ms = None
    if n_eng > 1 and not args.unsorted and not args.no_kmap:
        side_ms = conv_only_ms(model, resident, device, n_eng, args.conv_grid, args.steps, flush)

    if rank != 0:
        return None
    pk = peaks()
    med = statistics.median(passes)
    value = world * args.steps / (med / 1e3)
    e2e_med = statistics.median(e2e_passes) if e2e_passes else float("nan")
    e2e_value = world * args.steps / (e2e_med / 1e3) if e2e_passes else float("nan")
    ms_per_step = med / args.steps

    # ---- roofline over all conv launches
    counts_cache = {}
    agg = {"ms": 0.0, "flops": 0.0, "bytes": 0.0, "issued": 0.0, "roof_ms": 0.0, "n": 0}
    by_shape, by_level = {}, {}
    for step_i, k_i, dims, ev0, ev1 in records:
        key_c = (step_i % SCAN_POOL, k_i)
        if key_c not in counts_cache:
            counts_cache[key_c] = launch_counts(dims)
        pairs, blocks = counts_cache[key_c]
        ms = ev0.elapsed_time(ev1)
        fl, by = conv_algorithmic(dims, pairs)
        issued = 2.0 * blocks * 128 * dims[3] * dims[4]
        roof = max(fl / (pk["tensor_tflops"] * 1e12), by / (pk["hbm_gbs"] * 1e9)) * 1e3
        shape = (dims[2], dims[3], dims[4], round(dims[1], -4))      # kvol, cin, cout, rows to the nearest 10k
        level = f"rows~{round(dims[1], -4) // 1000}k"
        for d in (agg, by_shape.setdefault(shape, dict.fromkeys(agg, 0.0)), by_level.setdefault(level, dict.fromkeys(agg, 0.0))):
            d["ms"] += ms; d["flops"] += fl; d["bytes"] += by; d["issued"] += issued; d["roof_ms"] += roof; d["n"] += 1

    def summary(d):
        sec = d["ms"] / 1e3
        return {"launches_per_step": round(d["n"] / args.steps, 2), "ms_per_step": round(d["ms"] / args.steps, 4),
                "useful_tflops": round(d["flops"] / sec / 1e12, 2), "issued_tflops": round(d["issued"] / sec / 1e12, 2),
                "algorithmic_gbs": round(d["bytes"] / sec / 1e9, 1),
                "roofline_min_ms_per_step": round(d["roof_ms"] / args.steps, 4),
                "frac_of_roofline": round(d["roof_ms"] / d["ms"], 4)}

    roof = None
    if agg["n"]:
        sec = agg["ms"] / 1e3
        tf, gb = agg["flops"] / sec / 1e12, agg["bytes"] / sec / 1e9
        t_tensor, t_hbm = agg["flops"] / (pk["tensor_tflops"] * 1e12), agg["bytes"] / (pk["hbm_gbs"] * 1e9)
        if t_tensor >= t_hbm:
            roof = {"bound": "tensor", "achieved": round(tf, 2), "peak": pk["tensor_tflops"], "unit": "TFLOP/s",
                    "frac": round(tf / pk["tensor_tflops"], 4)}
        else:
            roof = {"bound": "hbm", "achieved": round(gb, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                    "frac": round(gb / pk["hbm_gbs"], 4)}
        dom_key, dom = max(by_shape.items(), key=lambda kv: kv[1]["ms"])
        # DRAM bytes per launch of the dominant layer shape, from an ncu capture of that layer (small case, one launch:
        # 21.7 MB at 30 912 rows 256 -> 256 k3, 23.9 MB at 110 387 rows 96 -> 96 k3), scaled by rows
        captured = {(27, 256, 256): (21.7e6, 30912), (27, 96, 96): (23.9e6, 110387)}
        cap = captured.get(dom_key[:3])
        traffic = int(cap[0] * dom_key[3] / cap[1]) if cap else None
        roof.update({
            "traffic": traffic,
            "traffic_source": ("dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant layer shape "
                               "(ncu capture of `bench.py --layer ... --lidar-level L --smap`), scaled by rows; per launch"
                               if cap else None),
            "kernel": "igemm_umma_kernel (implicit-GEMM conv forward), all launches of a step",
            "scope": summary(agg),
            "note": "achieved / frac: useful FLOPs (2 * valid pairs * Cin * Cout) or algorithmic bytes (features, "
                    "weights, map once) of all conv launches over the sum of their durations; issued_* counts the "
                    "128-row blocks the tensor pipe executes, zero rows included; frac_of_roofline = sum over "
                    "launches of max(bytes / HBM peak, FLOPs / tensor peak) over the measured time",
            "dominant": dict(summary(dom), layer={"kvol": dom_key[0], "cin": dom_key[1], "cout": dom_key[2],
                                                  "rows_about": dom_key[3]}),
            "levels": {k: summary(v) for k, v in sorted(by_level.items())},
            "side_by_side": None if side_ms is None else {
                "ms_per_step": round(side_ms, 4),
                "useful_tflops": round(agg["flops"] / args.steps / (side_ms / 1e3) / 1e12, 2),
                "frac_of_roofline": round(agg["roof_ms"] / args.steps / side_ms, 4),
                "note": f"the same conv launches (and the head) alone, {n_eng} graphs replayed side by side with "
                        f"the step's launch bound and L2 flush: the regime `value` is measured in"},
            "measured_in": f"a serial eager pass over the same scans on their cached kernel maps (one stream, an event "
                           f"pair around every conv launch, the launches queued behind a spin kernel so that no host "
                           f"time falls between the events); the whole eager forward with its map builds takes "
                           f"{serial_ms / args.steps:.3f} ms per step",
            "peak_source": pk["source"]})
    # roofline-minimum time of a whole step: convs as above + the kernel-map bytes + quantisation bytes
    step_roof = None
    if agg["n"]:
        n_vox = int(forward_voxels(scans[0]))
        kmap_bytes = 0.0
        rows = n_vox
        for lvl in range(5):      # rough level sizes: each stride-2 level keeps the measured share of its rows
            kmap_bytes += rows * 16 * 2 + rows * 2 * 12 + rows * 27 * 4 + 13 * rows * 8
            if lvl < 4:
                kmap_bytes += rows * 16 + 4 * rows * 8 + rows * 8 * 4 * 2
            rows = int(rows * 0.72)
        quant_bytes = MAX_POINTS * (12 + 12 + 8 + 8 + 8)
        min_ms = agg["roof_ms"] / args.steps + (kmap_bytes + quant_bytes) / (pk["hbm_gbs"] * 1e9) * 1e3
        step_roof = {"roofline_min_ms": round(min_ms, 4), "measured_ms": round(ms_per_step, 4),
                     "frac": round(min_ms / ms_per_step, 4),
                     "parts_ms": {"convs": round(agg["roof_ms"] / args.steps, 4),
                                  "kernel_maps_and_quantize": round((kmap_bytes + quant_bytes) / (pk["hbm_gbs"] * 1e9) * 1e3, 4)}}

    out = {
        "metric": METRIC, "value": round(value, 3), "unit": "scans/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "BASELINE config 2: SparseResUNet42 (MinkUNet-class, cr=1.0) + 19-class head, fp16 "
                               "inference, one synthetic 64-ring LiDAR scan (144k points, 0.05 m voxels) per GPU per step",
                   "voxels_per_scan": int(forward_voxels(scans[0])), "scans_per_step": world,
                   "l2": f"{L2_FLUSH_BYTES >> 20} MiB buffer written before every step (inside the timed region); "
                         f"{SCAN_POOL} scans rotated",
                   "engine": "one CUDA graph per scan (sizes in device memory), row-sorted column-major copies of every kernel map"
                             if not args.unsorted else "one CUDA graph per scan, kernel maps as built",
                   "streams": n_eng,
                   "conv_grid": (f"{args.conv_grid} persistent CTAs per convolution launch (of {2 * 148} resident slots): "
                                 "launches of different engines run side by side" if args.conv_grid else "all resident slots"),
                   "parallelism": (f"scan-sharded x{world}, NCCL all-gather of the logits of every step"
                                   if world > 1 else "single GPU")},
        "timing": {"passes": len(passes), "steps_per_pass": args.steps,
                   "ms_per_step_min": round(min(passes) / args.steps, 4),
                   "ms_per_step_max": round(max(passes) / args.steps, 4),
                   "timed_seconds": round(sum(passes) / 1e3, 3),
                   "host_ms_per_step": round(host_wall_ms, 4)},
        "e2e": {"value": round(e2e_value, 3), "unit": "scans/s", "h2d_bytes_per_step": int(host[0].numel() * 4),
                "d2h_bytes_per_step": int(MAX_POINTS * NUM_CLASSES * 2 + 64),
                "ms_per_step_min": round(min(e2e_passes) / args.steps, 4) if e2e_passes else None,
                "ms_per_step_max": round(max(e2e_passes) / args.steps, 4) if e2e_passes else None},
        "gpu_launches": int(launches_per_step * args.steps),
        "gpu_launches_per_step": int(launches_per_step),
        "clocks": clocks,
        "roofline": roof,
        "step_roofline": step_roof,
        "kmap_build_ms": kmap_ms,
        "batch32": batch32,
    }
    if world == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_baseline()
    return out


def forward_voxels(pts: np.ndarray) -> int:
    q = np.floor(pts[:, :3] / VOXEL).astype(np.int64)
    return len(np.unique((q[:, 0] * 100003 + q[:, 1]) * 100003 + q[:, 2]))


def kmap_build_ms(model, pts_dev, device):
    """The kernel maps of one scan built in isolation through the size-in-device-memory builders (the ones the
    graph replays): per map the build and, separately, its row-sorted column-major copy.  Median of 5, events on
    the launching stream, L2 flushed before each."""
    from torchsparse_b200.nn import static_engine as se
    from torchsparse_b200.nn.static_engine import StaticEngine

    eng = StaticEngine(model.backbone, lambda outs: outs[-1].feats, max_points=MAX_POINTS, point_channels=4,
                       voxel_size=VOXEL, max_extent=MAX_EXTENT, device=device, overlap_maps=False)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    result = {}

    class Stop(Exception):
        pass

    def front(post):
        eng.post = post
        eng.points.copy_(pts_dev)
        return eng._forward()

    times = {}

    def timed(name, fn):
        flush.fill_(1)
        torch.cuda._sleep(300000)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); r = fn(); e1.record()
        torch.cuda.synchronize()
        times.setdefault(name, []).append(e0.elapsed_time(e1))
        return r

    sizes = {}     # name -> (kind, row-count tensors on the device): read after the last pass

    class Probe(torch.nn.Module):
        def forward(self, x):
            for lvl in range(5):
                km = timed(f"subm_k3_level{lvl}", lambda: se._subm_map(x, (3, 3, 3)))
                sizes[f"subm_k3_level{lvl}"] = ("subm", x.dyn.rec, x.dyn.rec, 27)
                timed(f"sorted_copy_subm_level{lvl}", lambda: se._sorted(km, "", x.dyn))
                sizes[f"sorted_copy_subm_level{lvl}"] = ("sorted", x.dyn.rec, x.dyn.rec, 27)
                if lvl == 4:
                    break
                kd = timed(f"strided_k2s2_level{lvl}_with_transposed", lambda: se._down_map(x, (2, 2, 2), (2, 2, 2), (0, 0, 0)))
                sizes[f"strided_k2s2_level{lvl}_with_transposed"] = ("down", x.dyn.rec, kd["dyn_out"].rec, 8)
                timed(f"sorted_copy_strided_level{lvl}", lambda: se._sorted(kd, "", kd["dyn_out"]))
                sizes[f"sorted_copy_strided_level{lvl}"] = ("sorted", kd["dyn_out"].rec, kd["dyn_out"].rec, 8)
                timed(f"sorted_copy_transposed_level{lvl}", lambda: se._sorted(kd, "_t", x.dyn))
                sizes[f"sorted_copy_transposed_level{lvl}"] = ("sorted", x.dyn.rec, x.dyn.rec, 8)
                x = se._out_tensor(x.feats, kd["coords"], tuple(2 * s for s in x.stride), kd["dyn_out"], x._caches)
            return [x]

    probe = Probe()
    eng.model = probe
    with torch.no_grad():
        for _ in range(6):
            front(lambda outs: outs[-1].feats)
    med = {k: round(statistics.median(v[1:]), 4) for k, v in times.items()}
    total_build = sum(v for k, v in med.items() if not k.startswith("sorted_copy"))
    total_sorted = sum(v for k, v in med.items() if k.startswith("sorted_copy"))
    # algorithmic bytes of each build (every array read or written once; probes 8 bytes each) over its time
    hbm = peaks()["hbm_gbs"]
    gbs = {}
    for name, (kind, rec_in, rec_out, kvol) in sizes.items():
        n, m = int(rec_in[0].item()), int(rec_out[0].item())
        cap = 512
        while cap < 2 * MAX_POINTS:
            cap *= 2
        pad = lambda r: (r + 127) // 128 * 128
        if kind == "subm":      # coords (insert) + table + coords again + map + one probe per (row, offset pair)
            byts = 16 * n + 8 * cap + 16 * n + pad(n) * kvol * 4 + (kvol // 2) * n * 8
        elif kind == "down":    # coords + candidate keys (written, read) + unique keys + table + output coords +
            byts = 16 * n + 16 * n + 8 * m + 8 * cap + 16 * m + pad(m) * kvol * 4 + pad(n) * kvol * 4 + 8 * n   # both maps + probes
        else:                   # the map read for the keys and for the copy, the copy written, 8-byte (key, row) pairs
            byts = 3 * pad(n) * kvol * 4 + 8 * n
        rate = byts / (med[name] * 1e-3) / 1e9
        gbs[name] = {"rows": n, "algorithmic_gbs": round(rate, 1), "frac_of_hbm": round(rate / hbm, 4)}
    return {"maps_total": round(total_build, 4), "sorted_copies_total": round(total_sorted, 4), "per_map": med,
            "per_map_bandwidth": gbs,
            "note": "5 submanifold k3 maps + 4 strided k2 s2 maps (each with its transposed map) of one scan; "
                    "sizes stay on the device, no host read; median of 5 isolated builds, host launch cost hidden "
                    "behind a spin kernel; per_map_bandwidth: algorithmic bytes over that time against the measured "
                    "copy bandwidth (110 k rows or fewer per build: these launches are latency-bound)"}


def run_batch(args, rank, world, device, model, barrier, kind, total):
    """`total` scans sharded total / world per rank, each rank's shard collated into ONE batch with a common
    spatial range and run through the eager engine, outputs gathered once (NCCL).  Median of 5 passes; one event
    pair around quantisation + collation + forward + gather, max over ranks."""
    import torch.distributed as dist
    from torchsparse_b200.sharding import shard_range, gather_rows_padded

    lo, hi = shard_range(total, world, rank)
    if kind == "seg":
        pts = [torch.from_numpy(scan_points(5000 + i)).to(device) for i in range(lo, hi)]
        voxel, srange = VOXEL, MAX_EXTENT
    else:
        pts = [torch.from_numpy(c4_points(7000 + i)).to(device) for i in range(lo, hi)]
        voxel, srange = C4_VOXEL, C4_RANGE
    rows_bound = 2 * sum(p.shape[0] for p in pts)       # voxels of any level of the shard (k3 s2 can add rows)
    if world > 1:
        t = torch.tensor([rows_bound], dtype=torch.int64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        rows_bound = int(t.item())
    times = []
    out = None
    with torch.no_grad():
        for i in range(7):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = forward_batch(model, pts, voxel, srange)
            if world > 1:
                gather_rows_padded(out, rows_bound)
            e1.record()
            barrier()
            if i >= 2:
                times.append(e0.elapsed_time(e1))
    t = torch.tensor(times, dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = statistics.median([float(v) for v in t.tolist()])
    return {"scans": total, "scans_per_rank": hi - lo, "ms_per_batch": round(ms, 3),
            "value": round(total / (ms / 1e3), 3), "unit": "scans/s", "scaling": "strong",
            "output_rows_this_rank": int(out.shape[0]),
            "note": "eager engine (one collated batch per rank, common spatial range), quantisation of every scan, "
                    "forward and the one output gather inside the timed region; median of 5"}


def run_c4(args, rank, world, device):
    """BASELINE config 4: SparseResNet21D, fp16, batch 16 of multi-sweep scans, 16 / N per rank."""
    import torch.distributed as dist
    import torchsparse_b200  # noqa: F401

    model = make_model(device, kind="det")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(device.index or 0) if rank == 0 else None
    b = run_batch(args, rank, world, device, model, barrier, kind="det", total=16)
    clocks = sampler.stop() if sampler else None
    if rank != 0:
        return None
    return {"metric": "sparseresnet21d_fp16_scans_per_sec", "value": b["value"], "unit": "scans/s", "n_gpus": world,
            "steps": 5, "warmup": 2, "ms_per_step": b["ms_per_batch"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "BASELINE config 4: SparseResNet21D detection backbone, fp16, batch 16 of synthetic "
                                   "10-sweep scans (region 108 x 108 x 8 m, voxel 0.1 x 0.1 x 0.2 m, 5 input channels), "
                                   f"{b['scans_per_rank']} scans per rank, a step = the whole batch",
                       "parallelism": f"scan-sharded x{world}" if world > 1 else "single GPU"},
            "detail": b, "clocks": clocks}


# --------------------------------------------------------------------------------------- CPU arm
def cpu_forward_seconds(model, coords, feats, threads):
    from oracle import net_cpu

    t0 = time.perf_counter()
    net_cpu.forward_cpu(model, coords, feats, threads)
    return time.perf_counter() - t0


def cpu_scan():
    from oracle import kmap_oracle as ko

    pts = scan_points(0)
    vox, idx = ko.sparse_quantize(pts[:, :3], VOXEL, return_index=True)
    coords = np.concatenate([np.zeros((len(vox), 1), np.int32), vox], 1).astype(np.int32)
    return coords, pts[idx]


def cpu_baseline(passes_one: int = 1, with_all_threads: bool = True):
    """The network on the host cores through the reference's own CPU convolution (oracle/_ref) on the FULL scan:
    one thread (its OpenMP loops fork per row, so more threads make it slower) and all host threads."""
    from oracle import net_cpu

    kind = "reference" if net_cpu.reference_conv_module() is not None else "port"
    model = make_model(None)
    coords, feats = cpu_scan()
    n = coords.shape[0]
    all_threads = net_cpu.host_threads()
    small = coords[:2000]
    cpu_forward_seconds(model, small, feats[:2000], 1)        # warm caches / thread pools
    one = [cpu_forward_seconds(model, coords, feats, 1) for _ in range(max(passes_one, 1))]
    t_one = statistics.median(one)
    res = {"value": round(1.0 / t_one, 5), "unit": "scans/s", "cores": 1, "kind": kind,
           "sample": f"full network forward (fp32) on the full {n}-voxel scan, {t_one:.2f} s per pass at 1 thread",
           "seconds_per_pass": round(t_one, 3), "scan_voxels": n,
           "one_thread": {"seconds_per_pass": round(t_one, 3), "scans_per_sec": round(1.0 / t_one, 5)}}
    if with_all_threads and all_threads > 1:
        t_all = cpu_forward_seconds(model, coords, feats, all_threads)
        res["all_threads"] = {"threads": all_threads, "seconds_per_pass": round(t_all, 3),
                              "scans_per_sec": round(1.0 / t_all, 5)}
        if t_all < t_one:
            res.update({"value": round(1.0 / t_all, 5), "cores": all_threads, "seconds_per_pass": round(t_all, 3)})
        res["sample"] += f", {t_all:.2f} s at {all_threads} threads; value = the faster of the two"
    return res


def run_reference(args):
    """The reference's CPU path on the same workload: every step is one full-scan forward at the faster thread
    setting; the number of timed steps is cut so that the run ends within a few minutes."""
    from oracle import net_cpu

    first = cpu_baseline(1, True)
    threads = first["cores"]
    per = first["seconds_per_pass"]
    budget = 150.0
    n_steps = int(max(1, min(args.steps, budget / max(per, 1e-3))))
    model = make_model(None)
    coords, feats = cpu_scan()
    for _ in range(min(args.warmup, 1)):
        cpu_forward_seconds(model, coords, feats, threads)
    times = [cpu_forward_seconds(model, coords, feats, threads) for _ in range(n_steps)]
    sec = statistics.median(times)
    first.update({"value": round(1.0 / sec, 5), "seconds_per_pass": round(sec, 3),
                  "sample": first["sample"] + f"; {n_steps} timed full-scan passes at {threads} thread(s)"})
    return {
        "impl": "reference", "metric": METRIC, "value": first["value"], "unit": "scans/s", "n_gpus": args.gpus,
        "steps": n_steps, "warmup": min(args.warmup, 1), "ms_per_step": round(sec * 1e3, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "BASELINE config 2 network on the host CPU through the reference's CPU convolution "
                               "(fp32 gather-matmul-scatter; the reference has no fp16 / implicit-GEMM CPU path), "
                               "full scan"},
        "cpu_baseline": first,
        "e2e": {"value": first["value"], "unit": "scans/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


# --------------------------------------------------------------------------------------- single layers / maps
_VOXEL_CACHE: dict = {}


def run_layer(args, device):
    """Single sparse Conv3d layer (BASELINE config 5 cell): --layer N,Cin,Cout,kernel,stride,occupancy
    [--dataflow ImplicitGEMM|GatherScatter|FetchOnDemand] [--dtype f16|bf16|f32|tf32] [--sorted] [--transposed].
    Prints one JSON line with time, useful TFLOP/s and algorithmic GB/s of the conv launch."""
    import torchsparse_b200 as ts
    from torchsparse_b200 import backend, backends
    from torchsparse_b200.nn import functional as F
    from torchsparse_b200.utils.synthetic import uniform_voxels

    n, cin, cout, ks, st = [int(v) for v in args.layer.split(",")[:5]]
    occ = float(args.layer.split(",")[5]) if len(args.layer.split(",")) > 5 else 0.05
    dtype = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32, "tf32": torch.float32}[args.dtype]
    backends.allow_tf32 = args.dtype == "tf32"     # "f32" = exact fp32 arithmetic on the CUDA cores
    if args.lidar_level >= 0:
        # rows of the benchmark scan at tensor stride 2^level instead of uniformly scattered voxels
        from torchsparse_b200.utils import sparse_quantize
        vox = sparse_quantize(torch.from_numpy(scan_points(0)).to(device)[:, :3], VOXEL)
        coords = torch.cat([torch.zeros((vox.shape[0], 1), dtype=torch.int32, device=device), vox], 1)
        for _ in range(args.lidar_level):
            coords = F.build_kernel_map(coords, coords.shape[0], 2, 2, 0, None, None, None, "hashmap_on_the_fly")["coords"]
        n, side, occ = coords.shape[0], 0, f"lidar level {args.lidar_level}"
    else:
        key = (n, occ)
        if key not in _VOXEL_CACHE:
            _VOXEL_CACHE.clear()                       # one set at a time (a sweep visits equal keys in a row)
            _VOXEL_CACHE[key] = uniform_voxels(0, n, occ)
        coords_np, side = _VOXEL_CACHE[key]
        coords = torch.from_numpy(coords_np).to(device)
    g = torch.Generator(device=device).manual_seed(0)
    kvol = ks ** 3
    w = (torch.randn(kvol, cin, cout, device=device, generator=g) * (2.0 / (kvol * cin)) ** 0.5).to(dtype)
    cfg = F.conv_config.get_default_conv_config()
    cfg.dataflow = getattr(F.Dataflow, args.dataflow)
    cfg.ifsort = bool(args.sorted)
    pad = (ks - 1) // 2 if (ks % 2 == 1 and st == 1) else 0
    x = ts.SparseTensor(torch.randn(n, cin, device=device, generator=g).to(dtype), coords)
    if args.transposed:
        # the strided conv first (it builds the map), then the transposed conv back to the input coordinates
        mid = F.conv3d(x, w, ks, None, st, pad, config=cfg)
        wt = (torch.randn(kvol, cout, cin, device=device, generator=g) * (2.0 / (kvol * cout)) ** 0.5).to(dtype)
        run = lambda: F.conv3d(mid, wt, ks, None, st, pad, config=cfg, transposed=True)
    else:
        run = lambda: F.conv3d(x, w, ks, None, st, pad, config=cfg)
    run()
    torch.cuda.synchronize()
    kmap = x._caches.kmaps[((1, 1, 1), (ks,) * 3, (st,) * 3, (1, 1, 1))]
    if args.smap:
        # the engine's form of the map: row-sorted, column-major, per-tile masks (tsb_map_sorted_cm)
        sfx = "_t" if args.transposed else ""
        rows_valid = kmap["sizes"][0] if args.transposed else kmap["sizes"][1]
        sm = backend.sorted_cm_artefacts_cuda(kmap["out_in_map" + sfx], rows_valid)
        xin, wk = (mid.feats, wt) if args.transposed else (x.feats, w)
        run = lambda: backend.conv_forward_implicit_gemm_cuda(xin, wk, None, rows_valid, wk.shape[2], backends.allow_tf32,
                                                              True, smap=sm)
        run()
        torch.cuda.synchronize()
    if args.cmap:
        # the map as built, stored column-major ([kvol][rows]): the per-offset reads of the kernel become contiguous
        sfx = "_t" if args.transposed else ""
        rows_valid = kmap["sizes"][0] if args.transposed else kmap["sizes"][1]
        rm = kmap["out_in_map" + sfx]
        cm = rm.t().contiguous()
        tmask = backend.tile_mask_cuda(cm, rows_valid, 1, cm.shape[1])
        xin, wk = (mid.feats, wt) if args.transposed else (x.feats, w)
        run = lambda: backend.conv_forward_implicit_gemm_cuda(xin, wk, cm, rows_valid, wk.shape[2], backends.allow_tf32,
                                                              True, tile_mask=tmask, map_strides=(1, cm.shape[1]))
        run()
        torch.cuda.synchronize()
    n_out = kmap["sizes"][0] if args.transposed else kmap["sizes"][1]
    n_in = kmap["sizes"][1] if args.transposed else n
    if args.backward:
        # one gradient launch of the layer (not transposed): the weight gradient on the tensor cores (fp32 result), or
        # the input gradient = the forward kernel on the transposed map with W transposed per offset
        from torchsparse_b200.nn.functional.conv.kmap import transpose_kernel_map
        dy = torch.randn(n_out, cout, device=device, generator=g).to(dtype)
        fmap = kmap["out_in_map"]
        if args.backward == "wgrad":
            run = lambda: backend.conv_wgrad_implicit_gemm_cuda(x.feats, dy, fmap)
        else:
            tmap, wt_ = transpose_kernel_map(kmap)["out_in_map_t"], w.transpose(1, 2).contiguous()
            run = lambda: backend.conv_forward_implicit_gemm_cuda(dy, wt_, tmap, n, cin, backends.allow_tf32, True)
        run()
        torch.cuda.synchronize()
    pairs = int((kmap["out_in_map"][:kmap["sizes"][1]] >= 0).sum().item())
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    times = []
    with torch.no_grad():
        for i in range(args.warmup + args.steps):
            flush.fill_(i & 0xFF)
            torch.cuda._sleep(300000)          # the host finishes queueing behind this spin
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record(); run(); e1.record()
            torch.cuda.synchronize()
            if i >= args.warmup:
                times.append(e0.elapsed_time(e1))
    ms = statistics.median(times)
    code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dtype]
    ci, co = (cout, cin) if args.transposed else (cin, cout)
    fl, by = conv_algorithmic((n_in, n_out, kvol, ci, co, code), pairs)
    pk = peaks()
    return {"metric": "sparse_conv3d_layer_ms", "value": round(ms, 4), "unit": "ms", "higher_is_better": False,
            "config": {"workload": f"single Conv3d N={n} {cin}->{cout} k{ks} s{st}{' transposed' if args.transposed else ''} "
                                   f"occupancy {occ} (grid side {side})",
                       "dataflow": args.dataflow, "sorted": bool(args.sorted), "engine_sorted_map": bool(args.smap),
                       "pass": args.backward or "forward",
                       "dtype": args.dtype},
            "n_out": n_out, "pairs": pairs, "neighbours_per_row": round(pairs / max(n_out, 1), 2),
            "useful_tflops": round(fl / ms / 1e9, 2), "algorithmic_gbs": round(by / ms / 1e6, 1),
            "frac_tensor_peak": round(fl / ms / 1e9 / pk["tensor_tflops"], 4),
            "frac_hbm_peak": round(by / ms / 1e6 / pk["hbm_gbs"], 4), "steps": args.steps, "warmup": args.warmup}


def run_kmap(args, device):
    """Kernel-map build timing (--kmap N,kernel,stride[,occupancy|lidar]): median ms of a cold build through the
    eager builders (caches cleared every iteration, as torchsparse/utils/tune.py:67-71 does; includes the one
    size readback of a strided build), algorithmic bytes and GB/s."""
    from torchsparse_b200.nn import functional as F
    from torchsparse_b200.utils.synthetic import uniform_voxels

    parts = args.kmap.split(",")
    n, ks, st = int(parts[0]), int(parts[1]), int(parts[2])
    occ = parts[3] if len(parts) > 3 else "0.05"
    if occ == "lidar":
        from torchsparse_b200.utils import sparse_quantize
        pts = torch.from_numpy(scan_points(0)).to(device)
        vox = sparse_quantize(pts[:, :3], VOXEL)
        coords = torch.cat([torch.zeros((vox.shape[0], 1), dtype=torch.int32, device=device), vox], 1)
        n = coords.shape[0]
    else:
        coords = torch.from_numpy(uniform_voxels(0, n, float(occ))[0]).to(device)
    pad = (ks - 1) // 2 if (ks % 2 == 1 and st == 1) else 0
    kvol = ks ** 3
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    times, m = [], 0
    for i in range(args.warmup + args.steps):
        flush.fill_(i & 0xFF)
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        km = F.build_kernel_map(coords, n, ks, st, pad, None, None, None, "hashmap_on_the_fly")
        e1.record()
        torch.cuda.synchronize()
        m = km["sizes"][1]
        if i >= args.warmup:
            times.append(e0.elapsed_time(e1))
    ms = statistics.median(times)
    cap = 512
    while cap < 2 * max(n, m):
        cap *= 2
    m_pad = (m + 127) // 128 * 128
    if st == 1:   # coords + table write + coords re-read + map write + probe reads
        byts = n * 16 + cap * 12 + n * 16 + m_pad * kvol * 4 + (kvol // 2 if kvol % 2 else kvol) * n * 8
    else:         # + candidate keys written, sorted (read+write), unique; outputs; stage-3 probes
        slots = ((ks + st - 1) // st) ** 3
        byts = n * 16 + 4 * n * slots * 8 + m * 24 + cap * 12 + n * 16 + m_pad * kvol * 4 + n * 8
    pk = peaks()
    return {"metric": "kmap_build_ms", "value": round(ms, 4), "unit": "ms", "higher_is_better": False,
            "config": {"workload": f"kernel map N={n} k{ks} s{st} ({occ})", "n_out": m},
            "algorithmic_bytes": byts, "algorithmic_gbs": round(byts / ms / 1e6, 1),
            "frac_hbm_peak": round(byts / ms / 1e6 / pk["hbm_gbs"], 4), "min_ms": round(min(times), 4),
            "steps": args.steps, "warmup": args.warmup}


def run_pointops(args, device):
    """Point <-> voxel operators on N points (--pointops N): median ms, algorithmic bytes and GB/s of the coordinate
    hash, the hash join, the voxel quantisation, average-pool voxelisation and trilinear devoxelisation.  Inputs are
    larger than L2 at the default N; a 256 MiB fill separates the timed calls."""
    from torchsparse_b200 import backend

    n = int(args.pointops)
    g = torch.Generator(device=device).manual_seed(0)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    side = max(8, int(round((n / 0.05) ** (1 / 3))))                 # ~5 % occupancy of a cube
    coords = torch.randint(0, side, (n, 4), generator=g, device=device, dtype=torch.int32)
    coords[:, 0] = 0
    xyz = torch.rand((n, 3), generator=g, device=device) * (side * 0.05)
    c_pt, c_vox = 4, 32
    feats = torch.randn((n, c_pt), generator=g, device=device)
    uniq, inverse = torch.unique(backend.hash_cuda(coords), return_inverse=True)
    nv = uniq.numel()
    counts = torch.bincount(inverse, minlength=nv).int()
    idx = inverse.int()
    vfeat = torch.randn((nv, c_vox), generator=g, device=device).half()
    nbr = torch.randint(-1, nv, (n, 8), generator=g, device=device, dtype=torch.int32)
    wts = torch.rand((n, 8), generator=g, device=device)
    refs = uniq[torch.randperm(nv, generator=g, device=device)]
    queries = backend.hash_cuda(coords)
    cap = 512
    while cap < 2 * nv:
        cap *= 2
    cases = {
        # name: (callable, algorithmic bytes)
        "coord_hash": (lambda: backend.hash_cuda(coords), n * 16 + n * 8),
        "hash_query": (lambda: backend.hash_query_cuda(queries, refs), nv * 8 + cap * 16 + n * 8 + n * 8),
        "quantize_unique": (lambda: backend.quantize_unique_cuda(xyz, (0.05, 0.05, 0.05), False, True), n * 12 + n * 8),
        "voxelize": (lambda: backend.voxelize_forward_cuda(feats, idx, counts), n * c_pt * 4 + n * 4 + nv * (c_pt * 4 + 4)),
        "devoxelize": (lambda: backend.devoxelize_forward_cuda(vfeat, nbr, wts), n * 64 + n * c_vox * 2 + nv * c_vox * 2),
    }
    pk = peaks()
    out = {"metric": "pointops_ms", "unit": "ms", "higher_is_better": False,
           "config": {"workload": f"point ops on N={n} points, {nv} voxels, {c_pt} point channels (fp32), "
                                  f"{c_vox} voxel channels (fp16)"}, "steps": args.steps, "warmup": args.warmup, "ops": {}}
    for name, (fn, byts) in cases.items():
        times = []
        for i in range(args.warmup + args.steps):
            flush.fill_(i & 0xFF)
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= args.warmup:
                times.append(e0.elapsed_time(e1))
        ms = statistics.median(times)
        out["ops"][name] = {"ms": round(ms, 4), "algorithmic_bytes": int(byts), "algorithmic_gbs": round(byts / ms / 1e6, 1),
                            "frac_hbm_peak": round(byts / ms / 1e6 / pk["hbm_gbs"], 4)}
    out["value"] = round(sum(v["ms"] for v in out["ops"].values()), 4)
    return out


def run_sweep(args, device):
    """BASELINE config 5 (--sweep reduced|full): single-layer cells through `run_layer` in one process.
    reduced: {k3 s1, k2 s2, k2 s2 transposed} x {16, 64, 128, 256} channels x {10k, 100k, 1M} voxels at 5 % occupancy
    x the three dataflows x {f16, tf32, f32}, plus the 1 % and 20 % occupancies at 100k voxels and the 2M-voxel cells
    for the implicit GEMM in f16.  full: every cell of the grid.  One JSON line with a list of cells."""
    import copy

    kinds = [(3, 1, False), (2, 2, False), (2, 2, True)]
    chans = [16, 64, 128, 256]
    flows = ["ImplicitGEMM", "GatherScatter", "FetchOnDemand"]
    dtypes = ["f16", "tf32", "f32"]
    cells = []
    if args.sweep == "full":
        for n in (10_000, 100_000, 1_000_000, 2_000_000):
            for occ in (0.01, 0.05, 0.2):
                for kind in kinds:
                    for c in chans:
                        for fl in flows:
                            for dt in dtypes:
                                cells.append((n, occ, kind, c, fl, dt))
    else:
        for n in (10_000, 100_000, 1_000_000):
            for kind in kinds:
                for c in chans:
                    for fl in flows:
                        for dt in dtypes:
                            cells.append((n, 0.05, kind, c, fl, dt))
        for occ in (0.01, 0.2):
            for kind in kinds:
                for c in chans:
                    cells.append((100_000, occ, kind, c, "ImplicitGEMM", "f16"))
        for kind in kinds:
            for c in chans:
                cells.append((2_000_000, 0.05, kind, c, "ImplicitGEMM", "f16"))
    out = []
    for n, occ, (ks, st, tr), c, fl, dt in cells:
        a = copy.copy(args)
        a.layer, a.dataflow, a.dtype, a.transposed = f"{n},{c},{c},{ks},{st},{occ}", fl, dt, tr
        a.sorted, a.smap, a.lidar_level, a.backward = False, False, -1, ""
        try:
            r = run_layer(a, device)
            out.append({"n": n, "occupancy": occ, "kernel": ks, "stride": st, "transposed": tr, "channels": c,
                        "dataflow": fl, "dtype": dt, "ms": r["value"], "pairs": r["pairs"], "n_out": r["n_out"],
                        "useful_tflops": r["useful_tflops"], "algorithmic_gbs": r["algorithmic_gbs"],
                        "frac_tensor_peak": r["frac_tensor_peak"], "frac_hbm_peak": r["frac_hbm_peak"]})
        except Exception as e:      # a cell that does not fit or is not supported is reported, not fatal
            out.append({"n": n, "occupancy": occ, "kernel": ks, "stride": st, "transposed": tr, "channels": c,
                        "dataflow": fl, "dtype": dt, "error": f"{type(e).__name__}: {e}"[:200]})
        torch.cuda.empty_cache()
    pk = peaks()
    return {"metric": "layer_sweep", "unit": "ms", "higher_is_better": False, "steps": args.steps, "warmup": args.warmup,
            "config": {"workload": f"BASELINE config 5 layer sweep ({args.sweep}), {len(out)} cells"},
            "peaks": pk, "cells": out}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c2", "c4"])
    ap.add_argument("--repeats", type=int, default=25, help="timed passes of --steps steps each (the median is reported)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU leg (profiling runs)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer pass (profiling runs)")
    ap.add_argument("--no-batch32", action="store_true", help="skip the 32-scan batch (profiling runs)")
    ap.add_argument("--no-kmap", action="store_true", help="skip the isolated kernel-map timings")
    ap.add_argument("--layer", default=None, help="N,Cin,Cout,kernel,stride[,occupancy]: single-layer mode")
    ap.add_argument("--kmap", default=None, help="N,kernel,stride[,occupancy|lidar]: kernel-map build timing")
    ap.add_argument("--sweep", default=None, choices=["reduced", "full"], help="BASELINE config 5: single-layer cells")
    ap.add_argument("--pointops", default=None, help="N: timings of the point <-> voxel operators on N points")
    ap.add_argument("--dataflow", default="ImplicitGEMM")
    ap.add_argument("--dtype", default="f16")
    ap.add_argument("--sorted", action="store_true")
    ap.add_argument("--transposed", action="store_true")
    ap.add_argument("--backward", default="", choices=["", "wgrad", "dgrad"],
                    help="layer mode: time the weight-gradient or the input-gradient launch instead of the forward")
    ap.add_argument("--cmap", action="store_true", help="layer mode: run on a column-major copy of the map as built")
    ap.add_argument("--smap", action="store_true", help="layer mode: run on the row-sorted column-major map of the engines")
    ap.add_argument("--lidar-level", type=int, default=-1, help="layer mode: rows of the benchmark scan at stride 2^L")
    ap.add_argument("--streams", type=int, default=8,
                    help="engines (each with its own stream and graph) that consecutive scans alternate between")
    ap.add_argument("--unsorted", action="store_true", help="run on the kernel maps as built (no row-sorted copies)")
    ap.add_argument("--gather", type=int, default=0, choices=[0, 2],
                    help="gathered operand of the conv kernel: 0 = cp.async by the gather warps (default), 2 = copy engine (TMA gather4)")
    ap.add_argument("--max-offsets", type=int, default=0,
                    help="split tiles of the sorted maps with more kernel offsets than this into parts (0: library default)")
    ap.add_argument("--conv-grid", type=int, default=-1,
                    help="upper bound of the persistent CTAs of a convolution launch (0: every resident slot; "
                         "-1: 56 when several engines share the GPU, else every slot)")
    ap.add_argument("--sorted-max-stride", type=int, default=16, help="row-sorted map copies up to this tensor stride")
    ap.add_argument("--no-sorted-strided", dest="sorted_strided", action="store_false",
                    help="no row-sorted copies of the strided / transposed maps (only of the submanifold ones)")
    ap.add_argument("--serial-maps", action="store_true",
                    help="record every scan as one chain of launches (kernel maps built between the convolutions, "
                         "not on a second branch of the graph)")
    ap.add_argument("--hash64", action="store_true",
                    help="kernel-map tables with 64-bit keys even where the level's key space fits 32 bits")
    ap.add_argument("--tune", default="", help="launch-configuration overrides of the conv kernel, e.g. stages=3,ctas=2,cpb=2")
    args = ap.parse_args()
    if args.hash64:
        from torchsparse_b200 import backends as _backends
        _backends.hash_keys_32bit = False
    if args.tune:
        from torchsparse_b200 import backend as _backend
        for kv in args.tune.split(","):
            k, v = kv.split("=")
            _backend.igemm_tuning[k] = int(v)
    if not (args.layer or args.kmap or args.pointops or args.sweep) and args.steps < args.streams:
        args.streams = max(1, args.steps)        # a pass of fewer scans than engines keeps only that many in flight
    if args.conv_grid < 0 and 1 < args.streams < 6:
        args.conv_grid = 296 // args.streams       # few scans in flight: each convolution launch gets a larger share
    if args.conv_grid < 0:
        args.conv_grid = CONV_GRID_SHARED if (args.streams > 1 and not args.layer and not args.kmap and not args.pointops and not args.sweep) else 0
    if args.conv_grid and args.layer:      # the engines of the step benchmark get it as their own setting
        from torchsparse_b200 import backend as _backend
        _backend.igemm_tuning["grid"] = args.conv_grid
    if args.max_offsets:
        from torchsparse_b200 import backend as _backend
        _backend.split_max_offsets = args.max_offsets
    if args.gather:
        from torchsparse_b200 import backend as _backend
        _backend.igemm_tuning["gather"] = args.gather
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(run_reference(args)), flush=True)
        return

    import torch.distributed as dist

    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if args.layer or args.kmap or args.pointops or args.sweep:
        if rank == 0:
            fn = run_sweep if args.sweep else run_layer if args.layer else run_kmap if args.kmap else run_pointops
            print(json.dumps(fn(args, device)), flush=True)
        return
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    try:
        out = run_c4(args, rank, world, device) if args.workload == "c4" else run_ours(args, rank, world, device)
        if rank == 0:
            print(json.dumps(out), flush=True)
    finally:
        if world > 1:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
