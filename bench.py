#!/usr/bin/env python
"""Benchmark of the sparse-convolution hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE config 2, the one the metric is quoted on): a MinkUNet-class residual sparse
U-Net (the reference's own SparseResUNet42, width 1.0, plus a 19-way linear head) in fp16 inference
on one synthetic LiDAR-like scan per GPU per step (64 rings x 2048 azimuths, 120k rays + 20% box
points, 0.05 m voxels).  One step = voxelisation (sparse_quantize on the GPU) -> 9 kernel maps ->
42 sparse convolutions (+ BN/ReLU/skip) -> logits.  With N GPUs every rank runs its own scan (weak
scaling, scans are independent) and the logits are all-gathered over NCCL once per step.

Prints ONE JSON line (rank 0).  Three passes over the same K steps, each after W warm-up steps:
`value` = scans/s with the points already resident in HBM and `e2e` = the same through the public API
from pinned host memory (H2D of the points and D2H of the logits inside the timed region) — both with
alternate scans issued by two host threads on two streams, each thread waiting for its scan before it
starts its next, one event pair around the K steps and a 256 MiB L2 flush before every step inside it;
then a serial pass (one stream, one thread) with an event pair around every conv launch, from which
`roofline` describes the dominant kernel (the implicit-GEMM conv forward of the layer shape with the
largest total time).  `cpu_baseline` = the reference project's own CPU convolution (oracle/_ref) driving
the same network on a spatial crop of the same scan, scaled by voxel count.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

VOXEL = 0.05
NUM_CLASSES = 19
METRIC = "minkunet_fp16_scans_per_sec"
SCAN_POOL = 4          # distinct scans rotated through the timed steps
MAX_VOXELS = 144_000   # upper bound of the voxels of one scan (every point its own voxel): row bound of the output gather
L2_FLUSH_BYTES = 256 << 20


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "tensor_tflops": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "source": "measured (MEASURED_PEAKS.json; sustained 16-bit GEMM, copy bandwidth)"}
    return {"hbm_gbs": 6650.0, "tensor_tflops": 1400.0, "source": "fallback (6.65 TB/s, 1.4 PFLOP/s sustained)"}


# --------------------------------------------------------------------------------------- model
class SegNet(torch.nn.Module):
    """SparseResUNet42 + linear classifier on the finest decoder output."""

    def __init__(self):
        super().__init__()
        from torchsparse_b200.backbones import SparseResUNet42

        self.backbone = SparseResUNet42(in_channels=4, width_multiplier=1.0)
        self.head = torch.nn.Linear(96, NUM_CLASSES)

    def forward(self, x):
        return self.head(self.backbone(x)[-1].feats)


def make_model(device=None, half=True, engine=True, sort_max_stride=0):
    torch.manual_seed(0)
    model = SegNet()
    for m in model.modules():   # random Kaiming-style init, non-trivial BN statistics
        if hasattr(m, "kernel"):
            fan_in = m.kernel.shape[-2] * (m.kernel.shape[0] if m.kernel.dim() == 3 else 1)
            torch.nn.init.normal_(m.kernel, std=(2.0 / fan_in) ** 0.5)
        if isinstance(m, torch.nn.BatchNorm1d):
            torch.nn.init.uniform_(m.weight, 0.8, 1.2)
            torch.nn.init.uniform_(m.bias, -0.1, 0.1)
            m.running_mean.uniform_(-0.1, 0.1)
            m.running_var.uniform_(0.8, 1.2)
    model.eval()
    if device is not None:
        model = model.to(device)
        if half:
            model = model.half()
        if engine:
            from torchsparse_b200.nn import InferenceEngine
            model.backbone = InferenceEngine(model.backbone, sort_max_stride=sort_max_stride)
    return model


def scan_points(seed: int) -> np.ndarray:
    from torchsparse_b200.utils.synthetic import lidar_scan

    pts = lidar_scan(seed)
    pts[:, :3] -= pts[:, :3].min(0, keepdims=True)
    return pts


# --------------------------------------------------------------------------------------- our arm
def forward_scan(model, pts_dev: torch.Tensor):
    """points [Np,4] on the device -> logits [Nv, 19] (the public-API path a user runs)."""
    import torchsparse_b200 as ts
    from torchsparse_b200.utils import sparse_quantize

    vox, idx, (vmin, vmax) = sparse_quantize(pts_dev[:, :3], VOXEL, return_index=True, return_bounds=True)
    coords = torch.nn.functional.pad(vox, (1, 0))              # batch index 0 in front
    feats = torch.index_select(pts_dev, 0, idx).half()
    bounds = ((0, 0, 0, 0), (0,) + tuple(vmax))                # the points were shifted to start at the origin
    return model(ts.SparseTensor(feats, coords, coord_bounds=bounds))


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None
        self.idx = gpu_index
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "250", "-i", str(gpu_index)],
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
    n_in, n_out, kvol, cin, cout, code, _ = dims
    e = 4 if code == 0 else 2
    flops = 2.0 * pairs * cin * cout
    m_pad = (n_out + 127) // 128 * 128
    byts = n_in * cin * e + n_out * cout * e + kvol * cin * cout * e + m_pad * kvol * 4
    return flops, byts


# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one conv launch from the ncu captures
# summarised under profiles/ (igemm_umma_256x256_31k_rows.md, igemm_umma_96x96_110k_rows.md):
# (kvol, cin, cout) -> (bytes, output rows of the captured launch).  Feature, output and map bytes grow with
# the rows and the weights are small beside them, so the figure is scaled by the row count.
NCU_TRAFFIC = {(27, 256, 256): (23.3e6, 31788), (27, 96, 96): (33.6e6, 110000)}


def map_counts(dims):
    """(valid (row, offset) pairs, issued (128-row tile, offset) blocks) of one conv launch's map."""
    m = dims[6]
    valid = m[: dims[1]] >= 0
    pairs = int(valid.sum().item())
    rows = (m.shape[0] // 128) * 128
    blocks = int((m[:rows].reshape(-1, 128, m.shape[1]) >= 0).any(1).sum().item()) if rows else 0
    return pairs, blocks


def run_ours(args, rank: int, world: int, device: torch.device):
    import torch.distributed as dist
    import torchsparse_b200  # noqa: F401  (fails loudly when libtsb200.so is missing)
    from torchsparse_b200 import backend
    from torchsparse_b200.sharding import PaddedGather

    from torchsparse_b200.nn import functional as F
    F.set_conv_mode(args.conv_mode)
    model = make_model(device, engine=not args.unfused, sort_max_stride=args.sort_max_stride)
    scans = [scan_points(1000 * rank + i) for i in range(SCAN_POOL)]
    host = [torch.from_numpy(s).pin_memory() for s in scans]
    resident = [h.to(device) for h in host]
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step(i, e2e: bool, gather_inline: bool = True):
        h = host[i % SCAN_POOL]
        pts = h.to(device, non_blocking=True) if e2e else resident[i % SCAN_POOL]
        logits = forward_scan(model, pts)      # scans are independent: the only exchange is the gather of outputs
        if world > 1 and gather_inline:
            gather(logits)
        out = logits.cpu() if e2e else logits
        return logits, h.numel() * h.element_size(), (logits.numel() * logits.element_size() if e2e else 0)

    # useful-FLOP bookkeeping: the number of valid (row, offset) pairs of every conv launch of every
    # pooled scan, taken in an untimed pass (the timed pass must not keep maps alive or sync)
    pairs_of_scan = []
    with torch.no_grad():
        for i in range(SCAN_POOL):
            plist = []
            backend.set_launch_observer(lambda name, dims, e0, e1, plist=plist: plist.append(map_counts(dims)))
            forward_scan(model, resident[i])
            backend.set_launch_observer(None)
            pairs_of_scan.append(plist)
    torch.cuda.synchronize()

    records = []
    cur = threading.local()     # (step, launch index within the step) of the scan the calling thread is issuing

    def observer(name, dims, ev0, ev1):
        records.append((cur.step, cur.k, dims[:6], ev0, ev1))
        cur.k += 1

    n_streams = max(1, args.streams)
    # host threads that issue scans (each on its own stream); collectives of a sharded run stay on one thread
    n_threads = max(1, min(args.host_threads, n_streams))
    side = [torch.cuda.Stream(device) for _ in range(n_streams)] if n_streams > 1 else [stream]
    comm_stream = torch.cuda.Stream(device) if world > 1 else None
    gather = PaddedGather(MAX_VOXELS, 19, torch.float16, device) if world > 1 else None   # used on comm_stream only

    host_ms = {"issue": float("nan")}   # host wall time per step spent issuing the step (no final sync)

    def pipelined(n_steps: int, e2e: bool, n_streams: int, n_threads: int):
        """n_steps scans, consecutive ones on alternating streams, issued by n_threads host threads (thread t
        issues scans t, t + T, ... : the Python part of one scan overlaps the native part -- launch calls,
        allocator, readbacks -- of another).  In a sharded run the issuing threads hand each step's logits to
        the calling (main) thread, which alone talks to NCCL, in step order on every rank, on its own stream."""
        io_bytes = {}
        outputs = [None] * n_steps
        ready = [threading.Event() for _ in range(n_steps)]
        t0 = time.perf_counter()

        def issue(first, stride):
            torch.cuda.set_device(device)    # the current device is per thread (a new thread starts on 0)
            with torch.no_grad():
                for i in range(first, n_steps, stride):
                    with torch.cuda.stream(side[i % n_streams]):
                        flush.fill_(i & 0xFF)
                        cur.step, cur.k = i, 0
                        logits, bi, bo = step(i, e2e, gather_inline=False)
                        io_bytes["h2d"], io_bytes["d2h"] = bi, bo
                        if not e2e:
                            # an issuing thread keeps one scan in flight: it waits for its scan's result (as
                            # the e2e pass does by reading the logits back) before it starts its next one
                            torch.cuda.current_stream().synchronize()
                        if world > 1:
                            produced = torch.cuda.Event()
                            produced.record()
                            outputs[i] = (logits, produced)
                    ready[i].set()
                    if os.environ.get("TSB_BENCH_DEBUG"):
                        sys.stderr.write(f"[dbg rank {rank}] issued step {i} at {(time.perf_counter() - t0) * 1e3:.2f} ms\n")

        def gather_outputs():
            for i in range(n_steps):
                if not ready[i].wait(timeout=300) or outputs[i] is None:
                    raise RuntimeError(f"step {i} produced no output (an issuing thread failed)")
                logits, produced = outputs[i]
                outputs[i] = None
                comm_stream.wait_event(produced)
                with torch.cuda.stream(comm_stream):
                    logits.record_stream(comm_stream)
                    gather(logits)

        if n_threads == 1:
            issue(0, 1)
            if world > 1:
                gather_outputs()
        else:
            workers = [threading.Thread(target=issue, args=(t, n_threads)) for t in range(n_threads)]
            for wk in workers:
                wk.start()
            if world > 1:
                gather_outputs()
            for wk in workers:
                wk.join()
        return io_bytes.get("h2d", 0), io_bytes.get("d2h", 0)

    def timed(e2e: bool, observe: bool, n_streams: int = n_streams, n_threads: int = n_threads):
        with torch.no_grad():
            if n_streams == 1:
                for i in range(args.warmup):
                    step(i, e2e)
            else:
                # warm-up through the same threads-and-streams path as the timed steps (a thread's first
                # library calls create per-thread handles)
                pipelined(args.warmup, e2e, n_streams, n_threads)
            barrier()
            evs = []
            launches0 = backend.launch_count()
            backend.set_launch_observer(observer if observe else None)
            h2d = d2h = 0
            t_host0 = time.perf_counter()
            if n_streams == 1:
                for i in range(args.steps):
                    flush.fill_(i & 0xFF)       # evict L2 between steps (outside the timed events)
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(stream)
                    cur.step, cur.k = i, 0
                    _, bi, bo = step(i, e2e)
                    e1.record(stream)
                    h2d, d2h = bi, bo
                    evs.append((e0, e1))
            else:
                # the whole K-step region is timed with one event pair and the L2 flushes are INSIDE it
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for s in side:
                    s.wait_event(e0)
                h2d, d2h = pipelined(args.steps, e2e, n_streams, n_threads)
                for s in side + ([comm_stream] if world > 1 else []):
                    done = torch.cuda.Event()
                    done.record(s)
                    stream.wait_event(done)
                e1.record(stream)
                evs.append((e0, e1))
            host_ms["issue"] = (time.perf_counter() - t_host0) * 1e3 / max(1, args.steps)
            backend.set_launch_observer(None)
            barrier()
            launches = backend.launch_count() - launches0
        total_ms = sum(a.elapsed_time(b) for a, b in evs)
        t = torch.tensor([total_ms], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), launches, h2d, d2h

    sampler = ClockSampler(device.index or 0) if rank == 0 else None
    ms_total, launches, _, _ = timed(False, False)
    host_issue_ms = host_ms["issue"]
    e2e_ms, h2d, d2h = float("nan"), 0, 0
    if not args.no_e2e:
        e2e_ms, _, h2d, d2h = timed(True, False)
    clocks = sampler.stop() if sampler else None     # sampled over both timed passes
    # per-launch durations for the roofline: the same K steps once more, issued serially on one stream
    # with an event pair around every convolution launch (under concurrent streams an event pair would
    # also time the other stream's kernels)
    observed_ms, _, _, _ = timed(False, True, 1, 1)

    if rank != 0:
        return None
    scans_per_step = world
    value = scans_per_step * args.steps / (ms_total / 1e3)
    e2e_value = scans_per_step * args.steps / (e2e_ms / 1e3)

    # ---- roofline of the dominant kernel (largest total time among conv layer shapes)
    pk = peaks()
    by_shape = {}
    for step_i, k_i, key, ev0, ev1 in records:
        pairs, blocks = pairs_of_scan[step_i % SCAN_POOL][k_i]
        d = by_shape.setdefault(key, {"ms": 0.0, "n": 0, "flops": 0.0, "bytes": 0.0, "issued": 0.0})
        fl, by = conv_algorithmic(key + (None,), pairs)
        d["ms"] += ev0.elapsed_time(ev1); d["n"] += 1; d["flops"] += fl; d["bytes"] += by
        d["issued"] += 2.0 * blocks * 128 * key[3] * key[4]     # what the tensor pipe executes (padded tiles)
    roof = None
    conv_ms = sum(d["ms"] for d in by_shape.values())
    if args.dump_layers:
        for key, d in sorted(by_shape.items(), key=lambda kv: -kv[1]["ms"]):
            sys.stderr.write(f"layer n_in={key[0]:7d} n_out={key[1]:7d} kvol={key[2]:2d} {key[3]:3d}->{key[4]:3d}  "
                             f"launches/step={d['n'] / args.steps:4.1f} avg_us={d['ms'] * 1e3 / d['n']:8.1f} "
                             f"total_us/step={d['ms'] * 1e3 / args.steps:8.1f} useful_TF={d['flops'] / d['ms'] / 1e9:7.1f} "
                             f"GB/s={d['bytes'] / d['ms'] / 1e6:7.1f}\n")
    if by_shape:
        key, d = max(by_shape.items(), key=lambda kv: kv[1]["ms"])
        sec = d["ms"] / 1e3
        tf, gb = d["flops"] / sec / 1e12, d["bytes"] / sec / 1e9
        t_tensor, t_hbm = d["flops"] / (pk["tensor_tflops"] * 1e12), d["bytes"] / (pk["hbm_gbs"] * 1e9)
        if t_tensor >= t_hbm:
            roof = {"bound": "tensor", "achieved": round(tf, 3), "peak": pk["tensor_tflops"], "unit": "TFLOP/s",
                    "frac": round(tf / pk["tensor_tflops"], 4)}
        else:
            roof = {"bound": "hbm", "achieved": round(gb, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                    "frac": round(gb / pk["hbm_gbs"], 4)}
        cap = NCU_TRAFFIC.get((key[2], key[3], key[4]))
        roof.update({"traffic": None if cap is None else round(cap[0] * key[1] / cap[1]),
                     "traffic_source": None if cap is None else
                     f"ncu capture of the same kernel on {cap[1]} rows (profiles/), scaled by rows; bytes per launch",
                     "kernel": "igemm conv forward",
                     "layer": {"n_in": key[0], "n_out": key[1], "kvol": key[2], "cin": key[3], "cout": key[4]},
                     "launches": d["n"], "avg_us": round(d["ms"] * 1e3 / d["n"], 2),
                     "useful_flops_per_launch": d["flops"] / d["n"], "algorithmic_bytes_per_launch": d["bytes"] / d["n"],
                     "issued_flops_per_launch": d["issued"] / d["n"],
                     "issued_tflops": round(d["issued"] / sec / 1e12, 2),
                     "issued_frac_of_peak": round(d["issued"] / sec / 1e12 / pk["tensor_tflops"], 4),
                     "note": "achieved/frac count useful FLOPs (2 * valid pairs * Cin * Cout); issued_* count the "
                             "128-row blocks the tensor pipe executes, zero rows of absent neighbours included",
                     "share_of_step": round(d["ms"] / observed_ms, 4),
                     "all_conv_share_of_step": round(conv_ms / observed_ms, 4),
                     "measured_in": "a serial pass over the same steps (one stream, one host thread, an event "
                                    f"pair around every conv launch): {observed_ms / args.steps:.3f} ms per step",
                     "peak_source": pk["source"]})

    out = {
        "metric": METRIC, "value": round(value, 3), "unit": "scans/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_total / args.steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "BASELINE config 2: SparseResUNet42 (MinkUNet-class, cr=1.0) + 19-class head, fp16 "
                               "inference, one synthetic 64-ring LiDAR scan (144k points, 0.05 m voxels) per GPU per step",
                   "voxels_per_scan": int(forward_voxels(scans[0])), "scans_per_step": scans_per_step,
                   "l2": f"{L2_FLUSH_BYTES >> 20} MiB buffer written between steps"
                         + (" (inside the timed region)" if n_streams > 1 else " (outside the timed events)")
                         + f"; {SCAN_POOL} scans rotated",
                   "streams": n_streams, "host_threads": n_threads,
                   "conv_mode": args.conv_mode, "fused_inference_engine": not args.unfused,
                   "sort_max_stride": args.sort_max_stride,
                   "parallelism": (f"scan-sharded x{world}, NCCL all-gather of the logits of every step"
                                   if world > 1 else "single GPU")},
        "e2e": {"value": round(e2e_value, 3), "unit": "scans/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(launches),
        "host_issue_ms_per_step": round(host_issue_ms, 4),
        "clocks": clocks,
        "roofline": roof,
    }
    if world == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_baseline(budget_s=20.0)
    return out


def forward_voxels(pts: np.ndarray) -> int:
    q = np.floor(pts[:, :3] / VOXEL).astype(np.int64)
    return len(np.unique((q[:, 0] * 100003 + q[:, 1]) * 100003 + q[:, 2]))


# --------------------------------------------------------------------------------------- CPU arm
def _crop(pts: np.ndarray, n_target: int):
    """Spatial crop around the sensor holding about n_target voxels; returns (coords, feats, n_vox, n_full)."""
    from oracle import kmap_oracle as ko

    vox, idx = ko.sparse_quantize(pts[:, :3], VOXEL, return_index=True)
    n_full = vox.shape[0]
    centre = np.median(vox, axis=0)
    d = np.abs(vox - centre).max(axis=1)
    order = np.argsort(d, kind="stable")
    keep = np.sort(order[: min(n_target, n_full)])
    coords = np.concatenate([np.zeros((len(keep), 1), np.int32), vox[keep]], 1).astype(np.int32)
    return coords, pts[idx[keep]], len(keep), n_full


def cpu_forward_seconds(model, coords, feats, threads):
    from oracle import net_cpu

    t0 = time.perf_counter()
    net_cpu.forward_cpu(model, coords, feats, threads)
    return time.perf_counter() - t0


def cpu_baseline(budget_s: float = 20.0, steps: int = 1, warmup: int = 0):
    """The network on the host cores through the reference's own CPU convolution (oracle/_ref),
    on a crop of the scan sized for about `budget_s` seconds per pass; scans/s scaled by voxel count."""
    from oracle import net_cpu

    threads = net_cpu.host_threads()
    kind = "reference" if net_cpu.reference_conv_module() is not None else "port"
    model = make_model(None)
    pts = scan_points(0)
    c, f, n, n_full = _crop(pts, 8000)
    cpu_forward_seconds(model, c, f, threads)            # warm caches / thread pools
    probe = cpu_forward_seconds(model, c, f, threads)
    n_target = int(max(3000, min(n_full, 0.7 * n * budget_s / max(probe, 1e-3))))
    c, f, n, n_full = _crop(pts, n_target)
    for _ in range(warmup):
        cpu_forward_seconds(model, c, f, threads)
    times = [cpu_forward_seconds(model, c, f, threads) for _ in range(max(steps, 1))]
    per_pass = sum(times) / len(times)
    value = 1.0 / (per_pass * n_full / n)
    return {"value": round(value, 5), "unit": "scans/s", "cores": threads, "kind": kind,
            "sample": f"full network forward (fp32) on a {n}-voxel crop of the {n_full}-voxel scan, "
                      f"{per_pass:.2f} s per pass, scaled by voxel count",
            "seconds_per_pass": round(per_pass, 3), "crop_voxels": n, "scan_voxels": n_full}


def run_reference(args):
    total_budget = 150.0
    per_step = max(2.0, total_budget / max(args.steps + args.warmup, 1))
    b = cpu_baseline(budget_s=per_step, steps=args.steps, warmup=args.warmup)
    return {
        "impl": "reference", "metric": METRIC, "value": b["value"], "unit": "scans/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(b["seconds_per_pass"] * 1e3, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "BASELINE config 2 network on the host CPU through the reference's CPU convolution "
                               "(fp32 gather-matmul-scatter; the reference has no fp16 / implicit-GEMM CPU path)"},
        "cpu_baseline": b,
        "e2e": {"value": b["value"], "unit": "scans/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def run_layer(args, device):
    """Single sparse Conv3d layer (BASELINE config 5 cell): --layer N,Cin,Cout,kernel,stride,occupancy
    [--dataflow ImplicitGEMM|GatherScatter|FetchOnDemand] [--dtype f16|bf16|f32|tf32] [--sorted].
    Prints one JSON line with time, useful TFLOP/s and algorithmic GB/s of the conv launch."""
    import torchsparse_b200 as ts
    from torchsparse_b200 import backend
    from torchsparse_b200.nn import functional as F
    from torchsparse_b200.utils.synthetic import uniform_voxels

    n, cin, cout, ks, st = [int(v) for v in args.layer.split(",")[:5]]
    occ = float(args.layer.split(",")[5]) if len(args.layer.split(",")) > 5 else 0.05
    dtype = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32, "tf32": torch.float32}[args.dtype]
    from torchsparse_b200 import backends
    backends.allow_tf32 = args.dtype == "tf32"     # "f32" = exact fp32 arithmetic on the CUDA cores
    coords_np, side = uniform_voxels(0, n, occ)
    coords = torch.from_numpy(coords_np).to(device)
    g = torch.Generator(device=device).manual_seed(0)
    feats = torch.randn(n, cin, device=device, generator=g).to(dtype)
    kvol = ks ** 3
    w = (torch.randn(kvol, cin, cout, device=device, generator=g) * (2.0 / (kvol * cin)) ** 0.5).to(dtype)
    cfg = F.conv_config.get_default_conv_config()
    cfg.dataflow = getattr(F.Dataflow, args.dataflow)
    cfg.ifsort = bool(args.sorted)
    pad = (ks - 1) // 2 if (ks % 2 == 1 and st == 1) else 0
    x = ts.SparseTensor(feats, coords)
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record(); y = F.conv3d(x, w, ks, None, st, pad, config=cfg); t1.record()
    torch.cuda.synchronize()
    first_ms = t0.elapsed_time(t1)          # includes the kernel-map build
    kmap = x._caches.kmaps[((1, 1, 1), (ks,) * 3, (st,) * 3, (1, 1, 1))]
    n_out = kmap["sizes"][1]
    pairs = int((kmap["out_in_map"][:n_out] >= 0).sum().item())
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    times = []
    with torch.no_grad():
        for i in range(args.warmup + args.steps):
            flush.fill_(i & 0xFF)
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record(); F.conv3d(x, w, ks, None, st, pad, config=cfg); e1.record()
            torch.cuda.synchronize()
            if i >= args.warmup:
                times.append(e0.elapsed_time(e1))
    ms = statistics.median(times)
    code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dtype]
    fl, by = conv_algorithmic((n, n_out, kvol, cin, cout, code, None), pairs)
    pk = peaks()
    return {"metric": "sparse_conv3d_layer_ms", "value": round(ms, 4), "unit": "ms", "higher_is_better": False,
            "config": {"workload": f"single Conv3d N={n} {cin}->{cout} k{ks} s{st} occupancy {occ} (grid side {side})",
                       "dataflow": args.dataflow, "sorted": bool(args.sorted), "dtype": args.dtype},
            "n_out": n_out, "pairs": pairs, "neighbours_per_row": round(pairs / max(n_out, 1), 2),
            "useful_tflops": round(fl / ms / 1e9, 2), "algorithmic_gbs": round(by / ms / 1e6, 1),
            "frac_tensor_peak": round(fl / ms / 1e9 / pk["tensor_tflops"], 4),
            "frac_hbm_peak": round(by / ms / 1e6 / pk["hbm_gbs"], 4),
            "first_call_ms_incl_kmap": round(first_ms, 3), "steps": args.steps, "warmup": args.warmup}


def run_kmap(args, device):
    """Kernel-map build timing (--kmap N,kernel,stride[,occupancy|lidar]): median ms of a cold build (caches
    cleared every iteration, as torchsparse/utils/tune.py:67-71 does), algorithmic bytes and GB/s."""
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU leg (profiling runs)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer pass (profiling runs)")
    ap.add_argument("--dump-layers", action="store_true", help="per-layer-shape conv timings to stderr")
    ap.add_argument("--layer", default=None, help="N,Cin,Cout,kernel,stride[,occupancy]: single-layer mode")
    ap.add_argument("--kmap", default=None, help="N,kernel,stride[,occupancy|lidar]: kernel-map build timing")
    ap.add_argument("--dataflow", default="ImplicitGEMM")
    ap.add_argument("--dtype", default="f16")
    ap.add_argument("--sorted", action="store_true")
    ap.add_argument("--streams", type=int, default=2,
                    help="CUDA streams the scans of consecutive steps alternate between (1 = strictly serial steps)")
    ap.add_argument("--host-threads", type=int, default=2,
                    help="host threads issuing scans, each on its own stream (<= --streams)")
    ap.add_argument("--unfused", action="store_true", help="run the module graph as written (no InferenceEngine)")
    ap.add_argument("--sort-max-stride", type=int, default=0,
                    help="row-sorted kernel maps for convolutions at tensor strides <= this value (0 = none)")
    ap.add_argument("--conv-mode", type=int, default=0, choices=[0, 1, 2],
                    help="0 unsorted, 1 row-sorted maps, 2 sorted with 3 mask splits (F.set_conv_mode)")
    args = ap.parse_args()
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
    if args.layer or args.kmap:
        if rank == 0:
            print(json.dumps(run_layer(args, device) if args.layer else run_kmap(args, device)), flush=True)
        return
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    try:
        out = run_ours(args, rank, world, device)
        if rank == 0:
            print(json.dumps(out), flush=True)
    finally:
        if world > 1:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
