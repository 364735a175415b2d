"""Seeded synthetic inputs with the shapes of the benchmark workloads: LiDAR-like scans
(rings + boxes), multi-sweep detection scans, and uniformly occupied grids."""
from typing import Tuple

import numpy as np

__all__ = ["lidar_scan", "multisweep_scan", "uniform_voxels"]


def _ring_points(rng: np.random.Generator, n_rays: int, origin=(0.0, 0.0, 0.0)) -> np.ndarray:
    """n_rays rays drawn from a 64-ring x 2048-azimuth spinning-LiDAR pattern (elevations
    -25..+3 degrees); each ray ends at its ground-plane hit (z = -1.7 m) or at 80 m."""
    elev = np.deg2rad(np.linspace(-25.0, 3.0, 64))
    azim = np.linspace(0.0, 2.0 * np.pi, 2048, endpoint=False)
    pick = rng.choice(64 * 2048, size=n_rays, replace=False)
    e, a = elev[pick // 2048], azim[pick % 2048]
    rng_max = np.full(n_rays, 80.0)
    down = np.sin(e) < -1e-6
    ground = np.where(down, -1.7 / np.where(down, np.sin(e), -1.0), np.inf)
    r = np.minimum(rng_max, ground)
    r = r * (1.0 + 0.002 * rng.standard_normal(n_rays))   # range noise
    xyz = np.stack([r * np.cos(e) * np.cos(a), r * np.cos(e) * np.sin(a), r * np.sin(e)], axis=1)
    return xyz + np.asarray(origin)[None, :]


def lidar_scan(seed: int, n_rays: int = 120_000, box_fraction: float = 0.2, n_boxes: int = 30) -> np.ndarray:
    """One synthetic scan, float32 [n_rays*(1+box_fraction), 4] = (x, y, z, intensity):
    ring points plus points uniform inside random axis-aligned boxes with 1-4 m sides."""
    rng = np.random.default_rng(seed)
    pts = [_ring_points(rng, n_rays)]
    n_box_pts = int(n_rays * box_fraction)
    centres = np.stack([rng.uniform(-40, 40, n_boxes), rng.uniform(-40, 40, n_boxes), rng.uniform(-1.7, 0.5, n_boxes)], 1)
    sides = rng.uniform(1.0, 4.0, (n_boxes, 3))
    which = rng.integers(0, n_boxes, n_box_pts)
    pts.append(centres[which] + (rng.uniform(0, 1, (n_box_pts, 3)) - 0.5) * sides[which])
    xyz = np.concatenate(pts, 0)
    inten = rng.uniform(0, 1, (xyz.shape[0], 1))
    return np.concatenate([xyz, inten], 1).astype(np.float32)


def multisweep_scan(seed: int, sweeps: int = 10, n_rays: int = 25_000, box_fraction: float = 0.2,
                    n_boxes: int = 30) -> np.ndarray:
    """Detection-style input: `sweeps` copies of the scan generator (rings + the same boxes seen from
    a moving sensor) with small ego offsets merged, cropped to [-54,54]^2 x [-5,3] m; float32
    [~sweeps*n_rays*(1+box_fraction), 5] = (x, y, z, intensity, time in [0,0.5])."""
    rng = np.random.default_rng(seed)
    centres = np.stack([rng.uniform(-40, 40, n_boxes), rng.uniform(-40, 40, n_boxes), rng.uniform(-1.7, 0.5, n_boxes)], 1)
    sides = rng.uniform(1.0, 4.0, (n_boxes, 3))
    n_box_pts = int(n_rays * box_fraction)
    out = []
    for s in range(sweeps):
        origin = (0.4 * s * rng.uniform(0.8, 1.2), 0.05 * rng.standard_normal(), 0.0)
        which = rng.integers(0, n_boxes, n_box_pts)
        boxes = centres[which] + (rng.uniform(0, 1, (n_box_pts, 3)) - 0.5) * sides[which]
        xyz = np.concatenate([_ring_points(rng, n_rays, origin), boxes], 0)
        t = np.full((xyz.shape[0], 1), 0.5 * s / max(sweeps - 1, 1))
        out.append(np.concatenate([xyz, rng.uniform(0, 1, (xyz.shape[0], 1)), t], 1))
    p = np.concatenate(out, 0)
    keep = (np.abs(p[:, 0]) < 54) & (np.abs(p[:, 1]) < 54) & (p[:, 2] > -5) & (p[:, 2] < 3)
    return p[keep].astype(np.float32)


def uniform_voxels(seed: int, n: int, occupancy: float, batch: int = 1) -> Tuple[np.ndarray, int]:
    """n distinct int32 voxel coordinates (b,x,y,z) per batch item, uniform in a cubic grid whose
    side is chosen so that n = occupancy * side^3.  Returns (coords, side)."""
    rng = np.random.default_rng(seed)
    side = max(int(np.ceil((n / occupancy) ** (1.0 / 3.0))), 1)
    rows = []
    for b in range(batch):
        lin = rng.choice(side ** 3, size=n, replace=False)
        xyz = np.stack(np.unravel_index(lin, (side,) * 3), 1)
        rows.append(np.concatenate([np.full((n, 1), b), xyz], 1))
    return np.concatenate(rows).astype(np.int32), side
