"""Data-generation throughput: the GPU chaos-game / voxeliser kernels against the native CPU generator.

Three stages of ``scaffold generate_fractals`` + volume generation are timed on the same inputs:

* category search: orbit statistics of a batch of IFS candidates (``sb_ifs_search`` vs ``sb_ifs_orbit_cpu``),
* instance generation: point clouds (``sb_ifs_points`` vs the CPU orbit with points kept),
* volume generation: point cloud -> occupancy / coloured volume (``sb_voxel_bbox`` + ``sb_voxel_paint`` vs
  ``sb_voxelize_cpu``).

The CPU numbers are one core of this machine (the generator is block-partitioned over ranks, one core each);
GPU numbers include the host <-> device copies the front ends do. Both produce the same bits
(``tests/test_datagen_gpu.py``), so items per second is the whole story.

Role of the reference's hot loops: ScaFFold/datagen/category_search.py:114-201, volumegen.py:221-294.
"""
from __future__ import annotations

import time

import numpy as np
import torch

from ..data import ifs


def _time(fn, repeat: int = 3) -> float:
    fn()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    best = float("inf")
    for _ in range(repeat):
        t0 = time.perf_counter()
        fn()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        best = min(best, time.perf_counter() - t0)
    return best


def main(args=None):
    rng = np.random.default_rng(7)
    rows = []
    scale = 7
    grid = 2 ** scale
    n_points = grid ** 3 // 256  # points per orbit at this scale (the CLI's point_num rule)
    # contractive maps so that the orbits stay finite
    batch = 256
    params = rng.uniform(-0.6, 0.6, (batch, 2, 13))
    params[:, 0, 12] = 0.5
    params[:, 1, 12] = 1.0
    seeds = rng.integers(1, 2 ** 62, batch, dtype=np.uint64)

    t_cpu = _time(lambda: ifs.orbit_stats(params[:32], seeds[:32], n_points, "cpu"), 2) / 32
    t_gpu = _time(lambda: ifs.orbit_stats(params, seeds, n_points, "cuda")) / batch
    rows.append({"stage": "category search (orbit statistics)", "points": n_points, "cpu_items_s": 1 / t_cpu,
                 "gpu_items_s": 1 / t_gpu, "speedup": t_cpu / t_gpu})

    t_cpu = _time(lambda: ifs.orbit_points(params[:32], seeds[:32], n_points, "cpu"), 2) / 32
    t_gpu = _time(lambda: ifs.orbit_points(params, seeds, n_points, "cuda")) / batch
    rows.append({"stage": "instance generation (point clouds)", "points": n_points, "cpu_items_s": 1 / t_cpu,
                 "gpu_items_s": 1 / t_gpu, "speedup": t_cpu / t_gpu})

    pts, flags = ifs.orbit_points(params[:8], seeds[:8], n_points, "cuda")
    clouds = [p for p, f in zip(pts, flags) if f == 0 and np.isfinite(p).all()] or [rng.normal(size=(n_points, 3)).astype(np.float32)]
    colors = [(1.0, 0.5, 0.25)] * len(clouds)
    labels = list(range(1, len(clouds) + 1))
    t_cpu = _time(lambda: [ifs.voxelize_cpu(c, grid) for c in clouds], 2) / len(clouds)
    t_gpu = _time(lambda: ifs.render_shard_cuda(clouds, colors, labels, grid, (0, 0, 0), (grid,) * 3)) / len(clouds)
    rows.append({"stage": f"voxelise + paint one instance into a {grid}^3 volume", "points": n_points,
                 "cpu_items_s": 1 / t_cpu, "gpu_items_s": 1 / t_gpu, "speedup": t_cpu / t_gpu})
    for r in rows:
        print(f"datagen  {r['stage']:55s} {r['points']:8d} points/item : CPU {r['cpu_items_s']:10.1f} items/s   "
              f"GPU {r['gpu_items_s']:10.1f} items/s   -> {r['speedup']:.1f}x", flush=True)
    return rows
