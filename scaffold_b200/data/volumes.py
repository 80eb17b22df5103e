"""Volume generation: compose fractal instances into labelled, physically sharded volumes.

Layout written below ``config.dataset_dir`` (ScaFFold/datagen/volumegen.py:297-590):

    volumes_contents.csv                       [idx, cat1, inst1, cat2, inst2, ...] one row per volume
    volumes/<split>/<i>_shardNNNNNN.npy        float32 (3, d, h, w): per-category RGB colour
    masks/<split>/<i>_shardNNNNNN_mask.npy     uint16  (d, h, w):    category + 1, 0 = background
    train_unique_mask_vals, val_unique_mask_vals   pickles {"mask_values": [...]}

``<split>`` is ``training`` / ``validation`` (``val_split`` percent, drawn with
``random.sample`` seeded by ``dataset_seed``); one file per (volume, shard) with
shards as defined by ``dc_num_shards`` / ``dc_shard_dims``. Tasks
``(volume, shard)`` are block-partitioned over the ranks. Every rank reports
success or failure and all ranks raise together. A heartbeat file marks the
staging directory as alive for concurrent jobs' garbage collection.

Rasterisation runs on the GPU when one is visible (``csrc/ifs.cu``), else on the
native CPU rasteriser.
"""
from __future__ import annotations

import os
import pickle
import random
import time
from math import ceil
from pathlib import Path
from typing import List, Optional, Sequence, Tuple

import numpy as np

from ..utils import dist as D
from ..utils.sharding import canonical_sharding, shard_file_suffix, spatial_slices, total_shards
from . import ifs
from .category_search import _pick_device
from .layout import instance_path, instances_dir

VOLUME_DTYPE = np.float32
MASK_DTYPE = np.uint16
HEARTBEAT_FILE = ".staging_heartbeat"
HEARTBEAT_PERIOD_S = 300.0


class StagingHeartbeat:
    """Touches ``<dir>/.staging_heartbeat`` at most every five minutes."""

    def __init__(self, directory):
        self.path = Path(directory) / HEARTBEAT_FILE
        self._last = 0.0

    def beat(self, force: bool = False) -> None:
        now = time.time()
        if force or now - self._last >= HEARTBEAT_PERIOD_S:
            try:
                self.path.parent.mkdir(parents=True, exist_ok=True)
                with open(self.path, "w") as f:
                    f.write(f"{now:.0f}\n")
                self._last = now
            except OSError:
                pass


def build_volume_contents(config, log=None) -> np.ndarray:
    """Rank-0 decision: which (category, instance) pairs go into which volume."""
    k = int(config.n_fracts_per_vol)
    used = int(config.n_instances_used_per_fractal)
    if used % k != 0:
        if log is not None:
            log.warning("n_instances_used_per_fractal (%s) is not a multiple of n_fracts_per_vol=%s. Rounding down.",
                        used, k)
        used = used // k * k
        config.n_instances_used_per_fractal = used
    random.seed(config.dataset_seed)
    np.random.seed(config.dataset_seed)
    pairs: List[List[int]] = []
    for cat in range(int(config.n_categories)):
        left, picks = used, []
        while left > 0:
            take = min(145, left)
            picks.extend(random.sample(range(145), take))
            left -= take
        pairs.extend([cat, inst] for inst in picks)
    arr = np.array(pairs, dtype=int)
    np.random.shuffle(arr)
    n_vol = arr.shape[0] // k
    contents = arr[: n_vol * k].reshape(n_vol, 2 * k)
    return np.hstack([np.arange(n_vol).reshape(-1, 1), contents])


def validation_indices(num_volumes: int, config) -> set:
    random.seed(config.dataset_seed)
    return set(random.sample(range(num_volumes), int(num_volumes * config.val_split / 100)))


def category_colors(config) -> np.ndarray:
    np.random.seed(config.dataset_seed)
    return np.random.rand(int(config.n_categories), 3)


def load_point_cloud(path) -> np.ndarray:
    if not os.path.exists(path):
        raise FileNotFoundError(f"File {path} does not exist. Ensure you have run 'scaffold generate_fractals ...'")
    return np.load(path)


def render_volume_shard(clouds: Sequence[np.ndarray], cats: Sequence[int], colors: np.ndarray, grid: int,
                        num_shards, shard_dims, shard_id: int, device: str) -> Tuple[np.ndarray, np.ndarray]:
    """One physical shard: (volume float32 (3,d,h,w), mask uint16 (d,h,w))."""
    sl = spatial_slices((grid, grid, grid), num_shards, shard_dims, shard_id)
    lo = [s.start for s in sl]
    shape = [s.stop - s.start for s in sl]
    if device == "cuda":
        return ifs.render_shard_cuda(clouds, [colors[c] for c in cats], [c + 1 for c in cats], grid, lo, shape)
    volume = np.zeros((3, *shape), dtype=VOLUME_DTYPE)
    mask = np.zeros(tuple(shape), dtype=MASK_DTYPE)
    for pts, c in zip(clouds, cats):
        occ = ifs.voxelize_cpu(pts, grid)[sl[0], sl[1], sl[2]].astype(bool)
        volume[:, occ] = colors[c].astype(VOLUME_DTYPE)[:, None]
        mask[occ] = c + 1
    return volume, mask


def _write_npy(path: Path, arr: np.ndarray) -> None:
    with open(path, "wb") as f:
        np.save(f, arr)


def main(config, log=None, device: Optional[str] = None) -> int:
    """Collective. Writes the dataset below ``config.dataset_dir``; returns the number of volumes."""
    rank, world = D.get_world_rank(), D.get_world_size()
    root = Path(config.dataset_dir)
    device = device or _pick_device(config)
    grid = int(config.vol_size)
    # shard ids on disk are row-major over the dims in sorted order, whatever order the config lists them in
    num_shards, shard_dims = (list(v) for v in canonical_sharding(config.dc_num_shards, config.dc_shard_dims))
    n_shards = total_shards(num_shards)
    k = int(config.n_fracts_per_vol)

    def prepare():
        for sub in ("training", "validation"):
            (root / "volumes" / sub).mkdir(parents=True, exist_ok=True)
            (root / "masks" / sub).mkdir(parents=True, exist_ok=True)
        contents = build_volume_contents(config, log)
        with open(root / "volumes_contents.csv", "wb") as f:
            np.savetxt(f, contents.astype(int), fmt="%i", delimiter=",")
        return contents

    contents = D.run_on_root(prepare)
    D.barrier()
    n_vol = len(contents)
    val_idx = validation_indices(n_vol, config)
    colors = category_colors(config)
    idir = instances_dir(config.fract_base_dir, config.variance_threshold, config.dataset_seed, config.point_num)
    total = n_vol * n_shards
    stride = ceil(total / world) if total else 0
    start, end = rank * stride, min((rank + 1) * stride, total)
    beat = StagingHeartbeat(root)
    beat.beat(force=True)
    err = None
    cached: Tuple[int, Optional[list], Optional[list]] = (-1, None, None)
    try:
        for task in range(start, end):
            vol, shard = divmod(task, n_shards)
            beat.beat()
            if cached[0] != vol:
                row = contents[vol]
                cats = [int(row[1 + 2 * j]) for j in range(k)]
                clouds = [load_point_cloud(instance_path(idir, cats[j], int(row[2 + 2 * j]))) for j in range(k)]
                cached = (vol, cats, clouds)
            _, cats, clouds = cached
            volume, mask = render_volume_shard(clouds, cats, colors, grid, num_shards, shard_dims, shard, device)
            split = "validation" if vol in val_idx else "training"
            suffix = shard_file_suffix(shard)
            _write_npy(root / "volumes" / split / f"{vol}{suffix}.npy", volume.astype(VOLUME_DTYPE, copy=False))
            _write_npy(root / "masks" / split / f"{vol}{suffix}_mask.npy", mask.astype(MASK_DTYPE, copy=False))
    except KeyboardInterrupt:
        raise
    except Exception as exc:
        err = f"{type(exc).__name__}: {exc}"
    D.consensus(err is None, err or "")

    def finish():
        cats_of = lambda rows: sorted({0} | {int(c) + 1 for r in rows for c in r[1::2]})  # noqa: E731
        train_rows = [contents[i] for i in range(n_vol) if i not in val_idx]
        val_rows = [contents[i] for i in range(n_vol) if i in val_idx]
        with open(root / "train_unique_mask_vals", "wb") as out:
            pickle.dump({"mask_values": cats_of(train_rows)}, out)
        with open(root / "val_unique_mask_vals", "wb") as out:
            pickle.dump({"mask_values": cats_of(val_rows)}, out)
        return n_vol

    n = D.run_on_root(finish)
    D.barrier()
    return n
