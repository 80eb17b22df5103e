"""Instance generation: 145 weighted variants of every fractal category.

Instance ``i`` of a category scales the 12 IFS coefficients (matrix + translation)
of both maps by row ``i`` of the instance weight table; the cloud has
``point_num`` float32 points and is written atomically to
``instances/np<P>/<cat>/<cat>_<inst>.npy``. A weight row that makes the orbit
diverge is attenuated towards 1 (factors 0.5, 0.25, 0.1) and finally dropped to
the unweighted parameters, so every slot fills deterministically. Rank 0 builds
the work list (existing, loadable files are skipped) and broadcasts it; ranks
take contiguous blocks. (ScaFFold/datagen/instance.py:63-408.)

All orbits of a rank's block run as one batch (one GPU thread each).
"""
from __future__ import annotations

import os
import tempfile
from pathlib import Path
from typing import List, Optional, Tuple

import numpy as np

from ..utils import dist as D
from . import ifs
from .category_search import _pick_device, existing_categories
from .layout import instance_path, instances_dir, params_dir
from .rng import derive_seed

N_INSTANCES = 145
ATTENUATION = (0.5, 0.25, 0.1)


def instance_weights() -> np.ndarray:
    """The 145 x 12 weight table: coefficient ``c`` swept over 0.4 .. 1.6 in steps of 0.1.

    Row 6 is the all-ones (unweighted) instance; the value 1.0 appears only in
    the first sweep. The last row of the sweep of coefficient 8 carries 0.6
    instead of 1.6, as in the published table
    (ScaFFold/package_data/weights_ins145.csv); it is kept so that instance
    numbering and content stay compatible.
    """
    rows = []
    sweep = [round(0.4 + 0.1 * i, 1) for i in range(13)]
    for c in range(12):
        for v in sweep:
            if v == 1.0 and c > 0:
                continue
            r = np.ones(12)
            r[c] = v
            rows.append(r)
    table = np.array(rows)
    table[108, 8] = 0.6
    return table


def item_seed(seed: int, category: int, instance: int) -> int:
    return (derive_seed(seed, category, instance, 1) << 32) | derive_seed(seed, category, instance)


def _valid_file(path: Path, point_num: int) -> bool:
    try:
        arr = np.load(path, mmap_mode="r")
        return arr.shape == (point_num, 3) and arr.dtype == np.float32
    except Exception:
        return False


def _atomic_save(path: Path, arr: np.ndarray) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=str(path.parent), prefix=".tmp_", suffix=".npy")
    try:
        with os.fdopen(fd, "wb") as f:
            np.save(f, arr)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
    finally:
        if os.path.exists(tmp):
            os.unlink(tmp)


def generate_batch(base_params: List[np.ndarray], items: List[Tuple[int, int]], point_num: int, seed: int,
                   weights: np.ndarray, device: str) -> List[np.ndarray]:
    """Point clouds for ``items`` [(category, instance)], with the attenuation ladder for diverging ones."""
    n = len(items)
    out: List[Optional[np.ndarray]] = [None] * n
    todo = list(range(n))
    ladder = [1.0, *ATTENUATION, 0.0]  # 0.0 == unweighted parameters
    for factor in ladder:
        if not todo:
            break
        params = []
        for k in todo:
            cat, inst = items[k]
            p = np.array(base_params[cat], dtype=np.float64, copy=True)
            p[:, :12] *= 1.0 + (weights[inst % len(weights)] - 1.0) * factor
            params.append(p)
        seeds = np.array([item_seed(seed, *items[k]) for k in todo], dtype=np.uint64)
        pts, flags = ifs.orbit_points(np.stack(params), seeds, point_num, device=device)
        still = []
        for j, k in enumerate(todo):
            if flags[j] == 0 and np.isfinite(pts[j]).all():
                out[k] = pts[j]
            else:
                still.append(k)
        todo = still
    if todo:
        cat, inst = items[todo[0]]
        raise ValueError(f"Unweighted parameters for category {cat} produced a non-finite point cloud (instance {inst})")
    return out  # type: ignore[return-value]


def main(config, log=None, device: Optional[str] = None) -> int:
    """Collective over all ranks. Returns the number of instance files written by this rank."""
    rank, world = D.get_world_rank(), D.get_world_size()
    pdir = params_dir(config.fract_base_dir, config.variance_threshold, config.dataset_seed)
    idir = instances_dir(config.fract_base_dir, config.variance_threshold, config.dataset_seed, config.point_num)
    device = device or _pick_device(config)
    n_cat, point_num = int(config.n_categories), int(config.point_num)

    def build_work():
        cats = existing_categories(pdir)
        missing = [c for c in range(n_cat) if c not in cats]
        if missing:
            raise FileNotFoundError(f"IFS parameters missing for categories {missing[:8]} under {pdir}; run the "
                                    "category search first")
        work = [(c, i) for c in range(n_cat) for i in range(N_INSTANCES)
                if getattr(config, "datagen_from_scratch", False) or not _valid_file(instance_path(idir, c, i), point_num)]
        return [cats[c] for c in range(n_cat)], work

    base_params, work = D.run_on_root(build_work)
    per = -(-len(work) // world) if work else 0
    mine = work[rank * per:(rank + 1) * per]
    err, written = None, 0
    try:
        weights = instance_weights()
        chunk = 512
        for o in range(0, len(mine), chunk):
            items = mine[o:o + chunk]
            clouds = generate_batch(base_params, items, point_num, int(config.dataset_seed), weights, device)
            for (c, i), pts in zip(items, clouds):
                _atomic_save(instance_path(idir, c, i), np.ascontiguousarray(pts, dtype=np.float32))
                written += 1
    except Exception as exc:
        err = f"{type(exc).__name__}: {exc}"
    D.consensus(err is None, err or "")
    if log is not None:
        log.info("instances: %d files written by rank %d (%d work items in total)", written, rank, len(work))
    D.barrier()
    return written
