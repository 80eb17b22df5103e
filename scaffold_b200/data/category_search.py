"""Search for valid IFS fractal categories.

A candidate is ``uniform(-1, 1, (2, 13))`` float64 drawn from a generator keyed
by ``(dataset_seed, rank, attempt)``; column 12 is replaced by the selection
probability ``|det A_t| / sum_t |det A_t|``. It is accepted when its chaos-game
orbit is finite, does not run away and, normalised to ``[-normalize, normalize]``
per axis, has a variance above ``variance_threshold`` on every axis. Accepted
parameter blocks are written by rank 0 as ``NNNNNN.csv`` (2 rows x 13 columns),
deduplicated, filling index holes first. Each rank keeps a persistent attempt
counter (``.rng_attempt_rank<r>``) so that a resumed or extended search never
replays candidates. Rounds are sized adaptively from the observed acceptance
rate. (ScaFFold/datagen/category_search.py:42-683.)

The candidates of one round are evaluated as ONE batch: on a GPU, one thread
per candidate runs the orbit and keeps only running statistics.
"""
from __future__ import annotations

import os
import tempfile
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import numpy as np

from ..utils import dist as D
from . import ifs
from .layout import category_name, params_dir
from .rng import derive_seed

SEED_MASK = 0xFFFFFFFF


def propose_params(base_seed: int, rank: int, attempt: int) -> np.ndarray:
    ss = np.random.SeedSequence((int(base_seed) & SEED_MASK, int(rank) & SEED_MASK, int(attempt) & SEED_MASK))
    params = np.random.default_rng(ss).uniform(-1.0, 1.0, (2, 13)).astype(np.float64)
    det = np.abs(np.linalg.det(params[:, 0:9].reshape(-1, 3, 3)))
    params[:, -1] = det / det.sum()
    return params


def orbit_seed(base_seed: int, rank: int, attempt: int) -> int:
    """64-bit orbit seed: two independent 32-bit derivations."""
    return (derive_seed(base_seed, rank, attempt, 1) << 32) | derive_seed(base_seed, rank, attempt)


def evaluate_round(base_seed: int, rank: int, first_attempt: int, count: int, point_num: int, normalize: float,
                   variance_threshold: float, device: str) -> Tuple[List[np.ndarray], Dict[str, int]]:
    """Evaluate ``count`` consecutive attempts of one rank; returns accepted blocks and rejection counts."""
    if count <= 0:
        return [], {"attempts": 0, "nonfinite": 0, "variance": 0, "runaway": 0}
    params = np.stack([propose_params(base_seed, rank, first_attempt + i) for i in range(count)])
    seeds = np.array([orbit_seed(base_seed, rank, first_attempt + i) for i in range(count)], dtype=np.uint64)
    stats = ifs.orbit_stats(params, seeds, int(point_num), device=device)
    valid, reason = ifs.accept(stats, normalize, variance_threshold)
    counts = {"attempts": count, "nonfinite": int((reason == 1).sum()), "variance": int((reason == 2).sum()),
              "runaway": int((reason == 3).sum())}
    return [params[i] for i in np.nonzero(valid)[0]], counts


# -- files ---------------------------------------------------------------------
def existing_categories(pdir: Path) -> Dict[int, np.ndarray]:
    out: Dict[int, np.ndarray] = {}
    if not pdir.exists():
        return out
    for f in sorted(pdir.glob("[0-9][0-9][0-9][0-9][0-9][0-9].csv")):
        try:
            arr = np.loadtxt(f, delimiter=",", dtype=np.float64)
        except Exception:
            continue
        if arr.shape == (2, 13) and np.isfinite(arr).all():
            out[int(f.stem)] = arr
    return out


def _atomic_savetxt(path: Path, arr: np.ndarray) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=str(path.parent), prefix=".tmp_", suffix=".csv")
    try:
        with os.fdopen(fd, "w") as f:
            np.savetxt(f, arr, delimiter=",", fmt="%.17g")
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
    finally:
        if os.path.exists(tmp):
            os.unlink(tmp)


def save_new_categories(pdir: Path, found: List[np.ndarray], wanted: int) -> int:
    """Rank 0: append new unique categories until ``wanted`` exist; returns how many are still missing."""
    have = existing_categories(pdir)
    known = {arr.tobytes() for arr in have.values()}
    holes = [i for i in range(wanted) if i not in have]
    for arr in found:
        if not holes:
            break
        key = np.asarray(arr, dtype=np.float64).tobytes()
        if key in known:
            continue
        known.add(key)
        _atomic_savetxt(pdir / f"{category_name(holes.pop(0))}.csv", arr)
    return len(holes)


def _counter_path(pdir: Path, rank: int) -> Path:
    return pdir / f".rng_attempt_rank{rank}"


def load_attempt_counter(pdir: Path, rank: int) -> int:
    try:
        return int(_counter_path(pdir, rank).read_text().strip())
    except Exception:
        return 0


def store_attempt_counter(pdir: Path, rank: int, value: int) -> None:
    pdir.mkdir(parents=True, exist_ok=True)
    tmp = _counter_path(pdir, rank).with_suffix(".tmp")
    tmp.write_text(str(int(value)))
    os.replace(tmp, _counter_path(pdir, rank))


def round_size(remaining: int, attempts_so_far: int, accepted_so_far: int, batch_cap: int, world: int) -> int:
    """Attempts per rank for the next round: enough for the remainder at the observed rate, with slack."""
    if remaining <= 0:
        return 0
    rate = (accepted_so_far + 1) / (attempts_so_far + 50)  # optimistic prior, converges to the observed rate
    need = int(np.ceil(remaining / max(rate, 1e-6) * 1.25 / max(world, 1)))
    return int(max(8, min(batch_cap, need)))


def main(config, log=None, device: Optional[str] = None) -> int:
    """Collective over all ranks. Returns the number of categories available afterwards."""
    rank, world = D.get_world_rank(), D.get_world_size()
    pdir = params_dir(config.fract_base_dir, config.variance_threshold, config.dataset_seed)
    device = device or _pick_device(config)
    wanted = int(config.n_categories)
    batch_cap = int(getattr(config, "datagen_batch_size", 10000) or 10000)

    def scan():
        if getattr(config, "datagen_from_scratch", False) and pdir.exists():
            for f in pdir.glob("*.csv"):
                f.unlink()
        pdir.mkdir(parents=True, exist_ok=True)
        return wanted - len([i for i in existing_categories(pdir) if i < wanted])

    remaining = D.run_on_root(scan)
    attempt = load_attempt_counter(pdir, rank)
    total_attempts = total_accepted = 0
    rounds = 0
    while remaining > 0:
        n = D.bcast_obj(round_size(remaining, total_attempts, total_accepted, batch_cap, world))
        err = None
        found: List[np.ndarray] = []
        counts = {"attempts": 0}
        try:
            found, counts = evaluate_round(config.dataset_seed, rank, attempt, n, config.point_num,
                                           float(config.normalize), float(config.variance_threshold), device)
            attempt += n
            store_attempt_counter(pdir, rank, attempt)
        except Exception as exc:  # reported through the consensus below
            err = f"{type(exc).__name__}: {exc}"
        D.consensus(err is None, err or "")
        gathered = D.allgather_obj((found, counts["attempts"]))
        total_attempts += sum(a for _, a in gathered)
        all_found = [p for f, _ in gathered for p in f]
        total_accepted += len(all_found)
        remaining = D.run_on_root(lambda: save_new_categories(pdir, all_found, wanted))
        rounds += 1
        if log is not None:
            log.info("category search round %d: %d attempts/rank, %d accepted, %d still missing", rounds, n,
                     len(all_found), remaining)
        if rounds > 10000:
            raise RuntimeError("category search did not converge")
    D.barrier()
    return wanted


def _pick_device(config) -> str:
    choice = getattr(config, "datagen_device", "auto")
    if choice in ("cpu", "cuda"):
        return choice
    try:
        import torch
        return "cuda" if torch.cuda.is_available() else "cpu"
    except Exception:
        return "cpu"
