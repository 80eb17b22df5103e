"""Stand-alone tool: scan mask files for their unique label values and pickle the result.

``python -m scaffold_b200.data.mask_scan <masks_dir> <out_file> [--workers N]``
(ScaFFold/datagen/mask_detection.py:27-108).
"""
from __future__ import annotations

import argparse
import pickle
import multiprocessing
from pathlib import Path
from typing import List

import numpy as np


def unique_values(path: str) -> List[int]:
    return [int(v) for v in np.unique(np.load(path, mmap_mode="r"))]


def scan(masks_dir, workers: int = 4) -> List[int]:
    files = sorted(str(p) for p in Path(masks_dir).glob("*.npy"))
    if not files:
        raise FileNotFoundError(f"no .npy masks under {masks_dir}")
    if workers > 1:
        # "spawn": the caller may be multi-threaded (a fork of such a process can deadlock in the child)
        with multiprocessing.get_context("spawn").Pool(workers) as pool:
            parts = pool.map(unique_values, files)
    else:
        parts = [unique_values(f) for f in files]
    return sorted({v for p in parts for v in p})


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("masks_dir")
    ap.add_argument("out_file")
    ap.add_argument("--workers", type=int, default=4)
    a = ap.parse_args(argv)
    with open(a.out_file, "wb") as f:
        pickle.dump({"mask_values": scan(a.masks_dir, a.workers)}, f)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
