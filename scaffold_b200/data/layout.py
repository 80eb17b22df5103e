"""Directory layout of the fractal library (ScaFFold/datagen/layout.py:47-103).

    <fract_base_dir>/var<threshold>/seed<seed>/3DIFS_param/NNNNNN.csv
    <fract_base_dir>/var<threshold>/seed<seed>/instances/np<point_num>/<cat>/<cat>_<inst>.npy
"""
from __future__ import annotations

from pathlib import Path


def _fmt_threshold(v: float) -> str:
    return f"{float(v):g}"


def library_root(fract_base_dir, variance_threshold: float, dataset_seed: int) -> Path:
    return Path(fract_base_dir) / f"var{_fmt_threshold(variance_threshold)}" / f"seed{int(dataset_seed)}"


def params_dir(fract_base_dir, variance_threshold: float, dataset_seed: int) -> Path:
    return library_root(fract_base_dir, variance_threshold, dataset_seed) / "3DIFS_param"


def instances_dir(fract_base_dir, variance_threshold: float, dataset_seed: int, point_num: int) -> Path:
    return library_root(fract_base_dir, variance_threshold, dataset_seed) / "instances" / f"np{int(point_num)}"


def category_name(index: int) -> str:
    return f"{int(index):06d}"


def instance_path(inst_dir: Path, category: int, instance: int) -> Path:
    c = category_name(category)
    return Path(inst_dir) / c / f"{c}_{int(instance):04d}.npy"


def warn_if_legacy_layout(fract_base_dir, log=None) -> None:
    """Older trees kept ``3DIFS_param`` directly below the base dir; they are not reused."""
    legacy = Path(fract_base_dir) / "3DIFS_param"
    if legacy.exists() and log is not None:
        log.warning("legacy fractal layout found at %s; it is ignored (libraries now live under var*/seed*/)", legacy)
