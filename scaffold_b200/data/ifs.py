"""IFS chaos game: Python front end of the native CPU / CUDA generators.

One candidate or instance is a ``(2, 13)`` float64 parameter block (3x3 matrix,
translation, selection probability per map). ``orbit_stats`` and ``orbit_points``
run batches either on the GPU (``csrc/ifs.cu``, one thread per orbit) or on the
CPU (``csrc/ifs_cpu.cpp``); both use the same SplitMix64 stream per orbit, so
the results agree bit for bit. A pure-numpy implementation of the same stream is
kept as the oracle of the tests (``orbit_numpy``).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import numpy as np
import torch

from ..ops import _lib

_P = C.c_void_p
_lib.register("sb_ifs_orbit_cpu", [_P, C.c_ulonglong, C.c_longlong, _P, _P], C.c_int)
_lib.register("sb_voxelize_cpu", [_P, C.c_longlong, C.c_int, _P], C.c_int)
_lib.register("sb_ifs_search", [_P, _P, C.c_int, C.c_longlong, _P, _P], C.c_int)
_lib.register("sb_ifs_points", [_P, _P, C.c_int, C.c_longlong, _P, _P, _P], C.c_int)
_lib.register("sb_voxel_bbox", [_P, C.c_int, C.c_longlong, _P, _P], C.c_int)
_lib.register("sb_voxel_paint", [_P, C.c_longlong, _P, C.c_int, _P, _P, _P, C.c_int, _P, _P, _P], C.c_int)

MASK64 = (1 << 64) - 1


def _native_ok() -> bool:
    try:
        _lib.lib()
        return True
    except Exception:
        return False


# ---------------------------------------------------------------------------
# numpy oracle of the native stream
# ---------------------------------------------------------------------------
def _splitmix(state: int) -> Tuple[int, int]:
    state = (state + 0x9E3779B97F4A7C15) & MASK64
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    return state, z ^ (z >> 31)


def orbit_numpy(params: np.ndarray, seed: int, n: int) -> Tuple[np.ndarray, bool]:
    """Reference orbit in plain Python/numpy: (points float64 [n,3], runaway_check_pass)."""
    P = np.asarray(params, dtype=np.float64).reshape(2, 13)
    pts = np.zeros((max(n, 0), 3), dtype=np.float64)
    state, ok = int(seed) & MASK64, True
    v = np.zeros(3)
    for i in range(1, n):
        state, z = _splitmix(state)
        r = (z >> 11) * (1.0 / 9007199254740992.0)
        m = P[0] if r < P[0, 12] else P[1]
        v = np.array([v[0] * m[0] + v[1] * m[1] + v[2] * m[2] + m[9],
                      v[0] * m[3] + v[1] * m[4] + v[2] * m[5] + m[10],
                      v[0] * m[6] + v[1] * m[7] + v[2] * m[8] + m[11]])
        pts[i] = v
        if np.any(np.abs(v) > 1e10):
            ok = False
    return pts, ok


# ---------------------------------------------------------------------------
# batched front ends
# ---------------------------------------------------------------------------
def orbit_stats(params: np.ndarray, seeds: np.ndarray, n: int, device: str = "cpu") -> np.ndarray:
    """Statistics of a batch of orbits: ``[B, 16]`` = min3, max3, mean3, var3, count, runaway, nonfinite, 0."""
    params = np.ascontiguousarray(params, dtype=np.float64).reshape(-1, 26)
    seeds = np.ascontiguousarray(seeds, dtype=np.uint64)
    b = params.shape[0]
    if device == "cuda":
        dp = torch.from_numpy(params).cuda()
        ds = torch.from_numpy(seeds.view(np.int64)).cuda()
        out = torch.empty((b, 16), dtype=torch.float64, device="cuda")
        _lib.check(_lib.lib().sb_ifs_search(dp.data_ptr(), ds.data_ptr(), b, n, out.data_ptr(), _lib.stream_ptr()),
                   "sb_ifs_search")
        return out.cpu().numpy()
    out = np.empty((b, 16), dtype=np.float64)
    L = _lib.lib()
    for i in range(b):
        L.sb_ifs_orbit_cpu(params[i].ctypes.data, int(seeds[i]), n, None, out[i].ctypes.data)
    return out


def orbit_points(params: np.ndarray, seeds: np.ndarray, n: int, device: str = "cpu") -> Tuple[np.ndarray, np.ndarray]:
    """Point clouds of a batch of orbits: (float32 ``[B, n, 3]``, flags ``[B]``: bit0 runaway, bit1 NaN)."""
    params = np.ascontiguousarray(params, dtype=np.float64).reshape(-1, 26)
    seeds = np.ascontiguousarray(seeds, dtype=np.uint64)
    b = params.shape[0]
    if device == "cuda":
        dp = torch.from_numpy(params).cuda()
        ds = torch.from_numpy(seeds.view(np.int64)).cuda()
        pts = torch.empty((b, n, 3), dtype=torch.float32, device="cuda")
        flags = torch.empty(b, dtype=torch.int32, device="cuda")
        _lib.check(_lib.lib().sb_ifs_points(dp.data_ptr(), ds.data_ptr(), b, n, pts.data_ptr(), flags.data_ptr(),
                                            _lib.stream_ptr()), "sb_ifs_points")
        return pts.cpu().numpy(), flags.cpu().numpy()
    pts = np.empty((b, n, 3), dtype=np.float32)
    flags = np.zeros(b, dtype=np.int32)
    stats = np.empty(16, dtype=np.float64)
    L = _lib.lib()
    for i in range(b):
        L.sb_ifs_orbit_cpu(params[i].ctypes.data, int(seeds[i]), n, pts[i].ctypes.data, stats.ctypes.data)
        flags[i] = int(stats[13]) | (int(stats[14]) << 1)
    return pts, flags


def accept(stats: np.ndarray, normalize: float, variance_threshold: float) -> Tuple[np.ndarray, np.ndarray]:
    """Acceptance test of the category search on orbit statistics.

    A candidate passes iff the orbit is finite, did not run away, every axis has
    a positive range, and the per-axis variance of the cloud normalised to
    ``[-normalize, normalize]`` exceeds the threshold
    (ScaFFold/datagen/category_search.py:114-201). Returns (valid, reason) with
    reason 0 ok, 1 non-finite, 2 low variance, 3 runaway.
    """
    stats = np.atleast_2d(stats)
    with np.errstate(invalid="ignore", over="ignore"):
        rng = stats[:, 3:6] - stats[:, 0:3]
    finite = (stats[:, 14] == 0) & np.isfinite(rng).all(1) & (rng > 0).all(1)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        var_n = stats[:, 9:12] * ((2.0 * normalize) / rng) ** 2
    finite &= np.isfinite(var_n).all(1)
    var_ok = finite & (var_n > variance_threshold).all(1)
    runaway = stats[:, 13] != 0
    valid = var_ok & ~runaway
    reason = np.where(~finite, 1, np.where(~var_ok, 2, np.where(runaway, 3, 0)))
    return valid, reason


# ---------------------------------------------------------------------------
# voxelisation
# ---------------------------------------------------------------------------
def points_to_voxel_indices(points: np.ndarray, grid_size: int, eps: float = 1e-6) -> np.ndarray:
    """numpy oracle: unique (K, 3) voxel coordinates of a cloud (ScaFFold/datagen/volumegen.py:103-160)."""
    if not np.isfinite(points).all():
        raise ValueError("points_to_voxel_indices received non-finite coordinates (NaN or inf); "
                         "refusing to rasterize corrupt point cloud")
    pts = points.astype(np.float64)
    mins, maxs = pts.min(0), pts.max(0)
    voxel = (float((maxs - mins).max()) + eps) / grid_size
    scaled = (pts - mins) / voxel
    offset = (grid_size - (maxs - mins) / voxel) / 2.0
    idx = np.clip(np.floor(scaled + offset).astype(np.int64), 0, grid_size - 1)
    return np.unique(idx, axis=0)


def voxelize_cpu(points: np.ndarray, grid_size: int) -> np.ndarray:
    """Native CPU rasteriser: uint8 occupancy ``[G, G, G]``."""
    pts = np.ascontiguousarray(points, dtype=np.float32)
    occ = np.zeros((grid_size,) * 3, dtype=np.uint8)
    rc = _lib.lib().sb_voxelize_cpu(pts.ctypes.data, pts.shape[0], grid_size, occ.ctypes.data)
    if rc != 0:
        raise ValueError("voxelize received non-finite coordinates (NaN or inf); refusing to rasterize corrupt "
                         "point cloud")
    return occ


def render_shard_cuda(clouds, colors, labels, grid_size: int, lo, shape):
    """Paint clouds (list of float32 [n,3] arrays) into one shard on the GPU.

    Returns (volume float32 ``(3, d, h, w)``, mask uint16 ``(d, h, w)``) as numpy arrays.
    """
    L = _lib.lib()
    vol = torch.zeros((3, *shape), dtype=torch.float32, device="cuda")
    mask = torch.zeros(tuple(shape), dtype=torch.int16, device="cuda")
    lo_a = (C.c_int * 3)(*[int(v) for v in lo])
    sh_a = (C.c_int * 3)(*[int(v) for v in shape])
    for pts, rgb, label in zip(clouds, colors, labels):
        if not np.isfinite(pts).all():
            raise ValueError("non-finite coordinates (NaN or inf); refusing to rasterize corrupt point cloud")
        dp = torch.from_numpy(np.ascontiguousarray(pts, dtype=np.float32)).cuda()
        bbox = torch.empty(6, dtype=torch.float32, device="cuda")
        n = dp.shape[0]
        _lib.check(L.sb_voxel_bbox(dp.data_ptr(), 1, n, bbox.data_ptr(), _lib.stream_ptr()), "sb_voxel_bbox")
        rgb_a = (C.c_float * 3)(*[float(v) for v in rgb])
        _lib.check(L.sb_voxel_paint(dp.data_ptr(), n, bbox.data_ptr(), grid_size, lo_a, sh_a, rgb_a, int(label),
                                    vol.data_ptr(), mask.data_ptr(), _lib.stream_ptr()), "sb_voxel_paint")
    return vol.cpu().numpy(), mask.cpu().numpy().view(np.uint16)
