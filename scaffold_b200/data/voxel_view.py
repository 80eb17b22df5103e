"""Headless look at a generated volume: orthogonal projections of the colour volume and its label mask.

``python -m scaffold_b200.data.voxel_view <volume.npy> [<mask.npy>] [-o out.ppm]`` writes one image with
three maximum-intensity projections (along D, H and W) of the ``(3, d, h, w)`` float volume and, when a mask
is given, the same three views of the class labels in a fixed palette. The image is a binary PPM written
with numpy alone, so it works on machines without a display or a plotting library; with matplotlib
installed, ``--png`` writes a PNG through the Agg backend instead.

Role of the reference's development viewer (ScaFFold/datagen/data_visualizer.py:21-59), which opens an
interactive 3-D scatter window; no window is opened here.
"""
from __future__ import annotations

import argparse
from pathlib import Path
from typing import Optional

import numpy as np

_PALETTE = np.array([[0, 0, 0], [230, 25, 75], [60, 180, 75], [255, 225, 25], [0, 130, 200], [245, 130, 48],
                     [145, 30, 180], [70, 240, 240], [240, 50, 230], [210, 245, 60], [250, 190, 212], [0, 128, 128],
                     [220, 190, 255], [170, 110, 40], [255, 250, 200], [128, 0, 0], [170, 255, 195]], dtype=np.uint8)


def projections(volume: np.ndarray, mask: Optional[np.ndarray] = None) -> np.ndarray:
    """uint8 image ``[rows, cols, 3]``: top row the volume's projections, bottom row (optional) the mask's."""
    vol = np.asarray(volume, dtype=np.float32)
    if vol.ndim == 3:
        vol = np.repeat(vol[None], 3, 0)
    if vol.ndim != 4 or vol.shape[0] != 3:
        raise ValueError(f"expected a (3, d, h, w) or (d, h, w) volume, got {vol.shape}")
    hi = float(vol.max()) or 1.0
    rows = []
    views = [np.moveaxis(vol.max(axis=a + 1), 0, -1) for a in range(3)]  # (h,w,3), (d,w,3), (d,h,3)
    size = max(max(v.shape[:2]) for v in views)

    def pad(img):
        out = np.zeros((size, size, 3), dtype=np.uint8)
        out[:img.shape[0], :img.shape[1]] = img
        return out
    rows.append(np.concatenate([pad((np.clip(v / hi, 0, 1) * 255).astype(np.uint8)) for v in views], axis=1))
    if mask is not None:
        m = np.asarray(mask).astype(np.int64)
        if m.shape != vol.shape[1:]:
            raise ValueError(f"mask shape {m.shape} does not match the volume's {vol.shape[1:]}")
        rows.append(np.concatenate([pad(_PALETTE[m.max(axis=a) % len(_PALETTE)]) for a in range(3)], axis=1))
    return np.concatenate(rows, axis=0)


def write_ppm(path, image: np.ndarray) -> Path:
    path = Path(path)
    h, w, _ = image.shape
    with open(path, "wb") as f:
        f.write(f"P6\n{w} {h}\n255\n".encode())
        f.write(np.ascontiguousarray(image, dtype=np.uint8).tobytes())
    return path


def save_view(volume_path, mask_path=None, out=None, png: bool = False) -> Path:
    vol = np.load(volume_path)
    mask = np.load(mask_path) if mask_path else None
    if mask is not None and mask.dtype == np.int16:
        mask = mask.view(np.uint16)
    img = projections(vol, mask)
    out = Path(out) if out else Path(volume_path).with_suffix(".png" if png else ".ppm")
    if png:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
        plt.imsave(out, img)
        return out
    return write_ppm(out, img)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("volume")
    ap.add_argument("mask", nargs="?")
    ap.add_argument("-o", "--out")
    ap.add_argument("--png", action="store_true", help="write a PNG through matplotlib's Agg backend")
    a = ap.parse_args(argv)
    print(save_view(a.volume, a.mask, a.out, a.png))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
