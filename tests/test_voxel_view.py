"""Headless volume viewer: projections and the PPM writer."""
import numpy as np

from scaffold_b200.data import voxel_view as vv


def test_projections_show_volume_and_mask(tmp_path):
    vol = np.zeros((3, 4, 6, 8), dtype=np.float32)
    vol[0, 1, 2, 3] = 2.0
    mask = np.zeros((4, 6, 8), dtype=np.uint16)
    mask[1, 2, 3] = 2
    img = vv.projections(vol, mask)
    assert img.shape == (16, 24, 3) and img.dtype == np.uint8
    assert img[2, 3, 0] == 255 and img[2, 3, 1] == 0            # projection along D: (h, w) = (2, 3), red channel
    assert tuple(img[8 + 2, 3]) == tuple(vv._PALETTE[2])         # the mask row uses the class palette
    np.save(tmp_path / "v.npy", vol)
    np.save(tmp_path / "m.npy", mask.view(np.int16))
    out = vv.save_view(tmp_path / "v.npy", tmp_path / "m.npy")
    data = out.read_bytes()
    assert data.startswith(b"P6\n24 16\n255\n") and len(data) == len(b"P6\n24 16\n255\n") + 16 * 24 * 3
