"""Shapes whose element offsets pass 2^31: the cost model flags them, the index arithmetic the kernels use
(64-bit voxel offsets, 32-bit per-axis TMA coordinates) holds them, and the partition helpers stay exact."""
import numpy as np

from scaffold_b200.analysis.shapes import ConvProblem, edge_cases
from scaffold_b200.utils.sharding import chunk_slice, spatial_slices


def test_scale_nine_stem_level_is_flagged_and_fits_the_index_types():
    p = ConvProblem(2, 64, 64, (256, 256, 256))
    assert p.max_elements == 2 * 256 ** 3 * 64 == 2 ** 31 and p.index_exceeds_int32
    big = [c for c in edge_cases(include_large=True) if c.index_exceeds_int32]
    assert big and big[0].spatial == (512, 512, 512)
    # what a kernel computes: voxel index (64-bit) * channels + channel; the last element's offset
    n, d, h, w, c = 2, 256, 256, 256, 64
    vox = (np.int64((n - 1) * d + d - 1) * np.int64(h) + np.int64(h - 1)) * np.int64(w) + np.int64(w - 1)
    off = vox * np.int64(c) + np.int64(c - 1)
    assert int(off) == n * d * h * w * c - 1 == 2 ** 31 - 1
    off = off + np.int64(c)                           # one voxel further (batch 3, or 128 channels): beyond int32
    assert int(off) > 2 ** 31 - 1
    assert int(np.int64(off) * 2) < 2 ** 40          # byte offsets: far inside the 64-bit range TMA strides use
    # per-axis TMA coordinates and extents stay 32-bit: the largest is the voxel count of one axis
    assert max(n, d, h, w, c) < 2 ** 31
    # a 32-bit voxel*channel product would have wrapped: the hazard the 64-bit arithmetic avoids
    wide = np.int64(vox + 1) * np.int64(c)
    assert int(wide) == 2 ** 31 and int(np.array(wide).astype(np.int32)) != int(wide)


def test_partition_helpers_are_exact_on_large_extents():
    s = chunk_slice(2 ** 20 + 3, 8, 7)
    assert s.stop == 2 ** 20 + 3 and s.start == 7 * ((2 ** 20 + 3 + 7) // 8)
    sl = spatial_slices((512, 512, 512), (2, 2, 2), (2, 3, 4), 5)
    assert [v.stop - v.start for v in sl] == [256, 256, 256]
    cover = set()
    for sid in range(8):
        cover.add(tuple((v.start, v.stop) for v in spatial_slices((512, 512, 512), (2, 2, 2), (2, 3, 4), sid)))
    assert len(cover) == 8
