"""Shapes whose element offsets pass 2^31: the cost model flags them, the index arithmetic the kernels use
(64-bit voxel offsets, 32-bit per-axis TMA coordinates) holds them, and the partition helpers stay exact."""
import numpy as np
import pytest

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


def _pair_jobs(n, d, h, w, cout_pad, bn, td):
    """Python restatement of the pair kernel's job decode (csrc/conv_plane2.cu:decode_job2): which
    (sample, depth group, h tile, w tile, channel tile) CTA `rank` of pair-job `pj` works on."""
    tiles_h, tiles_w, groups_d = -(-h // 8), -(-w // 16), -(-d // td)
    tiles_co = cout_pad // bn
    tiles = n * groups_d * tiles_h * tiles_w
    num_pair_jobs = ((tiles + 1) // 2) * tiles_co
    for pj in range(num_pair_jobs):
        co = pj % tiles_co
        for rank in (0, 1):
            t = (pj // tiles_co) * 2 + rank
            wt = t % tiles_w; t //= tiles_w
            ht = t % tiles_h; t //= tiles_h
            dg = t % groups_d; t //= groups_d
            yield pj, rank, (t, dg, ht, wt, co)


@pytest.mark.parametrize("shape", [(2, 64, 64, 64, 128, 128, 4), (1, 5, 16, 16, 256, 256, 2), (1, 3, 8, 16, 128, 128, 2),
                                   (3, 7, 24, 40, 512, 256, 1), (1, 1, 8, 32, 384, 128, 1)])
def test_pair_kernel_jobs_cover_every_tile_once_and_statistics_slots_are_unique(shape):
    n, d, h, w, cout_pad, bn, td = shape
    tiles_h, tiles_w, groups_d = -(-h // 8), -(-w // 16), -(-d // td)
    seen, spare = set(), 0
    slots = set()
    splits = groups_d * tiles_h * tiles_w * 4
    for pj, rank, (smp, dg, ht, wt, co) in _pair_jobs(n, d, h, w, cout_pad, bn, td):
        if smp >= n:                      # the odd tile out: its loads read the fill value, its stores are masked
            spare += 1
            assert rank == 1 and smp == n and (dg, ht, wt) == (0, 0, 0)
            continue
        key = (smp, dg, ht, wt, co)
        assert key not in seen
        seen.add(key)
        for q in range(4):                # one GroupNorm partial per epilogue warp of the tile
            sj = ((dg * tiles_h + ht) * tiles_w + wt) * 4 + q
            assert 0 <= sj < splits
            slots.add((smp, sj, co))
    tiles = n * groups_d * tiles_h * tiles_w
    assert len(seen) == tiles * (cout_pad // bn)
    assert spare == (tiles % 2) * (cout_pad // bn)
    assert len(slots) == len(seen) * 4    # no two (tile, warp) pairs share a slot of a channel tile
    # the widest offsets stay inside 64-bit voxel arithmetic and the 32-bit tile counters
    assert tiles * (cout_pad // bn) < 2 ** 31
