"""Host-side checks of the two-SM pair kernel's tile selection (csrc/conv_plane2.cu:p2_choose): no GPU needed.

The expected (tile width, job depth) pairs are the ones that measured fastest on B200 for the layers of the
scale-7 U-Net; the cost model has to keep reproducing them.
"""
import ctypes as C

import pytest

from scaffold_b200.ops import _lib

try:
    LIB = _lib.lib()
except Exception as e:  # the shared library is built by __graft_entry__.build()
    pytest.skip(f"native library not built: {e}", allow_module_level=True)


def plan(n, d, h, w, cin, cout_pad, clusters=74, src1=0, ksize=3, with_std=True):
    a = _lib.SbConvArgs()
    a.N, a.D, a.H, a.W = n, d, h, w
    a.ksize = ksize
    a.src_c[0], a.src_c[1] = cin, src1
    a.cout_pad = cout_pad
    a.wpack = 1 if with_std else None  # eligibility only asks whether tap-ordered weights were given
    bn, td = C.c_int(0), C.c_int(0)
    rc = LIB.sb_conv_pair_plan(C.byref(a), clusters, C.byref(bn), C.byref(td))
    return None if rc != 0 else (bn.value, td.value)


@pytest.mark.parametrize("shape,want", [
    ((2, 64, 64, 64, 128, 128), (128, 4)),   # 128->128 @64^3: deep jobs, 7 waves
    ((2, 64, 64, 64, 64, 128), (128, 2)),    # one channel block: double-buffered accumulators hide the epilogue
    ((2, 32, 32, 32, 256, 128), (128, 4)),   # backward-data of 128->256 @32^3: 64 jobs, still the deep tile
    ((2, 32, 32, 32, 256, 256), (256, 1)),   # depth 1 and 2 measured equal; depth 1 double-buffers the accumulators
    ((2, 16, 16, 16, 512, 512), (256, 1)),   # small volume: one plane per job fills more SM pairs
    ((2, 16, 16, 16, 512, 256), (128, 1)),   # backward-data of 256->512 @16^3: 32 wide jobs would idle half the GPU
    ((2, 128, 128, 128, 64, 128), (128, 2)),  # backward-data of 128->64 @128^3
])
def test_pair_plan_reproduces_the_measured_choices(shape, want):
    assert plan(*shape) == want


def test_pair_plan_eligibility():
    assert plan(2, 8, 8, 8, 512, 1024) is None            # planes of 8 x 8: the small-plane kernel's shapes
    assert plan(2, 64, 64, 64, 64, 64) is None            # narrow outputs stay on the kd-fused kernel
    assert plan(2, 64, 64, 64, 32, 128) is None           # sources in multiples of 64 channels only
    assert plan(2, 64, 64, 64, 64, 192) is None           # 192 = 128 + 64
    assert plan(1, 1, 8, 16, 64, 128) is None             # one tile: nothing to pair
    assert plan(2, 64, 64, 64, 64, 128, with_std=False) is None
    assert plan(2, 64, 64, 64, 64, 128, ksize=1) is None
    assert plan(2, 64, 64, 64, 64, 128, src1=64) == (128, 4)  # two concatenated sources


def test_pair_plan_depth_never_exceeds_the_volume_or_tmem():
    for d in (1, 2, 3, 5, 64):
        for cout in (128, 256, 384, 512):
            got = plan(1, d, 32, 32, 128, cout)
            assert got is not None
            bn, td = got
            assert td * bn <= 512 and (td <= d or td == 1) and cout % bn == 0


@pytest.mark.parametrize("bn,cg", [(128, 16), (128, 32), (128, 64), (128, 128), (256, 16), (256, 32), (256, 64),
                                   (256, 128), (256, 256)])
def test_statistics_epilogue_maps_every_16_channel_half_to_its_group(bn, cg):
    """Python restatement of the epilogue's group arithmetic (csrc/conv_plane2.cu): the job's BN columns arrive as
    chunks of 32 split in halves of 16; half (chunk, g) belongs to local group (chunk * 32 + g * 16) // cg. Every
    column must land in the group that holds its channel, and the groups of a tile must be <= 16."""
    groups_here = bn // cg
    assert 1 <= groups_here <= 16 and cg % 16 == 0
    cols_per_group = [0] * groups_here
    for chunk in range(bn // 32):
        for g in range(2):
            gl = (chunk * 32 + g * 16) // cg
            first, last = chunk * 32 + g * 16, chunk * 32 + g * 16 + 15
            assert first // cg == gl == last // cg          # a half never straddles two groups
            cols_per_group[gl] += 16
    assert cols_per_group == [cg] * groups_here
    # global group index of local group l in the channel tile that starts at co0: co0 // cg + l
    for co0 in (0, bn, 3 * bn):
        assert [(co0 + l * cg) // cg for l in range(groups_here)] == [co0 // cg + l for l in range(groups_here)]
