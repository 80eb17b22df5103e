"""Host-side argument validation of the native entry points: runs without a GPU.

The checks under test return before any CUDA call, so the library only has to load
(it links the CUDA runtime, which the toolkit provides on a CPU-only machine).
"""
import ctypes as C

import pytest

from scaffold_b200.ops import _lib


def _lib_or_skip():
    if not _lib.available():
        pytest.skip("native library not built")
    try:
        return _lib.lib()
    except OSError as exc:  # CUDA runtime not installed on this machine
        pytest.skip(f"native library does not load here: {exc}")


def test_gn_nsplit_never_divides_by_zero():
    L = _lib_or_skip()
    L.sb_gn_nsplit.argtypes = [C.c_int, C.c_longlong, C.c_int]
    L.sb_gn_nsplit.restype = C.c_int
    for c in (0, 1, 4, 7, 2056, 4096, 1 << 20):
        assert L.sb_gn_nsplit(2, 4096, c) == 1
    assert L.sb_gn_nsplit(2, 0, 64) == 1
    assert L.sb_gn_nsplit(0, 4096, 64) == 1
    assert L.sb_gn_nsplit(2, 128 ** 3, 64) > 1


def test_gn_supported_matches_the_documented_limits():
    L = _lib_or_skip()
    L.sb_gn_supported.argtypes = [C.c_int, C.c_int]
    L.sb_gn_supported.restype = C.c_int
    assert L.sb_gn_supported(64, 8) == 1
    assert L.sb_gn_supported(2048, 8) == 1
    assert L.sb_gn_supported(16, 8) == 1      # two channels per group: four groups share an octet
    assert L.sb_gn_supported(4096, 8) == 0    # wider than one thread per channel octet allows
    assert L.sb_gn_supported(4, 1) == 0
    assert L.sb_gn_supported(8, 8) == 0       # one channel per group: eight groups in an octet
    assert L.sb_gn_supported(64, 7) == 0


def test_noalloc_groupnorm_refuses_bad_shapes_on_the_host():
    L = _lib_or_skip()
    fn = L.sb_gn_forward_noalloc
    fn.argtypes = [C.c_void_p] * 6 + [C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p]
    fn.restype = C.c_int
    fake = 0x1000  # never dereferenced: every case below is refused before a launch
    for n, s, c, g in ((1, 64, 4, 1), (1, 64, 4096, 8), (1, 0, 64, 8), (0, 64, 64, 8), (1, 64, 64, 0), (65, 64, 64, 8)):
        assert fn(fake, fake, fake, fake, None, None, n, s, c, g, 1e-5, 1, None) == 4, (n, s, c, g)
    assert fn(None, fake, fake, fake, None, None, 1, 64, 64, 8, 1e-5, 1, None) == 4
