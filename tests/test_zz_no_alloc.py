"""GPU test of the allocation-free GroupNorm entry point (collected last on purpose).

Some users of the library cannot allocate device memory at the moment they need
a GroupNorm: code inside a stream capture, or a host application that fixed its
memory budget at start-up. ``sb_gn_forward_noalloc`` keeps its scratch inside
the library; this test calls it through its exported C symbol, twice in a row
(the scratch array is shared and keeps the previous call's contents), and
compares with the ordinary entry points, which take caller-allocated scratch.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, x, y, w, b, mean, rstd, G, relu):
    n, d, h, wd, c = x.shape
    fn = lib.sb_gn_forward_noalloc
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_longlong,
                   C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p]
    fn.restype = C.c_int
    return fn(x.data_ptr(), y.data_ptr(), w.data_ptr(), b.data_ptr(), mean.data_ptr() if mean is not None else None,
              rstd.data_ptr() if rstd is not None else None, n,
              d * h * wd, c, G, 1e-5, 1 if relu else 0, torch.cuda.current_stream().cuda_stream)


def test_noalloc_groupnorm_matches_the_allocating_entry_points_twice():
    from scaffold_b200.ops import _lib, gn_kernels as gk
    lib = _lib.lib()
    g = torch.Generator(device="cuda").manual_seed(0)
    for shape, G, relu in (((2, 8, 16, 16, 64), 8, True), ((1, 4, 8, 8, 128), 8, False)):
        x = (torch.randn(shape, generator=g, device="cuda") * 2 + 1).to(torch.bfloat16)
        w = torch.randn(shape[4], generator=g, device="cuda")
        b = torch.randn(shape[4], generator=g, device="cuda")
        want, wmean, wrstd = gk.gn_forward(x, w, b, G, 1e-5, relu)
        y = torch.empty_like(x)
        mean = torch.empty((shape[0], G), device="cuda")
        rstd = torch.empty((shape[0], G), device="cuda")
        # one warm call first: the first call on a device resolves the scratch array's address (and the
        # driver may load the kernels lazily), which is allowed to change the free-memory figure
        assert _call(lib, x, y, w, b, mean, rstd, G, relu) == 0
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]  # the driver's own figure: sees a cudaMalloc inside the library too
        for _ in range(2):  # second call reuses scratch that still holds the first call's partials
            y.fill_(float("nan"))
            assert _call(lib, x, y, w, b, mean, rstd, G, relu) == 0
            torch.cuda.synchronize()
            assert torch.cuda.memory_allocated() == before
            assert torch.cuda.mem_get_info()[0] == free_before
            assert torch.equal(y, want)
            assert torch.allclose(mean, wmean, rtol=1e-6, atol=1e-7) and torch.allclose(rstd, wrstd, rtol=1e-6)
        # the caller may pass no mean / rstd outputs: the statistics then stay inside the library's array
        y.fill_(float("nan"))
        assert _call(lib, x, y, w, b, None, None, G, relu) == 0
        torch.cuda.synchronize()
        assert torch.equal(y, want)


def test_noalloc_groupnorm_rejects_oversized_requests():
    from scaffold_b200.ops import _lib
    lib = _lib.lib()
    # 64 samples x 10 splits x 256 groups x 3 floats of partials do not fit the fixed array
    x = torch.zeros((64, 2, 2, 4, 2048), dtype=torch.bfloat16, device="cuda")
    y = torch.empty_like(x)
    w = torch.ones(2048, device="cuda")
    b = torch.zeros(2048, device="cuda")
    mean = torch.empty((64, 256), device="cuda")
    rc = _call(lib, x, y, w, b, mean, mean.clone(), 256, True)
    assert rc == 6  # SB_ERR_TOO_LARGE: refused before any launch


def test_noalloc_groupnorm_rejects_unsupported_channel_counts_without_a_launch():
    from scaffold_b200.ops import _lib
    lib = _lib.lib()
    for c, G in ((4, 1), (4096, 8), (64, 7), (8, 8)):
        x = torch.zeros((1, 2, 2, 2, c), dtype=torch.bfloat16, device="cuda")
        y = torch.full_like(x, 3.0)
        w = torch.ones(c, device="cuda")
        b = torch.zeros(c, device="cuda")
        st = torch.empty((1, max(G, 1)), device="cuda")
        assert _call(lib, x, y, w, b, st, st.clone(), G, True) == 4  # SB_ERR_SHAPE
        torch.cuda.synchronize()
        assert bool((y == 3.0).all())  # nothing ran
