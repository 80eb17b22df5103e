"""Out-of-bounds writes would be silent on a GPU without a sanitizer: here every kernel writes into the
middle of a larger buffer whose margins hold a canary pattern, and the margins must come back untouched.
Odd extents (tiles hanging over the edge of the volume) are the interesting cases."""
import pytest
import torch

pytestmark = pytest.mark.gpu

CANARY = -1234.0
MARGIN = 4096  # elements on either side


def _guarded(shape, dtype):
    n = 1
    for s in shape:
        n *= s
    buf = torch.full((n + 2 * MARGIN,), CANARY, dtype=dtype, device="cuda")
    return buf, buf[MARGIN:MARGIN + n].view(shape)


def _intact(buf, n):
    return bool((buf[:MARGIN] == CANARY).all()) and bool((buf[MARGIN + n:] == CANARY).all())


@pytest.mark.parametrize("dims,cin,cout", [((5, 13, 21), 64, 64), ((3, 9, 17), 32, 48), ((2, 8, 8), 128, 128),
                                           ((7, 20, 36), 64, 16), ((1, 4, 4), 64, 128)], ids=lambda v: str(v))
def test_convolution_outputs_stay_inside_their_tensor(dims, cin, cout):
    from scaffold_b200.ops import _lib, conv_kernels as ck
    d, h, w = dims
    torch.manual_seed(0)
    x = torch.randn(2, d, h, w, cin, device="cuda").to(torch.bfloat16)
    gy = torch.randn(2, d, h, w, cout, device="cuda").to(torch.bfloat16)
    wt = torch.randn(cout, cin, 3, 3, 3, device="cuda") * 0.05
    buf, y = _guarded((2, d, h, w, cout), torch.bfloat16)
    ck.conv_same([x], ck.pack_weight_fwd(wt), 3, [cout], out=[y])
    bufg, gx = _guarded((2, d, h, w, cin), torch.bfloat16)
    ck.conv_same([gy], ck.pack_weight_dgrad(wt), 3, [cin], out=[gx])
    bufw, dw = _guarded(tuple(wt.shape), torch.float32)
    ck.conv_wgrad(gy, [x], 3, dw)
    torch.cuda.synchronize()
    _lib.check_status()
    assert _intact(buf, y.numel()) and _intact(bufg, gx.numel()) and _intact(bufw, dw.numel())
    assert not bool((y == CANARY).any()) and torch.isfinite(dw).all()


@pytest.mark.parametrize("dims,c", [((5, 7, 9), 64), ((3, 3, 3), 256), ((16, 16, 16), 16)], ids=lambda v: str(v))
def test_groupnorm_outputs_stay_inside_their_tensor(dims, c):
    import ctypes as C
    from scaffold_b200.ops import _lib, gn_kernels as gk
    d, h, w = dims
    torch.manual_seed(1)
    x = torch.randn(2, d, h, w, c, device="cuda").to(torch.bfloat16)
    wt, b = torch.randn(c, device="cuda"), torch.randn(c, device="cuda")
    # the allocation-free entry point takes the output pointer from the caller: give it a guarded one
    buf, y = _guarded(tuple(x.shape), torch.bfloat16)
    fn = _lib.lib().sb_gn_forward_noalloc
    fn.argtypes = [C.c_void_p] * 6 + [C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p]
    fn.restype = C.c_int
    assert fn(x.data_ptr(), y.data_ptr(), wt.data_ptr(), b.data_ptr(), None, None, 2, d * h * w, c, 8, 1e-5, 1,
              torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    want, _, _ = gk.gn_forward(x, wt, b, 8, 1e-5, True)
    assert _intact(buf, y.numel()) and torch.equal(y, want)


def test_pool_and_transposed_convolution_outputs_stay_inside_their_tensor():
    from scaffold_b200.ops import _lib, conv_kernels as ck, pool_kernels as pk
    torch.manual_seed(2)
    x = torch.randn(1, 6, 10, 14, 64, device="cuda").to(torch.bfloat16)
    y = pk.maxpool2_fwd(x)
    gy = torch.randn_like(y)
    gx = pk.maxpool2_bwd(gy, x, y)
    torch.cuda.synchronize()
    assert gx.shape == x.shape and torch.isfinite(gx.float()).all()
    # odd extents: the last plane / row / column has no pooling window and must get a zero gradient
    xo = torch.randn(1, 5, 7, 9, 32, device="cuda").to(torch.bfloat16)
    yo = pk.maxpool2_fwd(xo)
    go = pk.maxpool2_bwd(torch.ones_like(yo), xo, yo)
    torch.cuda.synchronize()
    assert bool((go[:, 4] == 0).all()) and bool((go[:, :, 6] == 0).all()) and bool((go[:, :, :, 8] == 0).all())
    wt = torch.randn(64, 32, 2, 2, 2, device="cuda") * 0.1
    out = ck.convT_fwd(x, ck.pack_weight_convT_fwd(wt), 32, None)
    torch.cuda.synchronize()
    _lib.check_status()
    assert out.shape == (1, 12, 20, 28, 32) and torch.isfinite(out.float()).all()
