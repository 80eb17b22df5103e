"""GPU parity of the tcgen05 convolution kernels against float64 PyTorch.

Operands are drawn from {-1, 0, 1}: every product and partial sum is an exact
integer in fp32, so the kernels must match the float64 reference bit for bit
after the same bf16 rounding, whatever their accumulation order. A wrong tap,
a missing flip or a misplaced shift therefore cannot hide inside a tolerance;
the negative controls at the bottom show that the standard has teeth.
"""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _ck():
    from scaffold_b200.ops import _lib, conv_kernels as ck
    return _lib, ck


def tri(shape, gen, density=1.0, device="cuda"):
    t = torch.randint(-1, 2, shape, generator=gen, device=device).to(torch.float32)
    if density < 1.0:
        t = t * (torch.rand(shape, generator=gen, device=device) < density)
    return t


def ndhwc(x):  # NCDHW fp32 -> [N,D,H,W,C] bf16 contiguous
    return x.permute(0, 2, 3, 4, 1).contiguous().to(torch.bfloat16)


def ncdhw(y):  # [N,D,H,W,C] -> NCDHW fp64
    return y.permute(0, 4, 1, 2, 3).double()


def pad_c(x, c):  # pad channel dim (dim 1) of NCDHW with zeros
    if x.shape[1] == c:
        return x
    return F.pad(x, (0, 0, 0, 0, 0, 0, 0, c - x.shape[1]))


FWD_CASES = [
    # N, D, H, W, Cin(list), Cout, k, kernel mode (0 auto: kd-fused plane kernel for <= 64 output channels else
    # plane-walk, 1 plain, 2 w-shift, 3 hw-shift, 4 single-CTA plane-walk: no kd fusion, no pair kernel)
    (1, 4, 16, 32, [64], 64, 3, 4),
    (2, 7, 24, 48, [64], 64, 3, 4),
    (1, 2, 16, 16, [64, 64], 64, 3, 4),
    (1, 3, 12, 20, [32], 32, 3, 4),
    (1, 5, 16, 16, [128], 256, 3, 4),
    (2, 6, 16, 32, [64, 32], 192, 3, 0),
    (2, 8, 8, 8, [64], 128, 3, 0),       # 8 x 8 planes: whole-sample tiles, reduction split over channel blocks
    (1, 4, 8, 8, [256], 256, 3, 0),
    (3, 2, 8, 8, [48], 128, 3, 0),
    (1, 9, 16, 16, [32, 96], 48, 3, 0),
    (1, 1, 8, 16, [64], 64, 3, 0),
    (3, 6, 40, 40, [64], 16, 3, 0),
    (1, 4, 16, 32, [64], 64, 3, 0),
    (1, 4, 16, 32, [64], 64, 3, 1),
    (1, 4, 16, 32, [64], 64, 3, 2),
    (1, 4, 16, 32, [64], 64, 3, 3),
    (2, 7, 24, 48, [64], 64, 3, 0),
    (1, 5, 16, 16, [128], 256, 3, 0),
    (1, 2, 16, 16, [64, 64], 64, 3, 2),
    (2, 16, 64, 64, [64], 64, 3, 0),
    (2, 4, 8, 8, [128], 256, 3, 0),
    (1, 2, 16, 16, [64, 64], 64, 3, 0),
    (1, 2, 16, 16, [128, 64], 128, 3, 1),
    (1, 3, 12, 20, [64], 64, 3, 0),
    (1, 3, 12, 20, [32], 32, 3, 0),
    (1, 4, 16, 16, [3], 64, 3, 0),
    (2, 4, 4, 4, [64], 128, 3, 0),
    (1, 2, 16, 16, [64], 9, 1, 0),
    (1, 32, 32, 32, [64], 64, 3, 0),
    (1, 8, 8, 8, [512], 128, 3, 0),
    (2, 8, 16, 16, [9], 64, 1, 0),       # k = 1 from <= 16 channels (the head's backward-data shape)
    (2, 8, 16, 16, [9], 64, 1, 1),
    (1, 3, 5, 7, [16], 72, 1, 0),        # ragged voxel count, 80 padded outputs
]


@pytest.mark.parametrize("case", FWD_CASES, ids=lambda c: "x".join(map(str, c[:4])) + f"_{c[4]}to{c[5]}_k{c[6]}_m{c[7]}")
def test_conv_fwd_bitwise(case):
    _lib, ck = _ck()
    n, d, h, w, cins, cout, k, plain = case
    g = torch.Generator(device="cuda").manual_seed(1234)
    xs = [tri((n, c, d, h, w), g) for c in cins]
    wt = tri((cout, sum(cins), k, k, k), g, density=0.5)
    bias = tri((cout,), g) if k == 1 else None
    ref = F.conv3d(torch.cat(xs, 1).double(), wt.double(), bias.double() if bias is not None else None, padding=k // 2)
    ref = ref.round()  # exact integers; some float64 library algorithms leave 1e-14 noise
    srcs = [ndhwc(pad_c(x, ck.pad_channels(x.shape[1]))) for x in xs]
    wp_full = torch.zeros(cout, sum(s.shape[4] for s in srcs), k, k, k, device="cuda")
    o = 0
    oo = 0
    for x, s in zip(xs, srcs):
        wp_full[:, oo:oo + x.shape[1]] = wt[:, o:o + x.shape[1]]
        o += x.shape[1]
        oo += s.shape[4]
    wpack = ck.pack_weight_fwd(wp_full)
    cpad = ck.pad_channels(cout)
    bpad = None
    if bias is not None:
        bpad = torch.zeros(cpad, device="cuda")
        bpad[:cout] = bias
    (y,) = ck.conv_same(srcs, wpack, k, [cpad], bias=bpad, force_plain=plain, kd_fused=plain != 4)
    torch.cuda.synchronize()
    _lib.check_status()
    got = ncdhw(y)[:, :cout]
    want = ref.to(torch.bfloat16).double()
    assert torch.equal(got, want), f"max abs diff {(got - want).abs().max().item()}"


def test_conv_dgrad_two_destinations_bitwise():
    _lib, ck = _ck()
    n, d, h, w, cin, cout = 1, 4, 16, 16, 128, 64
    g = torch.Generator(device="cuda").manual_seed(7)
    gy = tri((n, cout, d, h, w), g)
    wt = tri((cout, cin, 3, 3, 3), g, density=0.5)
    ref = F.conv_transpose3d(gy.double(), wt.double(), padding=1).round()  # == dgrad of a same conv
    wpack = ck.pack_weight_dgrad(wt)
    g0, g1 = ck.conv_same([ndhwc(gy)], wpack, 3, [64, 64])
    torch.cuda.synchronize()
    _lib.check_status()
    got = torch.cat([ncdhw(g0), ncdhw(g1)], 1)
    assert torch.equal(got, ref.to(torch.bfloat16).double())


@pytest.mark.parametrize("shape", [(1, 4, 8, 16, 128, 64), (2, 2, 4, 4, 256, 128), (1, 8, 16, 16, 64, 32)],
                         ids=lambda s: "x".join(map(str, s)))
def test_convT_fwd_and_dgrad_bitwise(shape):
    _lib, ck = _ck()
    n, d, h, w, cin, cout = shape
    g = torch.Generator(device="cuda").manual_seed(11)
    x = tri((n, cin, d, h, w), g)
    wt = tri((cin, cout, 2, 2, 2), g, density=0.5)
    b = tri((cout,), g)
    ref = F.conv_transpose3d(x.double(), wt.double(), b.double(), stride=2).round()
    y = ck.convT_fwd(ndhwc(x), ck.pack_weight_convT_fwd(wt), cout, b.float())
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(ncdhw(y), ref.to(torch.bfloat16).double())
    gy = tri((n, cout, 2 * d, 2 * h, 2 * w), g)
    refg = F.conv3d(gy.double(), wt.double(), stride=2).round()  # dgrad of convT(k2,s2) is a stride-2 conv
    gx = ck.convT_dgrad(ndhwc(gy), ck.pack_weight_convT_dgrad(wt), cin)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(ncdhw(gx), refg.to(torch.bfloat16).double())


WGRAD_CASES = [
    # N, D, H, W, Cin(list), Cout, k, splits
    # splits: 0 automatic, k > 0 fixed; negative forces the generic kernel (-1 automatic, -(k+1) fixed k)
    (1, 4, 16, 32, [64], 64, 3, 0),
    (1, 4, 16, 32, [64], 64, 3, 3),
    (1, 4, 16, 32, [64], 64, 3, -1),
    (1, 4, 16, 32, [64], 64, 3, -4),
    (1, 2, 16, 16, [64, 64], 64, 3, -1),
    (1, 2, 16, 16, [128], 128, 3, -1),
    (2, 3, 16, 32, [32, 32], 32, 3, 0),
    (2, 5, 24, 40, [64], 128, 3, 2),
    (1, 2, 16, 16, [64, 64], 64, 3, 0),
    (1, 2, 16, 16, [64], 128, 3, 0),
    (1, 2, 16, 16, [128], 128, 3, 0),
    (1, 2, 16, 16, [128, 128], 128, 3, 0),
    (1, 2, 8, 16, [128], 64, 3, 0),
    (2, 4, 8, 8, [256], 256, 3, 0),
    (2, 4, 4, 4, [128], 128, 3, 0),
    (1, 3, 12, 20, [64], 64, 3, 0),
    (1, 4, 16, 16, [3], 64, 3, 0),
    (1, 2, 16, 16, [64], 9, 1, 0),
]


@pytest.mark.parametrize("case", WGRAD_CASES, ids=lambda c: "x".join(map(str, c[:4])) + f"_{c[4]}to{c[5]}_k{c[6]}_s{c[7]}")
def test_conv_wgrad_bitwise(case):
    _lib, ck = _ck()
    n, d, h, w, cins, cout, k, splits = case
    g = torch.Generator(device="cuda").manual_seed(99)
    xs = [tri((n, c, d, h, w), g, density=0.5) for c in cins]
    gy = tri((n, cout, d, h, w), g, density=0.5)
    xcat = torch.cat(xs, 1).double().requires_grad_(True)
    wt = torch.zeros(cout, sum(cins), k, k, k, device="cuda", dtype=torch.float64, requires_grad=True)
    F.conv3d(xcat, wt, padding=k // 2).backward(gy.double())
    ref = wt.grad.round()
    srcs = [ndhwc(pad_c(x, ck.pad_channels(x.shape[1]))) for x in xs]
    gyp = ndhwc(pad_c(gy, ck.pad_channels(cout)))
    dw = torch.full((cout, sum(cins), k, k, k), float("nan"), device="cuda")
    if len(cins) == 1:
        ck.conv_wgrad(gyp, srcs, k, dw, splits=splits)
    else:
        ck.conv_wgrad(gyp, srcs, k, dw, splits=splits)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(dw.double(), ref), f"max abs diff {(dw.double() - ref).abs().max().item()}"
    # deterministic: a second call is bitwise identical, and accumulate adds
    dw2 = torch.empty_like(dw)
    ck.conv_wgrad(gyp, srcs, k, dw2, splits=splits)
    ck.conv_wgrad(gyp, srcs, k, dw2, accumulate=True, splits=splits)
    torch.cuda.synchronize()
    assert torch.equal(dw2, 2 * dw)


@pytest.mark.parametrize("shape", [(1, 4, 8, 16, 128, 64), (2, 2, 4, 4, 256, 128)], ids=lambda s: "x".join(map(str, s)))
def test_convT_wgrad_bitwise(shape):
    _lib, ck = _ck()
    n, d, h, w, cin, cout = shape
    g = torch.Generator(device="cuda").manual_seed(5)
    x = tri((n, cin, d, h, w), g, density=0.5)
    gy = tri((n, cout, 2 * d, 2 * h, 2 * w), g, density=0.5)
    wt = torch.zeros(cin, cout, 2, 2, 2, device="cuda", dtype=torch.float64, requires_grad=True)
    F.conv_transpose3d(x.double(), wt, stride=2).backward(gy.double())
    dw = torch.full((cin, cout, 2, 2, 2), float("nan"), device="cuda")
    ck.conv_wgrad(ndhwc(gy), [ndhwc(x)], 2, dw)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(dw.double(), wt.grad.round())


def test_negative_control_unflipped_dgrad_differs():
    """Packing backward-data weights without the tap flip must be caught by the bitwise standard."""
    _lib, ck = _ck()
    g = torch.Generator(device="cuda").manual_seed(3)
    gy = tri((1, 64, 4, 16, 16), g)
    wt = tri((64, 64, 3, 3, 3), g, density=0.5)
    ref = F.conv_transpose3d(gy.double(), wt.double(), padding=1).round().to(torch.bfloat16).double()
    wrong = ck.pack_weight_fwd(wt.transpose(0, 1).contiguous())  # transposed but NOT flipped
    (gx,) = ck.conv_same([ndhwc(gy)], wrong, 3, [64])
    torch.cuda.synchronize()
    _lib.check_status()
    assert not torch.equal(ncdhw(gx), ref)


@pytest.mark.parametrize("dim,mode", [(0, 0), (1, 0), (2, 0), (0, 1), (2, 2)], ids=lambda v: str(v))
def test_halo_input_conv_fwd_dgrad_wgrad_bitwise(dim, mode):
    """A shard with a one-voxel halo on one dim: forward, backward-data and weight gradient against autograd."""
    _lib, ck = _ck()
    g = torch.Generator(device="cuda").manual_seed(21 + dim)
    cin, cout = 64, 64
    local = [4, 16, 32]
    in_dims = list(local)
    in_dims[dim] += 2
    x_h = tri((1, cin, *in_dims), g, density=0.5)
    wt = tri((cout, cin, 3, 3, 3), g, density=0.5)
    gy = tri((1, cout, *local), g, density=0.5)
    pad = [1, 1, 1]
    pad[dim] = 0
    xr = x_h.double().requires_grad_(True)
    wr = wt.double().requires_grad_(True)
    ref = F.conv3d(xr, wr, padding=tuple(pad))
    ref.backward(gy.double())
    off = [0, 0, 0]
    off[dim] = 1
    (y,) = ck.conv_same([ndhwc(x_h)], ck.pack_weight_fwd(wt), 3, [cout], force_plain=mode, out_dims=local, in_off=off)
    torch.cuda.synchronize(); _lib.check_status()
    assert torch.equal(ncdhw(y), ref.detach().round().to(torch.bfloat16).double())
    # backward-data grows the halo: output grid = halo'd extents, gy read at a negative offset
    (gx,) = ck.conv_same([ndhwc(gy)], ck.pack_weight_dgrad(wt), 3, [cin], force_plain=mode, out_dims=in_dims,
                         in_off=[-o for o in off])
    torch.cuda.synchronize(); _lib.check_status()
    assert torch.equal(ncdhw(gx), xr.grad.round().to(torch.bfloat16).double())
    dw = torch.full((cout, cin, 3, 3, 3), float("nan"), device="cuda")
    ck.conv_wgrad(ndhwc(gy), [ndhwc(x_h)], 3, dw, splits=0 if mode == 0 else -1, x_off=off)
    torch.cuda.synchronize(); _lib.check_status()
    assert torch.equal(dw.double(), wr.grad.round())


@pytest.mark.parametrize("shape", [(64, 64, [64], [64]), (48, 3, [16], [3]), (64, 160, [96, 64], [96, 64]),
                                   (130, 70, [80], [70])], ids=lambda s: f"{s[0]}x{s[1]}")
def test_fused_weight_pack_matches_torch_packs(shape):
    """The one-pass packing kernel against the ATen packers, all four layouts."""
    _lib, ck = _ck()
    co, ci, src_c, real_c = shape
    w = torch.randn(co, ci, 3, 3, 3, device="cuda")
    parts, o = [], 0
    for sc, rc in zip(src_c, real_c):
        parts.append(F.pad(w[:, o:o + rc], (0, 0, 0, 0, 0, 0, 0, sc - rc)))
        o += rc
    wp = torch.cat(parts, 1)
    ref_f, ref_d = ck.pack_weight_fwd(wp), ck.pack_weight_dgrad(wp)
    co_pad, k = ck.pad_channels(co), sum(src_c)
    want = {"fwd": torch.zeros(27, co_pad, k, dtype=torch.bfloat16, device="cuda"),
            "fwd_kd": torch.zeros(27, co_pad, k, dtype=torch.bfloat16, device="cuda"),
            "dgrad": torch.zeros(27, k, co_pad, dtype=torch.bfloat16, device="cuda"),
            "dgrad_kd": torch.zeros(27, k, co_pad, dtype=torch.bfloat16, device="cuda")}
    ck.pack_conv3(w, src_c, real_c, want)
    torch.cuda.synchronize()
    assert torch.equal(want["fwd"], ref_f)
    assert torch.equal(want["dgrad"], ref_d)
    assert torch.equal(want["fwd_kd"], ck.kd_order(ref_f))
    assert torch.equal(want["dgrad_kd"], ck.kd_order(ref_d))


def test_wgrad_two_narrow_sources_falls_back_to_their_concatenation():
    _lib, ck = _ck()
    g = torch.Generator(device="cuda").manual_seed(5)
    x0, x1 = tri((1, 16, 4, 16, 16), g), tri((1, 16, 4, 16, 16), g)
    gy = tri((1, 16, 4, 16, 16), g, density=0.3)
    xcat = torch.cat([x0, x1], 1).double().requires_grad_(False)
    w = torch.zeros(16, 32, 3, 3, 3, dtype=torch.float64, device="cuda", requires_grad=True)
    F.conv3d(xcat, w, padding=1).backward(gy.double())
    dw = torch.empty(16, 32, 3, 3, 3, device="cuda")
    ck.conv_wgrad(ndhwc(gy), [ndhwc(x0), ndhwc(x1)], 3, dw)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(dw.double(), w.grad.round())
