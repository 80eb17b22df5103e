"""GPU parity of the two-SM pair convolution kernel (tcgen05 cta_group::2, csrc/conv_plane2.cu).

Same standard as tests/test_conv_kernels.py: operands from {-1, 0, 1}, so the kernel must match
float64 PyTorch bit for bit after the bf16 rounding. The cases cover both tile widths (BN 128 / 256),
several output-channel tiles, an odd number of spatial tiles (the second CTA of the last pair has no
tile), more pair-jobs than SM pairs (the persistent loop and the accumulator double buffer), two
concatenated sources, a bias and two destinations; the controls show that the call really ran on
the pair kernel and that a swapped weight half is caught.
"""
import pytest
import torch
import torch.nn.functional as F

from test_conv_kernels import ncdhw, ndhwc, tri

pytestmark = pytest.mark.gpu


def _ck():
    from scaffold_b200.ops import _lib, conv_kernels as ck
    return _lib, ck


PAIR_CASES = [
    # N, D, H, W, Cin(list), Cout
    (1, 5, 16, 16, [128], 256),      # 10 tiles, BN 256
    (1, 3, 8, 16, [64], 128),        # 3 tiles: odd, BN 128
    (1, 1, 8, 16, [64], 128),        # a single tile: not eligible, falls back
    (2, 4, 16, 32, [64, 64], 128),   # two sources
    (1, 6, 24, 40, [128], 512),      # ragged edges, two output-channel tiles of 256
    (2, 16, 32, 32, [64], 128),      # 256 tiles at depth 4: more pair-jobs than SM pairs
    (1, 16, 64, 64, [128], 256),     # 2048 tiles: many jobs per pair
    (1, 7, 16, 16, [192], 384),      # 384 = 3 x 128
]


@pytest.mark.parametrize("case", PAIR_CASES, ids=lambda c: "x".join(map(str, c[:4])) + f"_{c[4]}to{c[5]}")
def test_pair_conv_fwd_bitwise(case):
    _lib, ck = _ck()
    n, d, h, w, cins, cout = case
    g = torch.Generator(device="cuda").manual_seed(4321)
    xs = [tri((n, c, d, h, w), g) for c in cins]
    wt = tri((cout, sum(cins), 3, 3, 3), g, density=0.5)
    bias = tri((cout,), g)
    ref = F.conv3d(torch.cat(xs, 1).double(), wt.double(), bias.double(), padding=1).round()
    want = ref.to(torch.bfloat16).double()
    wpack = ck.pack_weight_fwd(wt)
    srcs = [ndhwc(x) for x in xs]
    before = _lib.lib().sb_launch_count()
    (y,) = ck.conv_same(srcs, wpack, 3, [cout], bias=bias.contiguous())
    torch.cuda.synchronize()
    _lib.check_status()
    assert _lib.lib().sb_launch_count() == before + 1
    got = ncdhw(y)
    assert torch.equal(got, want), f"max abs diff {(got - want).abs().max().item()}"
    # the single-CTA kernels give the same bits
    (y1,) = ck.conv_same(srcs, wpack, 3, [cout], bias=bias.contiguous(), force_plain=4)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(y, y1)


def test_pair_conv_dgrad_two_destinations_bitwise():
    _lib, ck = _ck()
    n, d, h, w, cin, cout = 1, 4, 16, 32, 128, 64
    g = torch.Generator(device="cuda").manual_seed(7)
    gy = tri((n, cout, d, h, w), g)
    wt = tri((cout, cin, 3, 3, 3), g, density=0.5)
    ref = F.conv_transpose3d(gy.double(), wt.double(), padding=1).round()
    wpack = ck.pack_weight_dgrad(wt)
    assert ck.pair_eligible(wpack.shape[1], wpack.shape[2], (d, h, w))
    g0, g1 = ck.conv_same([ndhwc(gy)], wpack, 3, [64, 64])
    torch.cuda.synchronize()
    _lib.check_status()
    got = torch.cat([ncdhw(g0), ncdhw(g1)], 1)
    assert torch.equal(got, ref.to(torch.bfloat16).double())


def test_pair_conv_detects_swapped_weight_halves():
    """Negative control: the two CTAs read different halves of the weight rows; exchanging the halves of the
    packed operand must change the result (the comparison above would catch a kernel that mixed them up)."""
    _lib, ck = _ck()
    g = torch.Generator(device="cuda").manual_seed(5)
    x = tri((1, 64, 4, 16, 16), g)
    wt = tri((128, 64, 3, 3, 3), g, density=0.5)
    wpack = ck.pack_weight_fwd(wt)
    swapped = torch.cat([wpack[:, 64:], wpack[:, :64]], 1).contiguous()
    (y,) = ck.conv_same([ndhwc(x)], wpack, 3, [128])
    (ys,) = ck.conv_same([ndhwc(x)], swapped, 3, [128])
    torch.cuda.synchronize()
    _lib.check_status()
    assert not torch.equal(y, ys)
    assert torch.equal(y[..., :64], ys[..., 64:]) and torch.equal(y[..., 64:], ys[..., :64])


def test_pair_switch_routes_to_single_cta_kernels(monkeypatch):
    _lib, ck = _ck()
    assert ck.pair_eligible(256, 128, (8, 16, 16))
    assert not ck.kd_eligible(256, 128, (8, 16, 16))
    monkeypatch.setattr(ck, "PAIR_CONV", False)
    assert not ck.pair_eligible(256, 128, (8, 16, 16))
    assert ck.kd_eligible(256, 128, (8, 16, 16))
