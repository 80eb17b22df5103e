"""More bitwise standards and their negative controls: transposed-convolution tap order, weight-gradient
slot order, real layer widths, the one-launch repack, gradients written straight into the flat buffer, and
activation checkpointing on the kernel path."""
import pytest
import torch
import torch.nn.functional as F

from test_conv_kernels import ncdhw, ndhwc, tri

pytestmark = pytest.mark.gpu


def _ck():
    from scaffold_b200.ops import _lib, conv_kernels as ck
    return _lib, ck


def test_negative_control_convT_with_permuted_taps_differs():
    """A transposed convolution whose (kd, kh, kw) taps are packed in another order must fail the bitwise check."""
    _lib, ck = _ck()
    g = torch.Generator(device="cuda").manual_seed(2)
    x = tri((1, 64, 4, 8, 16), g)
    wt = tri((64, 32, 2, 2, 2), g, density=0.7)
    ref = F.conv_transpose3d(x.double(), wt.double(), stride=2).round().to(torch.bfloat16).double()
    good = ck.convT_fwd(ndhwc(x), ck.pack_weight_convT_fwd(wt), 32, None)
    for perm in ((0, 1, 3, 2, 4), (0, 1, 4, 3, 2), (0, 1, 2, 4, 3)):  # swap kd/kh, kd/kw, kh/kw
        bad = ck.convT_fwd(ndhwc(x), ck.pack_weight_convT_fwd(wt.permute(*perm).contiguous()), 32, None)
        torch.cuda.synchronize()
        _lib.check_status()
        assert not torch.equal(ncdhw(bad), ref), perm
    assert torch.equal(ncdhw(good), ref)
    flipped = ck.convT_fwd(ndhwc(x), ck.pack_weight_convT_fwd(wt.flip(2, 3, 4)), 32, None)
    torch.cuda.synchronize()
    assert not torch.equal(ncdhw(flipped), ref)


def test_negative_control_wgrad_lands_in_the_right_tap_and_channel_slots():
    """A one-hot gradient and a one-hot input make exactly one (co, ci, tap) entry non-zero: its position is
    checked directly, and a transposed or tap-mirrored result would put it elsewhere."""
    _lib, ck = _ck()
    n, d, h, w, cin, cout = 1, 4, 16, 32, 64, 64
    for (co, ci, (dz, dy, dx)) in ((5, 40, (1, 0, -1)), (63, 0, (-1, 1, 1)), (17, 17, (0, 0, 0))):
        x = torch.zeros(n, cin, d, h, w, device="cuda")
        gy = torch.zeros(n, cout, d, h, w, device="cuda")
        vz, vy, vx = 2, 7, 13
        gy[0, co, vz, vy, vx] = 1.0
        x[0, ci, vz + dz, vy + dy, vx + dx] = 1.0   # y[v] reads x[v + tap - 1]: tap index = offset + 1
        dw = torch.full((cout, cin, 3, 3, 3), float("nan"), device="cuda")
        ck.conv_wgrad(ndhwc(gy), [ndhwc(x)], 3, dw)
        torch.cuda.synchronize()
        _lib.check_status()
        want = torch.zeros_like(dw)
        want[co, ci, dz + 1, dy + 1, dx + 1] = 1.0
        assert torch.equal(dw, want)
        assert not torch.equal(dw, want.flip(2, 3, 4)) or (dz, dy, dx) == (0, 0, 0)
        if co != ci:
            assert not torch.equal(dw, want.transpose(0, 1))


@pytest.mark.parametrize("cin,cout,dims", [(128, 64, (8, 64, 64)), (256, 128, (6, 32, 32)), (64, 128, (8, 32, 64)),
                                           (512, 256, (4, 16, 16))], ids=lambda v: str(v))
def test_real_layer_widths_forward_dgrad_wgrad_bitwise(cin, cout, dims):
    _lib, ck = _ck()
    g = torch.Generator(device="cuda").manual_seed(41)
    d, h, w = dims
    x = tri((1, cin, d, h, w), g, density=0.25)
    gy = tri((1, cout, d, h, w), g, density=0.25)
    wt = tri((cout, cin, 3, 3, 3), g, density=0.25)
    xr, wr = x.double().requires_grad_(True), wt.double().requires_grad_(True)
    ref = F.conv3d(xr, wr, padding=1)
    ref.backward(gy.double())
    (y,) = ck.conv_same([ndhwc(x)], ck.pack_weight_fwd(wt), 3, [cout])
    (gx,) = ck.conv_same([ndhwc(gy)], ck.pack_weight_dgrad(wt), 3, [cin])
    dw = torch.full_like(wt, float("nan"))
    ck.conv_wgrad(ndhwc(gy), [ndhwc(x)], 3, dw)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(ncdhw(y), ref.detach().round().to(torch.bfloat16).double())
    assert torch.equal(ncdhw(gx), xr.grad.round().to(torch.bfloat16).double())
    assert torch.equal(dw.double(), wr.grad.round())


def _tiny_model(width=32, layers=2, classes=5):
    from scaffold_b200.models.unet import UNet
    torch.manual_seed(0)
    return UNet(3, classes, layers=layers, base_width=width).cuda()


def test_one_launch_repack_and_direct_gradients_match_the_lazy_autograd_path():
    """Model ``a`` trains through FusedClipAdam (flat buffers: weight gradients are added straight into the flat
    buffer, every 3x3x3 pack is refreshed by ONE launch after the update); model ``b`` gets its gradients through
    autograd. Same kernels in the same order: the gradients are bitwise equal, and after the update the batched
    packs give the same logits as a fresh model that packs the same weights lazily, layer by layer."""
    from scaffold_b200.ops import _lib, loss as L
    from scaffold_b200.ops.optim import FusedClipAdam
    a, b = _tiny_model(), _tiny_model()
    b.load_state_dict(a.state_dict())
    opt_a = FusedClipAdam(a.parameters(), lr=1e-3, max_norm=1.0)
    opt_a.attach()
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.rand((2, 3, 32, 32, 32), generator=g, device="cuda")
    y = torch.randint(0, 5, (2, 32, 32, 32), generator=g, device="cuda", dtype=torch.int16)

    def fwd_bwd(model):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = model.forward_padded_logits(x)
        loss, _, _ = L.segmentation_loss_fused(logits, y, 5)
        loss.backward()
        return logits.detach()

    opt_a.zero_grad()
    fwd_bwd(a)
    fwd_bwd(b)
    torch.cuda.synchronize()
    _lib.check_status()
    for (name, pa), pb in zip(a.named_parameters(), b.parameters()):
        assert torch.equal(pa.grad, pb.grad), name
    opt_a.step()                     # update + the one-launch repack
    c = _tiny_model()
    c.load_state_dict(a.state_dict())
    n0 = _lib.launch_count()
    opt_a.zero_grad()
    la = fwd_bwd(a)
    n_a = _lib.launch_count() - n0
    n0 = _lib.launch_count()
    lc = fwd_bwd(c)
    n_c = _lib.launch_count() - n0
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(la, lc)
    assert n_a < n_c                 # no per-layer packing launches on the model whose packs were batched


def test_activation_checkpointing_on_the_kernel_path_gives_the_same_gradients():
    from scaffold_b200.ops import _lib, loss as L
    a, b = _tiny_model(), _tiny_model()
    b.load_state_dict(a.state_dict())
    b.use_checkpointing()
    g = torch.Generator(device="cuda").manual_seed(8)
    x = torch.rand((1, 3, 32, 32, 32), generator=g, device="cuda")
    y = torch.randint(0, 5, (1, 32, 32, 32), generator=g, device="cuda", dtype=torch.int16)
    grads = []
    for model in (a, b):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = model.forward_padded_logits(x)
        loss, _, _ = L.segmentation_loss_fused(logits, y, 5)
        loss.backward()
        grads.append([p.grad.clone() for p in model.parameters()])
    torch.cuda.synchronize()
    _lib.check_status()
    for ga, gb in zip(*grads):
        assert torch.equal(ga, gb)  # recomputation replays the same deterministic kernels


def test_kernel_selection_report_lists_every_layer():
    from scaffold_b200.ops.selection import format_selection, kernel_selection
    model = _tiny_model(width=64, layers=2)
    rows = kernel_selection(model, 2, (64, 64, 64))
    names = [r["layer"] for r in rows]
    assert "down_list.0.double_conv.0" in names and "up_list.2.conv" in names
    by = {r["layer"]: r for r in rows}
    assert by["down_list.0.double_conv.3"]["fwd"] == "conv_plane3"
    assert by["down_list.0.double_conv.0"]["dgrad"] == "-"
    assert by["up_list.0.up"]["fwd"].startswith("igemm")
    text = format_selection(rows, {"halo_exchange_effective": "none"})
    assert "weight-grad" in text and "halo_exchange_effective: none" in text


# the last five run the two-SM pair kernel (tile widths 128 and 256, groups of 16 to 128 channels, ragged planes)
@pytest.mark.parametrize("cin,cout,dims,groups", [(64, 64, (8, 24, 40), 8), (32, 128, (5, 16, 16), 8),
                                                  (64, 32, (4, 9, 17), 8), (64, 64, (2, 8, 16), 4),
                                                  (64, 128, (6, 16, 32), 8), (128, 256, (5, 16, 16), 8),
                                                  (64, 512, (4, 8, 16), 8), (64, 1024, (2, 8, 16), 8),
                                                  (64, 128, (5, 12, 20), 4)],
                         ids=lambda v: str(v))
def test_groupnorm_statistics_from_the_convolution_epilogue_match_the_statistics_pass(cin, cout, dims, groups):
    from scaffold_b200.ops import _lib, conv_kernels as ck, gn_kernels as gk
    torch.manual_seed(6)
    d, h, w = dims
    x = (torch.randn(2, d, h, w, cin, device="cuda") + 0.5).to(torch.bfloat16)
    wt = torch.randn(cout, cin, 3, 3, 3, device="cuda") * 0.1
    sink = []
    (y,) = ck.conv_same([x], ck.pack_weight_fwd(wt), 3, [cout], gn_groups=groups, gn_sink=sink)
    (y_plain,) = ck.conv_same([x], ck.pack_weight_fwd(wt), 3, [cout])
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(y, y_plain)                      # asking for statistics does not change the output
    assert len(sink) == 1
    part, splits, g = sink[0]
    fin = gk.gn_finalize(part, 2, groups, splits).view(2, groups, 3)
    wg, bg = torch.ones(cout, device="cuda"), torch.zeros(cout, device="cuda")
    ref = gk.gn_stats(y, wg, bg, groups, 1e-5, False).view(2, groups, 3)
    torch.cuda.synchronize()
    assert torch.equal(fin[..., 0], ref[..., 0])        # element counts
    assert torch.allclose(fin[..., 1], ref[..., 1], rtol=1e-4, atol=1e-5)
    assert torch.allclose(fin[..., 2], ref[..., 2], rtol=2e-4)
    # and through the modules: conv -> GroupNorm picks the partials up
    ya, _, _ = gk.gn_forward(y, wg, bg, groups, 1e-5, True, fin=fin.reshape(-1))
    yb, _, _ = gk.gn_forward(y, wg, bg, groups, 1e-5, True)
    assert (ya.float() - yb.float()).abs().max().item() <= 0.02


@pytest.mark.parametrize("swap,axis", [(1, 3), (2, 4)], ids=["kd_kh", "kd_kw"])
def test_tap_exchange_in_the_pack_and_weight_gradient_kernels_equals_a_transposed_weight(swap, axis):
    """A volume split along H or W is processed with that axis exchanged with depth; the kernels then pack the
    weight, and store its gradient, with the matching tap axes exchanged. Both must equal doing the exchange on
    the tensors with torch."""
    _lib, ck = _ck()
    g = torch.Generator(device="cuda").manual_seed(12)
    cin, cout = 64, 32
    wt = tri((cout, cin, 3, 3, 3), g, density=0.6)
    want = {n: torch.zeros((27, cout, cin) if n.startswith("fwd") else (27, cin, cout), dtype=torch.bfloat16,
                           device="cuda") for n in ("fwd", "fwd_kd", "dgrad", "dgrad_kd")}
    ck.pack_conv3(wt, [cin], [cin], want, tap_swap=swap)
    wt_t = wt.transpose(2, axis).contiguous()
    ref_f, ref_d = ck.pack_weight_fwd(wt_t), ck.pack_weight_dgrad(wt_t)
    torch.cuda.synchronize()
    assert torch.equal(want["fwd"], ref_f) and torch.equal(want["dgrad"], ref_d)
    assert torch.equal(want["fwd_kd"], ck.kd_order(ref_f)) and torch.equal(want["dgrad_kd"], ck.kd_order(ref_d))
    # weight gradient: computed in the kernels' tap order, stored in the parameter's
    x = tri((1, cin, 4, 16, 32), g, density=0.5)
    gy = tri((1, cout, 4, 16, 32), g, density=0.5)
    plain = torch.empty_like(wt)
    swapped = torch.full_like(wt, float("nan"))
    ck.conv_wgrad(ndhwc(gy), [ndhwc(x)], 3, plain)
    ck.conv_wgrad(ndhwc(gy), [ndhwc(x)], 3, swapped, tap_swap=swap)
    ck.conv_wgrad(ndhwc(gy), [ndhwc(x)], 3, swapped, tap_swap=swap, accumulate=True)
    generic = torch.empty_like(wt)
    ck.conv_wgrad(ndhwc(gy), [ndhwc(x)], 3, generic, tap_swap=swap, splits=-1)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(swapped, 2 * plain.transpose(2, axis)) and torch.equal(generic, plain.transpose(2, axis))
