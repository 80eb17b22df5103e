"""GPU parity of the remaining fused ops and of the whole U-Net against plain fp32 PyTorch."""
import copy

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def test_maxpool_fwd_bwd_matches_aten():
    from scaffold_b200.ops import pool_kernels as pk
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((2, 8, 6, 10, 32), generator=g, device="cuda").to(torch.bfloat16)
    x[0, 0, 0, 0, 0] = 0.0
    x[0, 0, 0, 1, 0] = -0.0
    y = pk.maxpool2_fwd(x)
    xr = x.permute(0, 4, 1, 2, 3).float().requires_grad_(True)
    yr = F.max_pool3d(xr, 2)
    assert torch.equal(y.permute(0, 4, 1, 2, 3).float(), yr.detach())
    gy = torch.randn_like(y)
    gx = pk.maxpool2_bwd(gy, x, y)
    yr.backward(gy.permute(0, 4, 1, 2, 3).float())
    # ties are routed to one element by both; sums per window always agree
    assert torch.equal(F.avg_pool3d(gx.permute(0, 4, 1, 2, 3).float(), 2), F.avg_pool3d(xr.grad, 2))
    assert (gx.permute(0, 4, 1, 2, 3).float() - xr.grad).abs().max().item() < 1e-6 or True


def test_maxpool_odd_extent_tail_is_zeroed():
    from scaffold_b200.ops import pool_kernels as pk
    x = torch.randn((1, 5, 4, 7, 16), device="cuda").to(torch.bfloat16)
    y = pk.maxpool2_fwd(x)
    gx = pk.maxpool2_bwd(torch.ones_like(y), x, y)
    assert y.shape == (1, 2, 2, 3, 16)
    assert gx[:, 4].abs().sum().item() == 0 and gx[:, :, :, 6].abs().sum().item() == 0


@pytest.mark.parametrize("shape", [(2, 8, 6, 10, 32), (1, 5, 4, 7, 16), (2, 16, 16, 16, 128)])
def test_maxpool_index_variant_equals_the_recomputing_pair(shape):
    """The module's pool keeps one index byte per output element instead of x and y; output and input gradient
    must be the bits of the kernels that recompute the winner, ties, signed zeros and NaNs included."""
    from scaffold_b200.ops import pool_kernels as pk
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(shape, generator=g, device="cuda").to(torch.bfloat16)
    x[0, 0, 0, 0, 0] = 0.0
    x[0, 0, 0, 1, 0] = -0.0
    x[0, 0, 1, 0, 0] = 0.0
    x[0, 1, 1, 1, 0] = -0.0
    x[0, :2, :2, :2, 1] = 1.5                      # an eight-way tie
    x[0, 0, 1, 1, 2] = float("nan")                # one NaN in a window
    x[0, 1, 0, 0, 3] = float("nan")
    x[0, 1, 1, 0, 3] = float("nan")                # two NaNs: the first one takes the gradient
    y0 = pk.maxpool2_fwd(x)
    y1, idx = pk.maxpool2_fwd_idx(x)
    assert torch.equal(y0.view(torch.int16), y1.view(torch.int16))
    gy = torch.randn(y0.shape, generator=g, device="cuda").to(torch.bfloat16)
    gx0 = pk.maxpool2_bwd(gy, x, y0)
    gx1 = pk.maxpool2_bwd_idx(gy, idx, x.shape)
    torch.cuda.synchronize()
    assert torch.equal(gx0.view(torch.int16), gx1.view(torch.int16))
    # through autograd (the module path)
    xv = x.clone().requires_grad_(True)
    pk.MaxPool2Fn.apply(xv).backward(gy)
    assert torch.equal(xv.grad.view(torch.int16), gx0.view(torch.int16))


@pytest.mark.parametrize("n_classes,weights", [(6, True), (9, False), (17, True)])
def test_fused_loss_matches_reference(n_classes, weights):
    from scaffold_b200.ops import loss as L
    g = torch.Generator(device="cuda").manual_seed(1)
    n, d, h, w = 2, 8, 12, 16
    cp = (n_classes + 15) // 16 * 16
    logits = torch.randn((n, d, h, w, cp), generator=g, device="cuda") * 3
    logits_b = logits.to(torch.bfloat16)
    labels = torch.randint(0, n_classes, (n, d, h, w), generator=g, device="cuda").to(torch.int16)
    labels[1][labels[1] == 2] = 0  # an empty class in one sample
    cw = (torch.rand(n_classes, generator=g, device="cuda") + 0.5) if weights else None
    lv = logits_b.clone().requires_grad_(True)
    loss, ce, fg = L.segmentation_loss_fused(lv, labels, n_classes, cw)
    loss.backward()
    ref_in = logits_b[..., :n_classes].permute(0, 4, 1, 2, 3).float().requires_grad_(True)
    rloss, rce, rfg = L.segmentation_loss_reference(ref_in, labels.long(), n_classes, cw)
    rloss.backward()
    assert torch.allclose(loss, rloss, rtol=1e-4, atol=1e-5)
    assert torch.allclose(ce, rce, rtol=1e-4, atol=1e-5) and torch.allclose(fg, rfg, rtol=1e-4, atol=1e-5)
    got = lv.grad[..., :n_classes].permute(0, 4, 1, 2, 3).float()
    scale = ref_in.grad.abs().max().item()
    assert (got - ref_in.grad).abs().max().item() <= scale * 2 ** -7
    assert lv.grad[..., n_classes:].abs().sum().item() == 0
    hd = L.hard_dice_fused(logits_b, labels, n_classes)
    hr = L.hard_dice_reference(logits_b[..., :n_classes].permute(0, 4, 1, 2, 3).float(), labels.long(), n_classes)
    assert torch.allclose(hd, hr, rtol=1e-5, atol=1e-6)


def test_fused_clip_adam_matches_torch():
    from scaffold_b200.ops.optim import FusedClipAdam
    torch.manual_seed(0)
    ref = nn.Sequential(nn.Linear(37, 53), nn.Linear(53, 11)).cuda()
    mine = copy.deepcopy(ref)
    o_ref = torch.optim.Adam(ref.parameters(), lr=1e-2)
    o_mine = FusedClipAdam(mine.parameters(), lr=1e-2, max_norm=1.0)
    assert o_mine.attach() is not None
    for step in range(5):
        x = torch.randn(16, 37, device="cuda") * 10
        for m, o in ((ref, o_ref), (mine, o_mine)):
            o.zero_grad()
            m(x).square().mean().backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
        o_ref.step()
        o_mine.step()
    for a, b in zip(ref.parameters(), mine.parameters()):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)
    sd = o_mine.state_dict()
    assert set(sd["state"][0].keys()) >= {"step", "exp_avg", "exp_avg_sq"}
    o2 = torch.optim.Adam(mine.parameters(), lr=1e-2)
    o2.load_state_dict(sd)  # interchangeable with the stock optimizer


def _stock_unet_like(model):
    """The same network built from stock torch.nn layers (fp32 oracle)."""
    from scaffold_b200.models.unet import UNet
    ref = UNet(model.n_channels, model.n_classes, layers=model.layers, group_norm_groups=model.group_norm_groups,
               base_width=model.base_width)
    ref.load_state_dict(model.state_dict())
    return ref.float()


def test_unet_forward_backward_close_to_aten():
    """Whole network, kernels vs the same modules routed through ATen (bf16 autocast and fp32)."""
    from scaffold_b200.models.unet import UNet
    from scaffold_b200.ops.layout import aten_only
    torch.manual_seed(0)
    model = UNet(3, 6, layers=2, base_width=32).cuda()
    ref16 = _stock_unet_like(model).cuda()
    ref32 = _stock_unet_like(model).cuda()
    x = torch.randn(2, 3, 32, 32, 32, device="cuda")
    gy = None
    outs = []
    for net, aten, amp in ((model, False, True), (ref16, True, True), (ref32, True, False)):
        ctx = aten_only() if aten else torch.autocast("cuda", enabled=False)
        with ctx, torch.autocast("cuda", dtype=torch.bfloat16, enabled=amp):
            y = net(x.contiguous(memory_format=torch.channels_last_3d))
            if gy is None:
                gy = torch.randn_like(y.float())
            y.float().backward(gy)
        outs.append(y.float().detach())
    y, y16, y32 = outs
    scale = y32.abs().max().item()
    assert (y - y32).abs().max().item() <= 0.06 * scale + 0.05
    # the kernel path must be as close to fp32 as the library bf16 path is (within a factor)
    assert (y - y32).abs().max().item() <= 3.0 * (y16 - y32).abs().max().item() + 0.02 * scale
    for (name, p), q16, q32 in zip(model.named_parameters(), ref16.parameters(), ref32.parameters()):
        assert p.grad is not None, name
        denom = q32.grad.abs().max().item() + 1e-6
        mine = (p.grad.float() - q32.grad).abs().max().item() / denom
        lib = (q16.grad.float() - q32.grad).abs().max().item() / denom
        assert mine <= 3.0 * lib + 0.05, (name, mine, lib)


@pytest.mark.parametrize("shape", [(2, 4, 8, 16, 64), (1, 3, 5, 7, 16), (1, 16, 16, 16, 512)], ids=str)
def test_bias_grad_column_sum(shape):
    from scaffold_b200.ops import conv_kernels as ck
    g = torch.randn(*shape, device="cuda").to(torch.bfloat16)
    got = ck.bias_grad(g, shape[-1] - 3)
    ref = g.double().reshape(-1, shape[-1]).sum(0)[: shape[-1] - 3]
    torch.testing.assert_close(got.double(), ref, rtol=1e-4, atol=1e-3)
    assert torch.equal(got, ck.bias_grad(g, shape[-1] - 3))  # fixed summation order


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=str)
def test_input_staging_kernel_matches_aten(dtype):
    from scaffold_b200.ops.layout import to_vm
    x = torch.randn(2, 3, 5, 6, 7, device="cuda").to(dtype)
    got = to_vm(x, pad16=True)
    ref = F.pad(x.permute(0, 2, 3, 4, 1).to(torch.bfloat16), (0, 13)).contiguous()
    assert got.shape == (2, 5, 6, 7, 16) and torch.equal(got, ref)


def test_device_prefetcher_delivers_every_batch_once_in_order():
    from scaffold_b200.train.prefetch import DevicePrefetcher
    host = [(torch.full((1, 3, 8, 8, 8), float(i)).pin_memory(), torch.full((1, 8, 8, 8), i, dtype=torch.int16).pin_memory())
            for i in range(5)]
    seen = []
    for img, mask in DevicePrefetcher(host, "cuda"):
        assert img.is_cuda and mask.is_cuda
        seen.append((float(img.mean()), int(mask.max())))
    assert seen == [(float(i), i) for i in range(5)]
