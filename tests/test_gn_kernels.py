"""GPU parity of the channels-last GroupNorm(+ReLU) kernels against float64 PyTorch."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

CASES = [
    # N, C, G, D, H, W, relu
    (2, 64, 8, 8, 16, 16, True),
    (1, 128, 8, 4, 8, 8, True),
    (2, 16, 8, 4, 8, 8, True),
    (1, 32, 8, 5, 7, 9, False),
    (1, 1024, 8, 2, 4, 4, True),
    (1, 64, 8, 32, 32, 32, True),
]


def _ref(x, w, b, G, relu):
    y = F.group_norm(x, G, w, b, 1e-5)
    return F.relu(y) if relu else y


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(map(str, c)))
def test_gn_forward_backward(case):
    from scaffold_b200.ops import gn_kernels as gk
    n, c, G, d, h, w, relu = case
    g = torch.Generator(device="cuda").manual_seed(0)
    x = (torch.randn((n, c, d, h, w), generator=g, device="cuda") * 2 + 3).to(torch.bfloat16)
    wt = torch.randn(c, generator=g, device="cuda")
    bs = torch.randn(c, generator=g, device="cuda")
    dy = torch.randn((n, c, d, h, w), generator=g, device="cuda").to(torch.bfloat16)
    xv = x.permute(0, 2, 3, 4, 1).contiguous()
    dyv = dy.permute(0, 2, 3, 4, 1).contiguous()
    y, mean, rstd = gk.gn_forward(xv, wt, bs, G, 1e-5, relu)
    xd = x.double().requires_grad_(True)
    wd = wt.double().requires_grad_(True)
    bd = bs.double().requires_grad_(True)
    ref = _ref(xd, wd, bd, G, relu)
    got = y.permute(0, 4, 1, 2, 3).double()
    # bf16 output: half an ulp of the reference magnitude
    tol = ref.detach().abs().clamp_min(1.0) * 2 ** -8
    assert ((got - ref.detach()).abs() <= tol).all()
    xg = xd.detach().reshape(n, G, -1)
    assert torch.allclose(mean.double(), xg.mean(-1), atol=1e-4, rtol=1e-5)
    assert torch.allclose(rstd.double(), (xg.var(-1, unbiased=False) + 1e-5).rsqrt(), atol=1e-4, rtol=1e-4)
    ref.backward(dy.double())
    dx, dw, db = gk.gn_backward(dyv, xv, wt, bs, mean, rstd, G, 1e-5, relu)
    gdx = dx.permute(0, 4, 1, 2, 3).double()
    scale = xd.grad.abs().max().item()
    assert (gdx - xd.grad).abs().max().item() <= scale * 2 ** -7 + 1e-6
    assert torch.allclose(dw.double(), wd.grad, rtol=2e-3, atol=2e-3 * wd.grad.abs().max().item())
    assert torch.allclose(db.double(), bd.grad, rtol=2e-3, atol=2e-3 * bd.grad.abs().max().item())


def test_gn_large_mean_is_stable():
    """Shifted/Welford statistics: a large common offset must not destroy the variance."""
    from scaffold_b200.ops import gn_kernels as gk
    g = torch.Generator(device="cuda").manual_seed(1)
    x = (torch.randn((1, 64, 8, 16, 16), generator=g, device="cuda") + 200.0).to(torch.bfloat16)
    w = torch.ones(64, device="cuda")
    b = torch.zeros(64, device="cuda")
    xv = x.permute(0, 2, 3, 4, 1).contiguous()
    _, mean, rstd = gk.gn_forward(xv, w, b, 8, 1e-5, False)
    xg = x.double().reshape(1, 8, -1)
    assert torch.allclose(mean.double(), xg.mean(-1), rtol=1e-6)
    assert torch.allclose(rstd.double(), (xg.var(-1, unbiased=False) + 1e-5).rsqrt(), rtol=1e-3)


def test_gn_two_shards_equal_whole_volume():
    """Merging a neighbour's partials reproduces the unsharded statistics (emulated on one GPU)."""
    from scaffold_b200.ops import gn_kernels as gk
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn((1, 8, 16, 16, 64), generator=g, device="cuda").to(torch.bfloat16)
    w = torch.randn(64, generator=g, device="cuda")
    b = torch.randn(64, generator=g, device="cuda")
    whole, mean, rstd = gk.gn_forward(x, w, b, 8)
    halves = [x[:, :4].contiguous(), x[:, 4:].contiguous()]
    parts = [gk.gn_stats(hv, w, b, 8, 1e-5, True) for hv in halves]
    outs = []
    for i, hv in enumerate(halves):
        order = [parts[i].data_ptr(), parts[1 - i].data_ptr()]
        y, m, r = gk.gn_apply(hv, w, b, 8, 1e-5, True, order, shards=2)
        outs.append(y)
        assert torch.allclose(m, mean, rtol=1e-5, atol=1e-6)
        assert torch.allclose(r, rstd, rtol=1e-5)
    got = torch.cat(outs, 1).float()
    assert (got - whole.float()).abs().max().item() <= 2 ** -6
